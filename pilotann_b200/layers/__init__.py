from .entry import IndexEntry
from .staged import IndexStaged, GraphModule
