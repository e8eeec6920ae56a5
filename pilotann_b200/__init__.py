"""pilotann_b200 -- B200 (sm_100a) implementation of PilotANN's GPU search stage
behind the ``pilot_ann`` Python surface: ``kernels`` (op wrappers), ``layers``
(IndexEntry / IndexStaged), ``extension`` (the module the ops bind to) and
``utils`` (build-time helpers).  The compute lives in a C-ABI CUDA library
(``include/pilotann_b200.h``); there is no CPU fallback."""
from . import utils, extension, kernels, layers, stage, sharding  # noqa: F401
from .stage import SearchStage  # noqa: F401
from .extension import set_refine, get_refine  # noqa: F401

__version__ = "0.1.0"
