"""Build-time and evaluation helpers; same names as ``pilot_ann/utils/__init__.py``."""
from .svd import svd
from .recall import recall
from .graphs import graph_init, subgraph_init, graph_sampling, build_graph
from .router import router_init
from .synthetic import (Workload, WORKLOADS, make_storage, make_queries, ground_truth,
                        fuzz_workload)
