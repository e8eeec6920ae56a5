"""ctypes loader for the C-ABI library (``include/pilotann_b200.h``).

There is no fallback: if the library has not been built, importing a compute
entry point raises.  Build it with ``python -m pilotann_b200.build`` (or
``__graft_entry__.build()``).
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_int32, c_int64, c_void_p, c_char_p, POINTER, Structure
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "_lib" / "libpilotann_b200.so"

PA_OK = 0
PA_ERR_ARG, PA_ERR_CUDA, PA_ERR_UNPACKABLE, PA_ERR_STATE = -1, -2, -3, -4

#: every symbol ``include/pilotann_b200.h`` declares
SYMBOLS = (
    "pa_version", "pa_last_error", "pa_heap_size_for", "pa_traverse_csr", "pa_pack_graph",
    "pa_traverse_packed", "pa_route", "pa_project", "pa_stage_create", "pa_stage_destroy",
    "pa_stage_search", "pa_stage_search_device", "pa_stage_synchronize", "pa_stage_stream",
    "pa_launch_count", "pa_search_reduced_noalloc", "pa_device_status", "pa_route_ws", "pa_route_workspace_floats",
    "pa_selftest_bounded_wait", "pa_visited_pool_bytes", "pa_visited_pool_create",
    "pa_visited_pool_destroy", "pa_visited_pool_slots", "pa_cpu_heap_size_for", "pa_refine_ctas_per_sm",
    "pa_pack_fullgraph", "pa_refine", "pa_stage_attach_refine", "pa_stage_search_ex",
    "pa_stage_search_device_ex", "pa_stage_slot_rows", "pa_stage_submit", "pa_stage_wait",
)

PA_OUT_HANDOFF, PA_OUT_STAGE2, PA_OUT_TOPK = 0, 1, 2


class RefineIndex(Structure):
    """``pa_refine_index``"""
    _fields_ = [("storage_full", c_void_p), ("full_nbr", c_void_p), ("full_degree", c_int)]



class StageIndex(Structure):
    """``pa_stage_index``"""
    _fields_ = [
        ("packed_nbr", c_void_p), ("row_of", c_void_p), ("storage", c_void_p),
        ("VT", c_void_p), ("route_vectors", c_void_p), ("entry_nodes", c_void_p),
        ("entry_vectors", c_void_p), ("n_nodes", c_int64), ("n_storage", c_int64),
        ("d_model", c_int), ("d_principle", c_int), ("n_neighbors", c_int),
        ("n_routers", c_int), ("n_leaves", c_int),
    ]


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.is_file():
        raise ImportError(
            f"{LIB_PATH} is missing: the CUDA library has not been built "
            "(run `python -m pilotann_b200.build`); there is no CPU fallback")
    L = ctypes.CDLL(str(LIB_PATH))
    P = c_void_p
    L.pa_version.restype = c_int
    L.pa_last_error.restype = c_char_p
    L.pa_heap_size_for.argtypes = [c_int]
    L.pa_traverse_csr.argtypes = [P, P, P, P, P, P, P, P, P, c_int64, c_int64, c_int64,
                                  c_int, c_int, c_int, c_int, P, P]
    L.pa_pack_graph.argtypes = [P, P, P, P, P, c_int64, c_int64, c_int, P]
    L.pa_traverse_packed.argtypes = [P, P, P, P, P, P, P, P, c_int64, c_int64, c_int64,
                                     c_int, c_int, c_int, c_int, P, P]
    L.pa_route.argtypes = [P, P, P, P, P, P, P, c_int64, c_int, c_int, c_int, P]
    L.pa_route_ws.argtypes = [P, P, P, P, P, P, P, c_int64, c_int, c_int, c_int, P, P]
    L.pa_route_ws.restype = c_int
    L.pa_route_workspace_floats.argtypes = [c_int64, c_int]
    L.pa_route_workspace_floats.restype = c_int64
    L.pa_project.argtypes = [P, P, P, c_int64, c_int, c_int, c_int64, P]
    L.pa_stage_create.argtypes = [POINTER(P), POINTER(StageIndex), c_int64, c_int, c_int]
    L.pa_stage_destroy.argtypes = [P]
    L.pa_stage_destroy.restype = None
    L.pa_stage_search.argtypes = [P, P, P, P, P, c_int64, c_int, c_int64]
    L.pa_stage_search_device.argtypes = [P, P, P, P, c_int64, c_int, P]
    L.pa_stage_synchronize.argtypes = [P]
    L.pa_stage_stream.argtypes = [P]
    L.pa_stage_stream.restype = P
    L.pa_launch_count.restype = c_int64
    L.pa_visited_pool_bytes.argtypes = [c_int64, c_int]
    L.pa_visited_pool_bytes.restype = c_int64
    L.pa_visited_pool_create.argtypes = [POINTER(P), c_int64, c_int]
    L.pa_visited_pool_create.restype = c_int
    L.pa_visited_pool_destroy.argtypes = [P]
    L.pa_visited_pool_destroy.restype = None
    L.pa_visited_pool_slots.argtypes = [P]
    L.pa_visited_pool_slots.restype = c_int
    L.pa_cpu_heap_size_for.argtypes = [c_int]
    L.pa_cpu_heap_size_for.restype = c_int
    L.pa_refine_ctas_per_sm.argtypes = [c_int]
    L.pa_refine_ctas_per_sm.restype = c_int
    L.pa_pack_fullgraph.argtypes = [P, P, P, c_int64, c_int, P]
    L.pa_pack_fullgraph.restype = c_int
    L.pa_refine.argtypes = [P, P, P, P, P, P, P, P, c_int, P, c_int, c_int64, c_int64, c_int,
                            c_int, c_int, c_int, c_int, c_int, P, P, P]
    L.pa_refine.restype = c_int
    L.pa_stage_attach_refine.argtypes = [P, POINTER(RefineIndex), c_int]
    L.pa_stage_attach_refine.restype = c_int
    L.pa_stage_search_ex.argtypes = [P, P, P, P, P, c_int64, c_int, c_int, c_int, c_int64]
    L.pa_stage_search_ex.restype = c_int
    L.pa_stage_search_device_ex.argtypes = [P, P, P, P, c_int64, c_int, c_int, c_int, P, P]
    L.pa_stage_search_device_ex.restype = c_int
    L.pa_stage_slot_rows.argtypes = [P]
    L.pa_stage_slot_rows.restype = c_int64
    L.pa_stage_submit.argtypes = [P, c_int, P, c_int64, c_int, c_int, c_int, c_int]
    L.pa_stage_submit.restype = c_int
    L.pa_stage_wait.argtypes = [P, c_int, POINTER(P), POINTER(P), POINTER(P), POINTER(c_int64)]
    L.pa_stage_wait.restype = c_int
    L.pa_selftest_bounded_wait.argtypes = [P]
    L.pa_selftest_bounded_wait.restype = c_int
    L.pa_device_status.argtypes = [c_int]
    L.pa_device_status.restype = c_int
    L.pa_search_reduced_noalloc.argtypes = [P, P, P, P, P, P, P, P, P, c_int64, c_int64, c_int64,
                                            c_int, c_int, c_int, c_int, c_int, P]
    L.pa_search_reduced_noalloc.restype = c_int
    for name in ("pa_traverse_csr", "pa_pack_graph", "pa_traverse_packed", "pa_route",
                 "pa_project", "pa_stage_create", "pa_stage_search", "pa_stage_search_device",
                 "pa_stage_synchronize", "pa_heap_size_for"):
        getattr(L, name).restype = c_int
    _lib = L
    return L


def check(rc: int) -> None:
    """Translate a status code the way upstream's TORCH_CHECK / CUDA_CHECH do
    (``extension/inc/common.h:15-41``): a RuntimeError carrying the message."""
    if rc != PA_OK:
        msg = lib().pa_last_error().decode(errors="replace")
        raise RuntimeError(f"pilotann_b200: {msg} (code {rc})")
