"""Python face of the CPU oracle (``oracle/pilot_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by the smoke check and by the
CPU-baseline leg of ``bench.py``; never by the package.  All functions take and
return CPU torch tensors (contiguous, the dtypes of the upstream extension:
int64 ids, float32 values).
"""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "_build" / "libpilot_oracle.so"
_lib = None


def build(force: bool = False) -> Path:
    """Compile the C restatement with gcc (a second or two)."""
    src = HERE / "pilot_oracle.c"
    if force or not LIB_PATH.is_file() or LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(HERE), "-B" if force else "-s"], check=True,
                       stdout=subprocess.DEVNULL)
    return LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.is_file():
            build()
        L = ctypes.CDLL(str(LIB_PATH))
        L.po_fnv1a_32.restype = ctypes.c_uint32
        L.po_fnv1a_32.argtypes = [ctypes.c_uint32, ctypes.c_uint32]
        L.po_reduced_distance.restype = ctypes.c_float
        L.po_heap_size_for.restype = ctypes.c_int
        L.po_heap_pushpop.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
                                      ctypes.c_float, ctypes.c_int64]
        L.po_heap_replace.argtypes = L.po_heap_pushpop.argtypes
        L.po_warp_distance.restype = ctypes.c_float
        L.po_warp_distance.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
                                       ctypes.c_int]
        L.po_cpu_heap_size_for.restype = ctypes.c_int
        _lib = L
    return _lib


def _p(t: torch.Tensor | None):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _chk(t: torch.Tensor, dtype, dim=None):
    assert t.device.type == "cpu" and t.dtype == dtype and t.is_contiguous(), (t.dtype, t.device)
    if dim is not None:
        assert t.dim() == dim
    return t


def fnv1a_32(x: int, offset: int) -> int:
    return int(lib().po_fnv1a_32(x & 0xFFFFFFFF, offset & 0xFFFFFFFF))


def bloom_positions(node: int) -> list[int]:
    out = (ctypes.c_uint32 * 4)()
    lib().po_bloom_positions(ctypes.c_int64(node), out)
    return list(out)


def heap_pop(keys: torch.Tensor, values: torch.Tensor):
    _chk(keys, torch.float32, 1), _chk(values, torch.int64, 1)
    k, v = ctypes.c_float(), ctypes.c_int64()
    lib().po_heap_pop(_p(keys), _p(values), ctypes.c_int(keys.numel()),
                      ctypes.byref(k), ctypes.byref(v))
    return k.value, v.value


def heap_replace(keys, values, key: float, value: int):
    _chk(keys, torch.float32, 1), _chk(values, torch.int64, 1)
    lib().po_heap_replace(_p(keys), _p(values), keys.numel(), key, value)


def heap_pushpop(keys, values, key: float, value: int):
    _chk(keys, torch.float32, 1), _chk(values, torch.int64, 1)
    lib().po_heap_pushpop(_p(keys), _p(values), keys.numel(), key, value)


def reduced_distance(row: torch.Tensor, query: torch.Tensor) -> float:
    _chk(row, torch.float32, 1), _chk(query, torch.float32, 1)
    return float(lib().po_reduced_distance(_p(row), _p(query), ctypes.c_int(row.numel())))


def heap_size_for(ef: int) -> int:
    return int(lib().po_heap_size_for(ctypes.c_int(ef)))


def traverse(indptr, indices, mapping, storage, query, initial_I, initial_D,
             n_neighbors: int, ef_search: int, with_stats: bool = False):
    """Restated ``traverse_cuda``: returns (output_I [B,4,ef], output_D [B,4,ef])
    and, when asked, stats int32 [B,4] = rounds, expansions E, evaluations C,
    bloom bits set."""
    _chk(indptr, torch.int64, 1), _chk(indices, torch.int64, 1), _chk(mapping, torch.int64, 1)
    _chk(storage, torch.float32, 2), _chk(query, torch.float32, 2)
    _chk(initial_I, torch.int64, 2), _chk(initial_D, torch.float32, 2)
    B, d = query.shape
    assert storage.size(1) == d and mapping.numel() == indptr.numel() - 1
    out_I = torch.empty(B, 4, ef_search, dtype=torch.int64)
    out_D = torch.empty(B, 4, ef_search, dtype=torch.float32)
    stats = torch.zeros(B, 4, dtype=torch.int32) if with_stats else None
    rc = lib().po_traverse(_p(out_I), _p(out_D), _p(indptr), _p(indices), _p(mapping),
                           _p(storage), _p(query), _p(initial_I), _p(initial_D),
                           ctypes.c_int64(B), ctypes.c_int(d), ctypes.c_int(n_neighbors),
                           ctypes.c_int(initial_I.size(1)), ctypes.c_int(ef_search),
                           _p(stats))
    if rc != 0:
        raise RuntimeError("oracle: arguments rejected (as the upstream launcher would)")
    return (out_I, out_D, stats) if with_stats else (out_I, out_D)


def route(query, route_vectors, entry_nodes, entry_vectors):
    """Restated ``routing_cuda`` + the id gather of ``IndexEntry.search``:
    returns (router [B], leaf_D [B,n_leaves], leaf_I [B,n_leaves])."""
    _chk(query, torch.float32, 2), _chk(route_vectors, torch.float32, 2)
    _chk(entry_nodes, torch.int64, 2), _chk(entry_vectors, torch.float32, 3)
    B, d = query.shape
    n_r, n_l = entry_nodes.shape
    router = torch.empty(B, dtype=torch.int64)
    leaf_D = torch.empty(B, n_l, dtype=torch.float32)
    leaf_I = torch.empty(B, n_l, dtype=torch.int64)
    rc = lib().po_route(_p(router), _p(leaf_D), _p(leaf_I), _p(query), _p(route_vectors),
                        _p(entry_nodes), _p(entry_vectors), ctypes.c_int64(B),
                        ctypes.c_int(d), ctypes.c_int(n_r), ctypes.c_int(n_l))
    if rc != 0:
        raise RuntimeError("oracle: n_leaves must be a multiple of 32")
    return router, leaf_D, leaf_I


def project(query, VT, d_out: int | None = None):
    """Restated ``query @ VT.T`` (first ``d_out`` output columns)."""
    _chk(query, torch.float32, 2), _chk(VT, torch.float32, 2)
    B, d = query.shape
    assert VT.size(1) == d
    d_out = VT.size(0) if d_out is None else d_out
    out = torch.empty(B, d_out, dtype=torch.float32)
    lib().po_project(_p(out), _p(query), _p(VT), ctypes.c_int64(B), ctypes.c_int(d),
                     ctypes.c_int(d_out))
    return out


def search_cpu(initial_I, initial_D, indptr, indices, storage, query, k: int, ef_search: int):
    """Restated ``traverse_cpu`` (full-graph CPU search)."""
    _chk(initial_I, torch.int64, 2), _chk(initial_D, torch.float32, 2)
    _chk(indptr, torch.int64, 1), _chk(indices, torch.int64, 1)
    _chk(storage, torch.float32, 2), _chk(query, torch.float32, 2)
    B, d = query.shape
    out_I = torch.empty(B, k, dtype=torch.int64)
    out_D = torch.empty(B, k, dtype=torch.float32)
    rc = lib().po_search_cpu(_p(out_I), _p(out_D), _p(initial_I), _p(initial_D), _p(indptr),
                             _p(indices), _p(storage), _p(query), ctypes.c_int64(B),
                             ctypes.c_int64(storage.size(0)), ctypes.c_int(d),
                             ctypes.c_int(initial_I.size(1)), ctypes.c_int(k),
                             ctypes.c_int(ef_search))
    if rc != 0:
        raise RuntimeError("oracle: ef_search not supported")
    return out_I, out_D


def refine(buffer_I, buffer_D, subgraph, fullgraph, storage, query, k: int, ef_search: int,
           d_principle: int):
    """Restated ``traverse_refine``; ``buffer_*`` [B,4*ef] is overwritten in place
    exactly as upstream does with the handoff."""
    _chk(buffer_I, torch.int64, 2), _chk(buffer_D, torch.float32, 2)
    _chk(storage, torch.float32, 2), _chk(query, torch.float32, 2)
    for g in (*subgraph, *fullgraph):
        _chk(g, torch.int64, 1)
    B, d = query.shape
    out_I = torch.empty(B, k, dtype=torch.int64)
    out_D = torch.empty(B, k, dtype=torch.float32)
    rc = lib().po_refine(_p(out_I), _p(out_D), _p(buffer_I), _p(buffer_D), _p(subgraph[0]),
                         _p(subgraph[1]), _p(fullgraph[0]), _p(fullgraph[1]), _p(storage),
                         _p(query), ctypes.c_int64(B), ctypes.c_int64(storage.size(0)),
                         ctypes.c_int(d), ctypes.c_int(d_principle),
                         ctypes.c_int(buffer_I.size(1)), ctypes.c_int(k),
                         ctypes.c_int(ef_search))
    if rc != 0:
        raise RuntimeError("oracle: ef_search not supported")
    return out_I, out_D


def warp_distance(query: torch.Tensor, row: torch.Tensor, offset: int = 0) -> float:
    """Squared distance over dims [offset, d) in the summation order of the GPU
    refinement kernel (32 lanes x float4 stripes, butterfly reduction)."""
    _chk(row, torch.float32, 1), _chk(query, torch.float32, 1)
    return float(lib().po_warp_distance(_p(query), _p(row), row.numel(), offset))


def cpu_heap_size_for(ef: int) -> int:
    """Heap capacity of the CPU consumer (``traverse_cpu.cpp:228-254``)."""
    return int(lib().po_cpu_heap_size_for(ctypes.c_int(ef)))


def refine_ex(buffer_I, buffer_D, subgraph, fullgraph, storage, query, k: int, ef_search: int,
              d_principle: int, gpu_order: bool = True, stages: int = 3,
              with_stats: bool = False):
    """``traverse_refine`` restated with a choice of summation order
    (``gpu_order``: the refinement kernel's, else upstream's AVX2 one) and of
    stages (2: sub-graph stage only, the buffer is rewritten in place and no top-k
    is produced; 3: both).  Returns ``(out_I, out_D[, stats int32 [B,4]])``."""
    _chk(buffer_I, torch.int64, 2), _chk(buffer_D, torch.float32, 2)
    _chk(storage, torch.float32, 2), _chk(query, torch.float32, 2)
    for g in (*subgraph, *fullgraph):
        _chk(g, torch.int64, 1)
    B, d = query.shape
    out_I = torch.full((B, k), -1, dtype=torch.int64)
    out_D = torch.zeros(B, k, dtype=torch.float32)
    stats = torch.zeros(B, 4, dtype=torch.int32) if with_stats else None
    rc = lib().po_refine_ex(_p(out_I), _p(out_D), _p(buffer_I), _p(buffer_D), _p(subgraph[0]),
                            _p(subgraph[1]), _p(fullgraph[0]), _p(fullgraph[1]), _p(storage),
                            _p(query), ctypes.c_int64(B), ctypes.c_int64(storage.size(0)),
                            ctypes.c_int(d), ctypes.c_int(d_principle),
                            ctypes.c_int(buffer_I.size(1)), ctypes.c_int(k),
                            ctypes.c_int(ef_search), ctypes.c_int(1 if gpu_order else 0),
                            ctypes.c_int(stages), _p(stats))
    if rc != 0:
        raise RuntimeError("oracle: ef_search not supported")
    return (out_I, out_D, stats) if with_stats else (out_I, out_D)
