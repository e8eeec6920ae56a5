"""Python mirror of the upstream pybind11 module ``pilot_ann.extension`` for the
GPU search stage (``extension/entry.cpp:65-86``): same function names, argument
order and error behaviour (``RuntimeError``), implemented as ctypes calls into
the C-ABI library.  Hot names: ``traverse_cuda``, ``routing_cuda``; plus the
entry points that have no upstream counterpart because upstream keeps its
tensors in CSR form (``pack_graph``, ``traverse_packed``, ``project``).

Tensors are checked exactly as ``CHECK_CUDA`` does (``extension/inc/common.h:
23-29``): CUDA device, rank, dtype, contiguity.  Work is enqueued on the
current torch CUDA stream of the tensors' device, like upstream
(``traverse_cuda.cu:284``); unlike upstream a device guard is applied.
"""
from __future__ import annotations

import threading

import torch

from . import _C

BEAM_WIDTH = 4


def _check_cuda(name: str, x: torch.Tensor, dim: int, dtype: torch.dtype) -> None:
    if not isinstance(x, torch.Tensor) or not x.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if x.dim() != dim:
        raise RuntimeError(f"{name} must be of dim {dim}")
    if x.dtype != dtype:
        raise RuntimeError(f"{name} must be type of {dtype}")
    if not x.is_contiguous():
        raise RuntimeError(f"{name} custom kernel requires contiguous tensor")


def _require(cond: bool, what: str) -> None:
    if not cond:
        raise RuntimeError(f"Expected {what} to be true, but got false.")


def _stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _traverse_checks(output_I, output_D, storage, query, initial_I, initial_D, n_neighbors):
    _check_cuda("storage", storage, 2, torch.float32)
    _check_cuda("query", query, 2, torch.float32)
    _check_cuda("initial_I", initial_I, 2, torch.int64)
    _check_cuda("initial_D", initial_D, 2, torch.float32)
    _check_cuda("output_I", output_I, 3, torch.int64)
    _check_cuda("output_D", output_D, 3, torch.float32)
    batch, d_model = query.shape
    _require(storage.size(-1) == d_model, "storage.size(-1) == d_model")
    _require(output_I.size(0) == batch, "output_I.size(0) == batch_size")
    _require(output_I.size(1) == BEAM_WIDTH, "output_I.size(1) == BEAM_WIDTH")
    _require(initial_I.size(0) == batch, "initial_I.size(0) == batch_size")
    _require(output_I.shape == output_D.shape, "output_I.sizes() == output_D.sizes()")
    _require(initial_I.shape == initial_D.shape, "initial_I.sizes() == initial_D.sizes()")
    _require(BEAM_WIDTH * n_neighbors <= 256, "BEAM_WIDTH * n_neighbors <= BUFFER_SIZE")
    _require(n_neighbors % 32 == 0, "n_neighbors % WARP_SIZE == 0")


# ---- packed form of a caller's CSR tensors, remembered between calls ---------
# ``traverse_cuda`` takes upstream's tensors as they are.  A caller that passes
# the SAME tensor objects again (upstream's layers and ``pipeline`` do: the
# sub-graph lives on the device for the life of the index) gets them packed once,
# on the second call, and searched in the packed layout from then on: identical
# results, ~20 % less time per call.  An entry is used only while the three
# tensor objects are alive and unmodified (torch's version counters); a graph
# that cannot be packed keeps the CSR path (the reason is kept in the entry).
# Packing allocates device memory and synchronises the stream once; it is never
# done while the current stream is being captured into a CUDA graph (the call
# then stays on the CSR path).  PILOTANN_B200_PACK_CACHE=0 turns this off.
_PACK_CACHE_SLOTS = 2
_pack_cache: dict = {}
_pack_lock = threading.Lock()


def _packed_for(indptr, indices, mapping, n_storage: int, n_neighbors: int):
    import os
    import weakref
    if os.environ.get("PILOTANN_B200_PACK_CACHE", "1") == "0":
        return None
    if torch.cuda.is_current_stream_capturing():
        capturing = True                 # no allocation, no synchronise under capture
    else:
        capturing = False
    key = (indptr.data_ptr(), indices.data_ptr(), mapping.data_ptr(), indptr.numel(),
           indices.numel(), n_storage, n_neighbors, indptr.device.index)
    stamp = (indptr._version, indices._version, mapping._version)
    with _pack_lock:
        for dead in [k for k, e in _pack_cache.items() if any(r() is None for r in e["refs"])]:
            del _pack_cache[dead]        # the caller's tensors are gone: free their packed form
        entry = _pack_cache.get(key)
        alive = entry is not None and all(r() is x for r, x in
                                          zip(entry["refs"], (indptr, indices, mapping)))
        if not alive or entry["stamp"] != stamp:
            while len(_pack_cache) >= _PACK_CACHE_SLOTS and key not in _pack_cache:
                _pack_cache.pop(next(iter(_pack_cache)))
            _pack_cache[key] = {"refs": tuple(weakref.ref(x) for x in (indptr, indices, mapping)),
                                "stamp": stamp, "packed": None, "usable": True, "why": None}
            return None                  # first sight of these tensors: search them as they are
        if entry["packed"] is None and entry["usable"] and not capturing:
            try:
                entry["packed"] = pack_graph(indptr, indices, mapping, n_storage, n_neighbors)
            except RuntimeError as exc:
                entry["usable"] = False  # e.g. a node with neighbours but no vector row
                entry["why"] = str(exc)
        return entry["packed"]


def traverse_cuda(output_I, output_D, indptr, indices, mapping, storage, query,
                  initial_I, initial_D, n_neighbors: int, stats=None) -> None:
    """``extension.traverse_cuda`` (``extension/traverse_cuda.cu:249-315``).  From the
    second call with the same graph tensors on, the search runs over their packed
    form (see ``_packed_for``); results are identical either way."""
    _check_cuda("indptr", indptr, 1, torch.int64)
    _check_cuda("indices", indices, 1, torch.int64)
    _check_cuda("mapping", mapping, 1, torch.int64)
    _traverse_checks(output_I, output_D, storage, query, initial_I, initial_D, n_neighbors)
    n_nodes = indptr.size(0) - 1
    _require(mapping.size(0) == n_nodes, "mapping.size(0) == n_nodes")
    if stats is not None:
        _check_cuda("stats", stats, 2, torch.int32)
    packed = _packed_for(indptr, indices, mapping, storage.size(0), n_neighbors)
    if packed is not None:  # same search, same results, over the packed form of these tensors
        traverse_packed(output_I, output_D, packed[0], packed[1], storage, query, initial_I,
                        initial_D, n_neighbors, stats=stats)
        return
    with torch.cuda.device(query.device):
        _C.check(_C.lib().pa_traverse_csr(
            output_I.data_ptr(), output_D.data_ptr(), indptr.data_ptr(), indices.data_ptr(),
            mapping.data_ptr(), storage.data_ptr(), query.data_ptr(), initial_I.data_ptr(),
            initial_D.data_ptr(), query.size(0), n_nodes, storage.size(0), query.size(1),
            n_neighbors, initial_I.size(1), output_I.size(2),
            0 if stats is None else stats.data_ptr(), _stream(query.device)))


def pack_graph(indptr, indices, mapping, n_storage: int, n_neighbors: int):
    """Packed device index from upstream's CSR tensors.  Returns
    ``(packed_nbr int32 [n_storage, n_neighbors, 4], row_of int32 [n_nodes])``:
    per neighbour slot the global id, the storage row and two words of
    precomputed bloom probes."""
    _check_cuda("indptr", indptr, 1, torch.int64)
    _check_cuda("indices", indices, 1, torch.int64)
    _check_cuda("mapping", mapping, 1, torch.int64)
    n_nodes = indptr.size(0) - 1
    _require(mapping.size(0) == n_nodes, "mapping.size(0) == n_nodes")
    dev = indptr.device
    packed = torch.empty(n_storage, n_neighbors, 4, dtype=torch.int32, device=dev)
    row_of = torch.empty(n_nodes, dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        _C.check(_C.lib().pa_pack_graph(
            packed.data_ptr(), row_of.data_ptr(), indptr.data_ptr(), indices.data_ptr(),
            mapping.data_ptr(), n_nodes, n_storage, n_neighbors, _stream(dev)))
    return packed, row_of


def traverse_packed(output_I, output_D, packed_nbr, row_of, storage, query, initial_I,
                    initial_D, n_neighbors: int, stats=None) -> None:
    """Same search as ``traverse_cuda`` over the packed index."""
    _check_cuda("packed_nbr", packed_nbr, 3, torch.int32)
    _check_cuda("row_of", row_of, 1, torch.int32)
    _traverse_checks(output_I, output_D, storage, query, initial_I, initial_D, n_neighbors)
    _require(packed_nbr.size(0) == storage.size(0), "packed_nbr.size(0) == n_storage")
    _require(packed_nbr.size(1) == n_neighbors, "packed_nbr.size(1) == n_neighbors")
    _require(packed_nbr.size(2) == 4, "packed_nbr.size(2) == 4")
    if stats is not None:
        _check_cuda("stats", stats, 2, torch.int32)
    with torch.cuda.device(query.device):
        _C.check(_C.lib().pa_traverse_packed(
            output_I.data_ptr(), output_D.data_ptr(), packed_nbr.data_ptr(), row_of.data_ptr(),
            storage.data_ptr(), query.data_ptr(), initial_I.data_ptr(), initial_D.data_ptr(),
            query.size(0), row_of.size(0), storage.size(0), query.size(1), n_neighbors,
            initial_I.size(1), output_I.size(2), 0 if stats is None else stats.data_ptr(),
            _stream(query.device)))


def routing_cuda(query, route_vectors, entry_nodes, entry_vectors, with_ids: bool = False):
    """``extension.routing_cuda`` (``extension/routing_cuda.cu:70-113``): returns
    ``[router int64 [B], distances f32 [B, n_leaves]]`` (+ the gathered leaf ids
    ``[B, n_leaves]`` when ``with_ids``)."""
    _check_cuda("query", query, 2, torch.float32)
    _check_cuda("route_vectors", route_vectors, 2, torch.float32)
    _check_cuda("entry_vectors", entry_vectors, 3, torch.float32)
    _check_cuda("entry_nodes", entry_nodes, 2, torch.int64)
    batch, d_model = query.shape
    n_leaves = entry_nodes.size(-1)
    n_routers = route_vectors.size(0)
    _require(route_vectors.size(-1) == d_model, "route_vectors.size(-1) == d_model")
    _require(entry_vectors.size(-1) == d_model, "entry_vectors.size(-1) == d_model")
    _require(entry_vectors.size(0) == n_routers, "entry_vectors.size(0) == n_routers")
    _require(entry_vectors.size(1) == n_leaves, "entry_vectors.size(1) == n_leaves")
    _require(n_leaves % 32 == 0, "n_leaves % BLOCK_SIZE == 0")
    router = torch.empty(batch, dtype=torch.int64, device=query.device)
    distances = torch.empty(batch, n_leaves, dtype=torch.float32, device=query.device)
    ids = torch.empty(batch, n_leaves, dtype=torch.int64, device=query.device) if with_ids else None
    # scratch for the tensor-core router scores (torch's caching allocator: no
    # device synchronisation)
    ws = torch.empty(int(_C.lib().pa_route_workspace_floats(batch, n_routers)),
                     dtype=torch.float32, device=query.device)
    with torch.cuda.device(query.device):
        _C.check(_C.lib().pa_route_ws(
            router.data_ptr(), distances.data_ptr(), 0 if ids is None else ids.data_ptr(),
            query.data_ptr(), route_vectors.data_ptr(), entry_nodes.data_ptr(),
            entry_vectors.data_ptr(), batch, d_model, n_routers, n_leaves, ws.data_ptr(),
            _stream(query.device)))
    return [router, distances, ids] if with_ids else [router, distances]


def entry_distances(query, entry_vectors):
    """Squared distances from every query to one shared list of entry vectors
    ``[n, d]`` (the 'random' entry method, ``pilot_ann/layers/entry.py:70-77``)."""
    _check_cuda("query", query, 2, torch.float32)
    _check_cuda("entry_vectors", entry_vectors, 2, torch.float32)
    batch, d_model = query.shape
    n = entry_vectors.size(0)
    _require(entry_vectors.size(1) == d_model, "entry_vectors.size(-1) == d_model")
    _require(n % 32 == 0, "n_entries % 32 == 0")
    distances = torch.empty(batch, n, dtype=torch.float32, device=query.device)
    with torch.cuda.device(query.device):
        _C.check(_C.lib().pa_route(0, distances.data_ptr(), 0, query.data_ptr(), 0, 0,
                                   entry_vectors.data_ptr(), batch, d_model, 1, n,
                                   _stream(query.device)))
    return distances


def project(query, VT, d_out: int | None = None):
    """``query @ VT.T`` on the GPU (``pilot_ann/layers/staged.py:198`` runs it on
    the CPU); first ``d_out`` output columns."""
    _check_cuda("query", query, 2, torch.float32)
    _check_cuda("VT", VT, 2, torch.float32)
    _require(VT.size(1) == query.size(1), "VT.size(1) == d_model")
    d_out = VT.size(0) if d_out is None else d_out
    _require(0 <= d_out <= VT.size(0), "d_out <= VT.size(0)")
    out = torch.empty(query.size(0), d_out, dtype=torch.float32, device=query.device)
    with torch.cuda.device(query.device):
        _C.check(_C.lib().pa_project(out.data_ptr(), query.data_ptr(), VT.data_ptr(),
                                     query.size(0), query.size(1), d_out, d_out,
                                     _stream(query.device)))
    return out


NOALLOC_MAX_BATCH = 1024
NOALLOC_MAX_LEAVES = 64


def search_reduced_noalloc(output_I, output_D, packed_nbr, row_of, storage, query,
                           route_vectors, entry_nodes, entry_vectors, n_neighbors: int) -> None:
    """Routing + traversal through ``pa_search_reduced_noalloc``: for callers that
    must not allocate device memory (the GPU was handed to a private pool, or the
    thread cannot afford the device-wide stall of an allocation).  This wrapper
    creates no tensor either; everything, outputs included, comes from the
    caller.  Limits: ``batch <= NOALLOC_MAX_BATCH``, ``n_leaves <=
    NOALLOC_MAX_LEAVES``.  Calls on one device must not overlap."""
    _check_cuda("packed_nbr", packed_nbr, 3, torch.int32)
    _check_cuda("row_of", row_of, 1, torch.int32)
    _check_cuda("storage", storage, 2, torch.float32)
    _check_cuda("query", query, 2, torch.float32)
    _check_cuda("output_I", output_I, 3, torch.int64)
    _check_cuda("output_D", output_D, 3, torch.float32)
    _check_cuda("entry_nodes", entry_nodes, 2 if route_vectors is not None else 1, torch.int64)
    _check_cuda("entry_vectors", entry_vectors, 3 if route_vectors is not None else 2,
                torch.float32)
    if route_vectors is not None:
        _check_cuda("route_vectors", route_vectors, 2, torch.float32)
    batch, d = query.shape
    n_leaves = entry_nodes.size(-1)
    _require(packed_nbr.size(0) == storage.size(0), "packed_nbr.size(0) == n_storage")
    _require(packed_nbr.size(1) == n_neighbors, "packed_nbr.size(1) == n_neighbors")
    _require(packed_nbr.size(2) == 4, "packed_nbr.size(2) == 4")
    _require(storage.size(1) == d, "storage.size(-1) == d_principle")
    _require(entry_vectors.size(-1) == d, "entry_vectors.size(-1) == d_principle")
    _require(entry_vectors.size(-2) == n_leaves, "entry_vectors.size(-2) == n_leaves")
    if route_vectors is not None:
        n_routers = route_vectors.size(0)
        _require(route_vectors.size(1) == d, "route_vectors.size(-1) == d_principle")
        _require(entry_nodes.size(0) == n_routers, "entry_nodes.size(0) == n_routers")
        _require(entry_vectors.size(0) == n_routers, "entry_vectors.size(0) == n_routers")
    _require(output_I.shape == output_D.shape and output_I.size(0) == batch
             and output_I.size(1) == BEAM_WIDTH, "output shape [batch, 4, ef]")
    with torch.cuda.device(query.device):
        _C.check(_C.lib().pa_search_reduced_noalloc(
            output_I.data_ptr(), output_D.data_ptr(), packed_nbr.data_ptr(), row_of.data_ptr(),
            storage.data_ptr(), query.data_ptr(),
            0 if route_vectors is None else route_vectors.data_ptr(), entry_nodes.data_ptr(),
            entry_vectors.data_ptr(), batch, row_of.size(0), storage.size(0), d, n_neighbors,
            0 if route_vectors is None else route_vectors.size(0), entry_nodes.size(-1),
            output_I.size(2), _stream(query.device)))


def pack_fullgraph(indptr, indices, degree: int):
    """The full graph as ``int32 [n_nodes, degree]`` rows, ``-1`` padded, from
    upstream's CSR tensors (``fullgraph.indptr / indices``): what stage 3 of the
    refinement walks.  A row ends at its first negative id; repeated ids are
    dropped."""
    _check_cuda("indptr", indptr, 1, torch.int64)
    _check_cuda("indices", indices, 1, torch.int64)
    n_nodes = indptr.size(0) - 1
    out = torch.empty(n_nodes, degree, dtype=torch.int32, device=indptr.device)
    with torch.cuda.device(indptr.device):
        _C.check(_C.lib().pa_pack_fullgraph(out.data_ptr(), indptr.data_ptr(), indices.data_ptr(),
                                            n_nodes, degree, _stream(indptr.device)))
    return out


class VisitedPool:
    """``pa_visited_pool``: the device counterpart of upstream's ``BitmaskPool``
    (``extension/inc/bitmask.hpp:51-76``) -- ``n_slots`` epoch-marked visited arrays
    over ``n_nodes`` nodes, one per resident CTA of the refinement kernel."""

    def __init__(self, n_nodes: int, n_slots: int, device=None):
        import ctypes
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None \
            else torch.device(device)
        self.n_nodes, self.n_slots = n_nodes, n_slots
        handle = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            _C.check(_C.lib().pa_visited_pool_create(ctypes.byref(handle), n_nodes, n_slots))
        self._h = handle

    @staticmethod
    def bytes_for(n_nodes: int, n_slots: int) -> int:
        return int(_C.lib().pa_visited_pool_bytes(n_nodes, n_slots))

    def close(self) -> None:
        if getattr(self, "_h", None) and _C is not None and _C.lib is not None:
            _C.lib().pa_visited_pool_destroy(self._h)   # (module globals are gone at exit)
            self._h = None

    __del__ = close


def cpu_heap_size_for(ef_search: int) -> int:
    """Heap capacity of upstream's CPU search for ``ef_search``
    (``extension/traverse_cpu.cpp:228-254``)."""
    return int(_C.lib().pa_cpu_heap_size_for(ef_search))


def refine_wave(d_model: int, device=None) -> int:
    """Queries the refinement kernel works on at once on ``device``: the number of
    visited slots (``VisitedPool``) worth allocating for one stream."""
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    return sms * int(_C.lib().pa_refine_ctas_per_sm(d_model))


def refine(cand_I, cand_D, query, storage, packed_nbr, row_of, full_nbr, pool: VisitedPool,
           ef_search: int, d_principle: int, k: int | None = None, stats=None, out=None):
    """``traverse_refine`` (``extension/traverse_cpu.cpp:261-369``) on the GPU over
    the candidate handoff ``cand_I / cand_D [B, 4, ef]`` (or ``[B, 4 * ef]``) in
    device memory.  ``k=None`` runs the sub-graph stage alone and returns the
    rewritten handoff rows ``[B, 4 * ef]`` (what upstream leaves in its buffer for
    the full-graph stage); otherwise both stages run and ``(topk_I [B, k],
    topk_D [B, k])`` comes back, ascending."""
    B = query.size(0)
    cand_I = cand_I.reshape(B, -1)
    cand_D = cand_D.reshape(B, -1)
    _check_cuda("cand_I", cand_I, 2, torch.int64)
    _check_cuda("cand_D", cand_D, 2, torch.float32)
    _check_cuda("query", query, 2, torch.float32)
    _check_cuda("storage", storage, 2, torch.float32)
    _check_cuda("packed_nbr", packed_nbr, 3, torch.int32)
    _check_cuda("row_of", row_of, 1, torch.int32)
    _require(cand_I.shape == cand_D.shape, "cand_I.sizes() == cand_D.sizes()")
    _require(storage.size(1) == query.size(1), "storage.size(-1) == d_model")
    _require(row_of.size(0) == storage.size(0), "row_of.size(0) == n_storage")
    _require(packed_nbr.size(2) == 4, "packed_nbr.size(2) == 4")
    _require(pool.n_nodes >= storage.size(0), "pool.n_nodes >= n_storage")
    stages = 2 if k is None else 3
    if stages == 3:
        _check_cuda("full_nbr", full_nbr, 2, torch.int32)
        _require(full_nbr.size(0) == storage.size(0), "full_nbr.size(0) == n_storage")
    if stats is not None:
        _check_cuda("stats", stats, 2, torch.int32)
    n_out = cand_I.size(1) if k is None else k
    if out is None:
        out_I = torch.empty(B, n_out, dtype=torch.int64, device=query.device)
        out_D = torch.empty(B, n_out, dtype=torch.float32, device=query.device)
    else:
        out_I, out_D = out
        _check_cuda("out_I", out_I, 2, torch.int64)
        _check_cuda("out_D", out_D, 2, torch.float32)
        _require(out_I.shape == (B, n_out) and out_D.shape == (B, n_out), "out shape [B, n_out]")
    with torch.cuda.device(query.device):
        _C.check(_C.lib().pa_refine(
            out_I.data_ptr(), out_D.data_ptr(), cand_I.data_ptr(), cand_D.data_ptr(),
            query.data_ptr(), storage.data_ptr(), packed_nbr.data_ptr(), row_of.data_ptr(),
            packed_nbr.size(1), 0 if full_nbr is None else full_nbr.data_ptr(),
            0 if full_nbr is None else full_nbr.size(1), B, storage.size(0), query.size(1),
            d_principle, cand_I.size(1), ef_search, 0 if k is None else k, stages, pool._h,
            0 if stats is None else stats.data_ptr(), _stream(query.device)))
    return out_I, out_D


# ---- pipeline -------------------------------------------------------------------
# Who consumes the candidate handoff in `pipeline` (and in IndexStaged.search):
#   "gpu"      the refinement kernel of this package (default): candidates never
#              leave the device, the call returns the final top-k;
#   callable   a CPU consumer with the signature of upstream's
#              extension.traverse_refine (extension/entry.cpp:39-46), e.g. that very
#              function: it refines chunk i-2 while the GPU traverses chunk i-1, as
#              upstream's pipeline does;
#   None       no consumer: pipeline raises.
_refine_consumer = "gpu"


def set_refine(consumer) -> None:
    """Chooses the consumer of the candidate handoff: ``"gpu"``, a callable with
    upstream's ``traverse_refine`` signature, or ``None``."""
    global _refine_consumer
    if consumer is not None and consumer != "gpu" and not callable(consumer):
        raise RuntimeError('set_refine: pass "gpu", a callable, or None')
    _refine_consumer = consumer


def get_refine():
    return _refine_consumer


_pipe_lock = threading.Lock()
_pipe_buffers: dict = {}      # (device, chunk, ef, k) -> persistent stream / buffer set
_resident: dict = {}          # device-resident forms of a caller's CPU index tensors
_N_PIPE_STREAMS = 2           # N_PREFETCH of upstream (extension/pipeline_cpu.cpp:5)


def _pipe_set(dev: torch.device, chunk: int, ef: int, k: int):
    """Streams, device handoff buffers and pinned host buffers of `pipeline`, made
    once per shape and kept (upstream allocates them in every call,
    ``extension/pipeline_cpu.cpp:78-96``)."""
    key = (dev.index if dev.index is not None else torch.cuda.current_device(), chunk, ef, k)
    with _pipe_lock:
        bs = _pipe_buffers.get(key)
        if bs is None:
            while len(_pipe_buffers) >= 4:
                _pipe_buffers.pop(next(iter(_pipe_buffers)))
            n = _N_PIPE_STREAMS
            bs = {
                "streams": [torch.cuda.Stream(device=dev) for _ in range(n)],
                "dev_I": [torch.empty(chunk, 4, ef, dtype=torch.int64, device=dev) for _ in range(n)],
                "dev_D": [torch.empty(chunk, 4, ef, dtype=torch.float32, device=dev) for _ in range(n)],
                "host_I": [torch.empty(chunk, 4 * ef, dtype=torch.int64, pin_memory=True)
                           for _ in range(n)],
                "host_D": [torch.empty(chunk, 4 * ef, dtype=torch.float32, pin_memory=True)
                           for _ in range(n)],
                "top_I": [torch.empty(chunk, k, dtype=torch.int64, device=dev) for _ in range(n)],
                "top_D": [torch.empty(chunk, k, dtype=torch.float32, device=dev) for _ in range(n)],
            }
            _pipe_buffers[key] = bs
    return bs


def _resident_for(graph, storage, subgraph_cuda, n_storage_sub: int, n_neighbors: int,
                  chunk: int, dev: torch.device):
    """Device-resident forms of the tensors upstream's CPU refinement reads: the
    full-dimension vectors, the full graph packed to int32 rows, the packed
    sub-graph, and one visited pool per side stream.  Built the first time a set of
    tensor objects is seen (an upload of the whole vector table: the counterpart of
    ``IndexStaged.to``), kept while they live."""
    import weakref
    tensors = (graph[0], graph[1], storage, *subgraph_cuda)
    key = tuple(t.data_ptr() for t in tensors) + (dev.index, n_neighbors)
    stamp = tuple(t._version for t in tensors)
    with _pipe_lock:
        for dead in [kk for kk, e in _resident.items() if any(r() is None for r in e["refs"])]:
            del _resident[dead]
        entry = _resident.get(key)
        if entry is not None and entry["stamp"] == stamp and \
                all(r() is t for r, t in zip(entry["refs"], tensors)) and entry["chunk"] >= chunk:
            return entry
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("pipeline: the first call with a new index uploads it; make that "
                               "call outside stream capture")
        while len(_resident) >= 2:
            _resident.pop(next(iter(_resident)))
        degree = int((graph[0][1:] - graph[0][:-1]).max().item()) if graph[0].numel() > 1 else 1
        degree = max(32, (degree + 31) // 32 * 32)
        packed = pack_graph(subgraph_cuda[0], subgraph_cuda[1], subgraph_cuda[2], n_storage_sub,
                            n_neighbors)
        full_nbr = pack_fullgraph(graph[0].to(dev), graph[1].to(dev), degree)
        entry = {"refs": tuple(weakref.ref(t) for t in tensors), "stamp": stamp, "chunk": chunk,
                 "packed": packed, "full_nbr": full_nbr,
                 "storage": storage.to(dev).contiguous(),
                 "pools": [VisitedPool(storage.size(0), min(chunk, refine_wave(storage.size(1), dev)), dev)
                           for _ in range(_N_PIPE_STREAMS)]}
        _resident[key] = entry
        return entry


def pipeline(graph, subgraph, subgraph_cuda, storage, storage_cuda, query, query_cuda,
             initial_I, initial_D, n_neighbors: int, ef_search: int, d_principle: int, k: int,
             chunk_size: int):
    """``extension.pipeline`` with upstream's positional order
    (``extension/entry.cpp:48-56``, ``extension/pipeline_cpu.cpp:32-145``); returns
    ``[topk_I int64 [B, k], topk_D f32 [B, k]]`` on the CPU, ascending.  Who turns
    the candidates into the top-k is set by :func:`set_refine`.  With a CPU
    consumer, chunks of ``chunk_size`` queries alternate over two side streams and
    the consumer refines one chunk while the GPU works on the next; with the GPU
    consumer ``chunk_size`` is only checked (upstream requires it to divide the
    batch) and the batch goes through in large pieces."""
    if len(graph) != 2 or len(subgraph) != 2 or len(subgraph_cuda) != 3:
        raise RuntimeError("graph / subgraph / subgraph_cuda must hold 2 / 2 / 3 tensors")
    _check_cuda("query_cuda", query_cuda, 2, torch.float32)
    _check_cuda("storage_cuda", storage_cuda, 2, torch.float32)
    batch = query.size(0)
    _require(chunk_size > 0 and batch % chunk_size == 0, "batch_size % chunk_size == 0")
    _require(query_cuda.size(0) == batch, "query_cuda.size(0) == batch_size")
    consumer = _refine_consumer
    if consumer is None:
        raise RuntimeError("pipeline: no consumer for the candidate handoff; call "
                           "pilotann_b200.set_refine(\"gpu\") or set_refine(<traverse_refine>)")
    dev = query_cuda.device
    n_streams = _N_PIPE_STREAMS
    topk_I = torch.empty(batch, k, dtype=torch.int64, pin_memory=True)
    topk_D = torch.empty(batch, k, dtype=torch.float32, pin_memory=True)
    n_chunks = batch // chunk_size
    ready = torch.cuda.Event()
    ready.record(torch.cuda.current_stream(dev))      # the inputs were produced on this stream

    def traverse(slot, lo, hi):
        traverse_cuda(bs["dev_I"][slot], bs["dev_D"][slot], subgraph_cuda[0], subgraph_cuda[1],
                      subgraph_cuda[2], storage_cuda, query_cuda[lo:hi], initial_I[lo:hi],
                      initial_D[lo:hi], n_neighbors)

    if consumer == "gpu":
        # nothing on the host to overlap with: chunking would only shorten the launches
        # (a 128-query launch lasts almost as long as a 1024-query one), so the whole
        # batch goes through in pieces of up to 4096 queries on the two side streams
        piece = batch
        while piece > 4096 and piece % 2 == 0:
            piece //= 2
        bs = _pipe_set(dev, piece, ef_search, k)
        streams = bs["streams"]
        res = _resident_for(graph, storage, subgraph_cuda, storage_cuda.size(0), n_neighbors,
                            piece, dev)
        q_full = query.to(dev, non_blocking=True)
        ready.record(torch.cuda.current_stream(dev))
        for i in range(batch // piece):
            slot = i % n_streams
            lo, hi = i * piece, (i + 1) * piece
            with torch.cuda.stream(streams[slot]):
                streams[slot].wait_event(ready)
                traverse_cuda(bs["dev_I"][slot], bs["dev_D"][slot], subgraph_cuda[0],
                              subgraph_cuda[1], subgraph_cuda[2], storage_cuda, query_cuda[lo:hi],
                              initial_I[lo:hi], initial_D[lo:hi], n_neighbors)
                refine(bs["dev_I"][slot], bs["dev_D"][slot], q_full[lo:hi], res["storage"],
                       res["packed"][0], res["packed"][1], res["full_nbr"], res["pools"][slot],
                       ef_search, d_principle, k=k, out=(bs["top_I"][slot], bs["top_D"][slot]))
                topk_I[lo:hi].copy_(bs["top_I"][slot], non_blocking=True)
                topk_D[lo:hi].copy_(bs["top_D"][slot], non_blocking=True)
        for s_ in streams:
            s_.synchronize()
        del q_full
        return [topk_I, topk_D]

    # a CPU consumer: chunk i is launched, then chunk i - n_streams (long finished on
    # the GPU) is refined on the host while the GPU works on the chunks in between
    bs = _pipe_set(dev, chunk_size, ef_search, k)
    streams = bs["streams"]
    for i in range(n_chunks + n_streams):
        slot = i % n_streams
        if i >= n_streams:
            streams[slot].synchronize()
            lo = (i - n_streams) * chunk_size
            hi = lo + chunk_size
            consumer(topk_I[lo:hi], topk_D[lo:hi], bs["host_I"][slot], bs["host_D"][slot],
                     bs["host_I"][slot], bs["host_D"][slot], subgraph, graph, storage,
                     query[lo:hi], ef_search, d_principle)
        if i < n_chunks:
            lo, hi = i * chunk_size, (i + 1) * chunk_size
            with torch.cuda.stream(streams[slot]):
                streams[slot].wait_event(ready)
                traverse(slot, lo, hi)
                bs["host_I"][slot].copy_(bs["dev_I"][slot].view(chunk_size, -1), non_blocking=True)
                bs["host_D"][slot].copy_(bs["dev_D"][slot].view(chunk_size, -1), non_blocking=True)
    return [topk_I, topk_D]


def launch_count() -> int:
    return int(_C.lib().pa_launch_count())
