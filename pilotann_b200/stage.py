"""``SearchStage``: the per-device stage object of the C ABI (``pa_stage_*``),
i.e. the GPU half of upstream ``pipeline`` (``extension/pipeline_cpu.cpp:32-145``)
with its streams and buffers created once instead of per call."""
from __future__ import annotations

import ctypes

import torch

from . import _C


class SearchStage:
    def __init__(self, *, packed_nbr, row_of, storage, VT, route_vectors, entry_nodes,
                 entry_vectors, n_neighbors: int, d_model: int, max_batch: int,
                 max_ef: int = 256, n_streams: int = 2):
        dev = storage.device
        assert dev.type == "cuda", "the search stage lives on a CUDA device"
        tensors = dict(packed_nbr=packed_nbr, row_of=row_of, storage=storage, VT=VT,
                       route_vectors=route_vectors, entry_nodes=entry_nodes,
                       entry_vectors=entry_vectors)
        for name, t in tensors.items():
            if t is None:
                continue
            if t.device != dev or not t.is_contiguous():
                raise RuntimeError(f"{name} must be contiguous on {dev}")
        if packed_nbr.dtype != torch.int32 or row_of.dtype != torch.int32:
            raise RuntimeError("packed index must be int32")
        if packed_nbr.dim() != 3 or packed_nbr.size(2) != 4:
            raise RuntimeError("packed_nbr must be [n_storage, n_neighbors, 4] (extension.pack_graph)")
        if entry_nodes.dtype != torch.int64:
            raise RuntimeError("entry_nodes must be int64")
        for name in ("storage", "VT", "route_vectors", "entry_vectors"):
            if tensors[name] is not None and tensors[name].dtype != torch.float32:
                raise RuntimeError(f"{name} must be float32")
        self._keep = tensors                       # the stage borrows these pointers
        self.device = dev
        self.d_model = d_model
        self.d_principle = storage.size(1)
        self.n_leaves = entry_nodes.size(-1)
        self.max_batch, self.max_ef = max_batch, max_ef
        ix = _C.StageIndex()
        ptr = lambda t: 0 if t is None else t.data_ptr()
        ix.packed_nbr, ix.row_of, ix.storage = ptr(packed_nbr), ptr(row_of), ptr(storage)
        ix.VT, ix.route_vectors = ptr(VT), ptr(route_vectors)
        ix.entry_nodes, ix.entry_vectors = ptr(entry_nodes), ptr(entry_vectors)
        ix.n_nodes, ix.n_storage = row_of.size(0), storage.size(0)
        ix.d_model, ix.d_principle, ix.n_neighbors = d_model, self.d_principle, n_neighbors
        ix.n_routers = 0 if route_vectors is None else route_vectors.size(0)
        ix.n_leaves = self.n_leaves
        handle = ctypes.c_void_p()
        with torch.cuda.device(dev):
            _C.check(_C.lib().pa_stage_create(ctypes.byref(handle), ctypes.byref(ix),
                                              max_batch, max_ef, n_streams))
        self._h = handle

    def close(self) -> None:
        if getattr(self, "_h", None):
            _C.lib().pa_stage_destroy(self._h)
            self._h = None

    __del__ = close

    def search_host(self, query: torch.Tensor, ef_search: int, chunk: int = 0,
                    out_I=None, out_D=None, rotated=None):
        """Host buffers in, host buffers out (the call a user of the stage makes).
        ``query`` [B, d_model] float32 CPU (pinned for speed).  Returns
        ``(handoff_I [B, 4*ef] int64, handoff_D [B, 4*ef] float32, rotated)``,
        pinned CPU tensors."""
        if query.device.type != "cpu" or query.dtype != torch.float32 or not query.is_contiguous():
            raise RuntimeError("query must be a contiguous float32 CPU tensor")
        B = query.size(0)
        if query.dim() != 2 or query.size(1) != self.d_model:
            raise RuntimeError("query must be [B, d_model]")
        n = 4 * ef_search
        if out_I is None:
            out_I = torch.empty(B, n, dtype=torch.int64, pin_memory=True)
        if out_D is None:
            out_D = torch.empty(B, n, dtype=torch.float32, pin_memory=True)
        _C.check(_C.lib().pa_stage_search(
            self._h, query.data_ptr(), 0 if rotated is None else rotated.data_ptr(),
            out_I.data_ptr(), out_D.data_ptr(), B, ef_search, chunk))
        return out_I, out_D, rotated

    def search_device(self, query: torch.Tensor, ef_search: int, out_I=None, out_D=None,
                      stats=None):
        """Device-resident variant, asynchronous on the stage's own stream; call
        :meth:`synchronize` (or wait on :attr:`stream`) before reading."""
        if query.device != self.device or query.dtype != torch.float32 or not query.is_contiguous():
            raise RuntimeError("query must be a contiguous float32 tensor on the stage's device")
        B = query.size(0)
        if out_I is None:
            out_I = torch.empty(B, 4, ef_search, dtype=torch.int64, device=self.device)
        if out_D is None:
            out_D = torch.empty(B, 4, ef_search, dtype=torch.float32, device=self.device)
        _C.check(_C.lib().pa_stage_search_device(
            self._h, query.data_ptr(), out_I.data_ptr(), out_D.data_ptr(), B, ef_search,
            0 if stats is None else stats.data_ptr()))
        return out_I, out_D

    def synchronize(self) -> None:
        _C.check(_C.lib().pa_stage_synchronize(self._h))

    @property
    def stream(self) -> torch.cuda.ExternalStream:
        return torch.cuda.ExternalStream(_C.lib().pa_stage_stream(self._h), device=self.device)
