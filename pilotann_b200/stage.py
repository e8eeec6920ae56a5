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
        self.n_streams = n_streams
        self.has_refine = False
        self.has_full_graph = False

    # -- refinement on the GPU ---------------------------------------------------
    def attach_refine(self, storage_full: torch.Tensor, full_nbr: torch.Tensor | None,
                      slots_per_stream: int = 0) -> None:
        """Gives the stage what ``traverse_refine`` reads on the CPU upstream: the
        full-dimension vectors ``[n_nodes, d_model]`` and (for the full-graph stage)
        the packed full graph ``int32 [n_nodes, degree]`` (``extension.pack_fullgraph``).
        Allocates the stage's visited pool and refined-row buffers, once."""
        if storage_full.device != self.device or storage_full.dtype != torch.float32 \
                or not storage_full.is_contiguous() or storage_full.dim() != 2 \
                or storage_full.size(1) != self.d_model:
            raise RuntimeError("storage_full must be contiguous float32 [n_nodes, d_model] on "
                               f"{self.device}")
        if full_nbr is not None and (full_nbr.device != self.device or full_nbr.dtype != torch.int32
                                     or not full_nbr.is_contiguous() or full_nbr.dim() != 2
                                     or full_nbr.size(0) != storage_full.size(0)):
            raise RuntimeError("full_nbr must be contiguous int32 [n_nodes, degree]")
        rx = _C.RefineIndex()
        rx.storage_full = storage_full.data_ptr()
        rx.full_nbr = 0 if full_nbr is None else full_nbr.data_ptr()
        rx.full_degree = 0 if full_nbr is None else full_nbr.size(1)
        with torch.cuda.device(self.device):
            _C.check(_C.lib().pa_stage_attach_refine(self._h, ctypes.byref(rx), slots_per_stream))
        self._keep["storage_full"], self._keep["full_nbr"] = storage_full, full_nbr
        self.has_refine, self.has_full_graph = True, full_nbr is not None

    def _mode(self, k, stage2: bool) -> int:
        if k is not None:
            return _C.PA_OUT_TOPK
        return _C.PA_OUT_STAGE2 if stage2 else _C.PA_OUT_HANDOFF

    def close(self) -> None:
        if getattr(self, "_h", None) and _C is not None and _C.lib is not None:
            _C.lib().pa_stage_destroy(self._h)       # (module globals are gone at exit)
            self._h = None

    __del__ = close

    def search_host(self, query: torch.Tensor, ef_search: int, chunk: int = 0,
                    out_I=None, out_D=None, rotated=None, k: int | None = None,
                    stage2: bool = False):
        """Host buffers in, host buffers out (the call a user of the stage makes).
        ``query`` [B, d_model] float32 CPU (pinned for speed).  Returns
        ``(out_I, out_D, rotated)``, pinned CPU tensors: the candidate handoff
        ``[B, 4*ef]`` by default; with ``stage2`` the rows after the sub-graph
        stage of the refinement; with ``k`` the final top-k ``[B, k]`` (both need
        :meth:`attach_refine`)."""
        if query.device.type != "cpu" or query.dtype != torch.float32 or not query.is_contiguous():
            raise RuntimeError("query must be a contiguous float32 CPU tensor")
        B = query.size(0)
        if query.dim() != 2 or query.size(1) != self.d_model:
            raise RuntimeError("query must be [B, d_model]")
        n = 4 * ef_search if k is None else k
        if out_I is None:
            out_I = torch.empty(B, n, dtype=torch.int64, pin_memory=True)
        if out_D is None:
            out_D = torch.empty(B, n, dtype=torch.float32, pin_memory=True)
        if out_I.shape != (B, n) or out_D.shape != (B, n):
            raise RuntimeError(f"output buffers must be [{B}, {n}]")
        _C.check(_C.lib().pa_stage_search_ex(
            self._h, query.data_ptr(), 0 if rotated is None else rotated.data_ptr(),
            out_I.data_ptr(), out_D.data_ptr(), B, ef_search, 0 if k is None else k,
            self._mode(k, stage2), chunk))
        return out_I, out_D, rotated

    def search_device(self, query: torch.Tensor, ef_search: int, out_I=None, out_D=None,
                      stats=None, k: int | None = None, stage2: bool = False, refine_stats=None):
        """Device-resident variant, asynchronous on the stage's own stream; call
        :meth:`synchronize` (or wait on :attr:`stream`) before reading.  Output as
        :meth:`search_host` (the handoff keeps its ``[B, 4, ef]`` shape)."""
        if query.device != self.device or query.dtype != torch.float32 or not query.is_contiguous():
            raise RuntimeError("query must be a contiguous float32 tensor on the stage's device")
        B = query.size(0)
        mode = self._mode(k, stage2)
        shape = (B, k) if k is not None else (B, 4 * ef_search) if stage2 else (B, 4, ef_search)
        if out_I is None:
            out_I = torch.empty(shape, dtype=torch.int64, device=self.device)
        if out_D is None:
            out_D = torch.empty(shape, dtype=torch.float32, device=self.device)
        if out_I.numel() != B * (k if k is not None else 4 * ef_search) or out_D.numel() != out_I.numel():
            raise RuntimeError("output buffers have the wrong size")
        _C.check(_C.lib().pa_stage_search_device_ex(
            self._h, query.data_ptr(), out_I.data_ptr(), out_D.data_ptr(), B, ef_search,
            0 if k is None else k, mode, 0 if stats is None else stats.data_ptr(),
            0 if refine_stats is None else refine_stats.data_ptr()))
        return out_I, out_D

    # -- submit / wait: chunks in flight while the caller consumes earlier ones --------
    @property
    def slot_rows(self) -> int:
        """Queries one slot takes (``max_batch // n_streams``)."""
        return int(_C.lib().pa_stage_slot_rows(self._h))

    def submit(self, slot: int, query: torch.Tensor, ef_search: int, k: int | None = None,
               stage2: bool = False, want_rotated: bool = False) -> None:
        """Enqueues one chunk (``query`` [n, d_model] float32 CPU, n <=
        :attr:`slot_rows`) on slot ``slot`` and returns at once; the results land in
        the slot's own pinned buffers, see :meth:`wait`."""
        if query.device.type != "cpu" or query.dtype != torch.float32 or not query.is_contiguous() \
                or query.dim() != 2 or query.size(1) != self.d_model:
            raise RuntimeError("query must be a contiguous float32 CPU tensor [n, d_model]")
        self._slot_meta = getattr(self, "_slot_meta", {})
        self._slot_meta[slot] = (4 * ef_search if k is None else k, query)   # keeps the source alive
        _C.check(_C.lib().pa_stage_submit(self._h, slot, query.data_ptr(), query.size(0),
                                          ef_search, 0 if k is None else k,
                                          self._mode(k, stage2), int(want_rotated)))

    def wait(self, slot: int):
        """Blocks until the chunk submitted on ``slot`` is complete.  Returns
        ``(out_I [n, row], out_D [n, row], rotated [n, d_model])`` as CPU tensors that
        view the slot's pinned buffers: valid until the slot's next submit."""
        pI, pD, pR, n = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_int64()
        _C.check(_C.lib().pa_stage_wait(self._h, slot, ctypes.byref(pI), ctypes.byref(pD),
                                        ctypes.byref(pR), ctypes.byref(n)))
        row, _ = self._slot_meta.pop(slot)
        rows = n.value

        def view(ptr, ctype, cols, dtype):
            if rows == 0:
                return torch.empty(0, cols, dtype=dtype)
            buf = (ctype * (rows * cols)).from_address(ptr.value)
            return torch.frombuffer(buf, dtype=dtype).view(rows, cols)

        return (view(pI, ctypes.c_int64, row, torch.int64),
                view(pD, ctypes.c_float, row, torch.float32),
                view(pR, ctypes.c_float, self.d_model, torch.float32))

    def synchronize(self) -> None:
        _C.check(_C.lib().pa_stage_synchronize(self._h))

    @property
    def stream(self) -> torch.cuda.ExternalStream:
        return torch.cuda.ExternalStream(_C.lib().pa_stage_stream(self._h), device=self.device)
