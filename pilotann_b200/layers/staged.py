"""The staged index: counterpart of ``pilot_ann/layers/staged.py``.

State-dict keys are upstream's (``VT, storage, mapping, nodelist,
subgraph.indptr/indices, fullgraph.indptr/indices, entry.*``) so that a
checkpoint written by ``dump`` of either implementation loads in the other.
The packed device layout is derived in :meth:`to` and never saved.
"""
from __future__ import annotations

import torch
from torch import nn

from .. import extension, utils
from ..stage import SearchStage
from .entry import IndexEntry


class GraphModule(nn.Module):
    """``pilot_ann/layers/staged.py:6-18``; accepts lists or tensors."""

    def __init__(self, indptr, indices):
        super().__init__()
        self.register_buffer("indptr", torch.as_tensor(indptr, dtype=torch.long))
        self.register_buffer("indices", torch.as_tensor(indices, dtype=torch.long))


class IndexStaged(nn.Module):
    def __init__(self, d_model: int, d_principle: int, sample_ratio: float,
                 graph_method: str = "nsw32", entry_method: str = "random32"):
        super().__init__()
        assert d_principle <= d_model
        self.d_model = d_model
        self.d_principle = d_principle
        self.sample_ratio = sample_ratio
        self.graph_method = graph_method
        self.entry_method = entry_method
        self.cuda_device = None
        for graph_type in ["nsw", "nsg"]:
            if graph_method.startswith(graph_type):
                self.graph_type = graph_type
                self.n_neighbors = int(graph_method.removeprefix(graph_type))
                break
        self.entry = IndexEntry(d_model=d_principle, method=entry_method)
        self.stage: SearchStage | None = None

    # -- checkpointing (pilot_ann/layers/staged.py:59-122) ---------------------
    @classmethod
    def load(cls, ckpt_file):
        checkpoint = torch.load(ckpt_file) if not isinstance(ckpt_file, dict) else ckpt_file
        sd, config = checkpoint["state_dict"], checkpoint["config"]
        index = cls(d_model=config["d_model"], d_principle=config["d_principle"],
                    graph_method=config["graph_method"], entry_method=config["entry_method"],
                    sample_ratio=-1.0)
        for name in ("VT", "storage", "mapping", "nodelist"):
            index.register_buffer(name, sd[name])
        index.register_module("subgraph", GraphModule(sd["subgraph.indptr"], sd["subgraph.indices"]))
        index.register_module("fullgraph", GraphModule(sd["fullgraph.indptr"], sd["fullgraph.indices"]))
        for name in ("entry_nodes", "entry_vectors", "route_vectors"):
            if "entry." + name in sd:
                index.entry.register_buffer(name, sd["entry." + name])
        return index

    def dump(self):
        sd = {k: v for k, v in self.state_dict().items()
              if not k.startswith(("subgraph_cuda.", "storage_cuda"))}
        return {"config": {"d_model": self.d_model, "d_principle": self.d_principle,
                           "graph_method": self.graph_method,
                           "entry_method": self.entry_method},
                "state_dict": sd}

    # -- build (pilot_ann/layers/staged.py:141-189) ------------------------------
    def train(self, x: torch.Tensor, generator: torch.Generator | None = None,
              build_device=None):
        """SVD rotation, full graph, sampled sub-graph, entry tables.  Heavy
        tensor work runs on ``build_device`` (defaults to x's device); the
        registered buffers live on the CPU like upstream's."""
        assert x.dim() == 2 and x.size(-1) == self.d_model
        assert 0.0 < self.sample_ratio <= 1.0
        dev = torch.device(build_device) if build_device is not None else x.device
        xr, V = utils.svd(x.to(dev), max_size=10_000_000, generator=generator)
        self.register_buffer("storage", xr.cpu())
        self.register_buffer("VT", V.T.contiguous().cpu())
        indptr, indices = utils.graph_init(xr, graph_type=self.graph_type,
                                           n_neighbors=self.n_neighbors)
        self.register_module("fullgraph", GraphModule(indptr, indices))
        sub = utils.subgraph_init(indptr=indptr, indices=indices, storage=self.storage,
                                  graph_type=self.graph_type,
                                  n_samples=round(self.sample_ratio * x.size(0)),
                                  n_neighbors=self.n_neighbors, generator=generator, device=dev)
        self.register_module("subgraph", GraphModule(sub[0], sub[1]))
        self.register_buffer("nodelist", sub[2])
        self.register_buffer("mapping", sub[3])
        self.entry.train(self.storage[:, :self.d_principle], generator=generator)
        return self

    # -- device residency (pilot_ann/layers/staged.py:124-139) -------------------
    def to(self, device, max_batch: int = 4096, max_ef: int = 256, n_streams: int = 2,
           refine: str | None = "gpu", refine_slots: int = 0):
        """Uploads the reduced vectors of the sampled nodes, the entry tables,
        the rotation, and the sub-graph in the packed layout (per neighbour slot
        int32 id, storage row and bloom probes, indexed by storage row); creates
        the per-device search stage.

        ``refine="gpu"`` (default) also makes resident what ``traverse_refine``
        reads on the CPU upstream -- the full-dimension vectors and the full graph
        as int32 rows -- so that :meth:`search` can finish on the device;
        ``refine="stage2"`` uploads the vectors only (the sub-graph stage on the GPU,
        the full-graph search stays with a CPU consumer); ``None`` uploads neither."""
        device = torch.device(device)
        self.cuda_device = device
        self.entry.to(device=device)
        self.mapping_cuda = self.mapping.to(device)
        self.subgraph_cuda = GraphModule(self.subgraph.indptr, self.subgraph.indices).to(device)
        storage = torch.index_select(self.storage, dim=0, index=self.nodelist.cpu())
        self.storage_cuda = storage[:, :self.d_principle].contiguous().to(device)
        self.VT_cuda = self.VT.to(device).contiguous()
        self.packed_nbr, self.row_of = extension.pack_graph(
            self.subgraph_cuda.indptr, self.subgraph_cuda.indices, self.mapping_cuda,
            n_storage=self.storage_cuda.size(0), n_neighbors=self.n_neighbors)
        if self.stage is not None:
            self.stage.close()
        self.stage = SearchStage(
            packed_nbr=self.packed_nbr, row_of=self.row_of, storage=self.storage_cuda,
            VT=self.VT_cuda, route_vectors=self.entry.route_vectors,
            entry_nodes=self.entry.entry_nodes, entry_vectors=self.entry.entry_vectors,
            n_neighbors=self.n_neighbors, d_model=self.d_model, max_batch=max_batch,
            max_ef=max_ef, n_streams=n_streams)
        self.storage_full_cuda = self.full_nbr = None
        if refine in ("gpu", "stage2"):
            self.storage_full_cuda = self.storage.to(device).contiguous()
            if refine == "gpu":
                lengths = self.fullgraph.indptr[1:] - self.fullgraph.indptr[:-1]
                degree = max(32, (int(lengths.max().item()) + 31) // 32 * 32)
                self.full_nbr = extension.pack_fullgraph(self.fullgraph.indptr.to(device),
                                                         self.fullgraph.indices.to(device), degree)
            self.stage.attach_refine(self.storage_full_cuda, self.full_nbr, refine_slots)
        elif refine is not None:
            raise RuntimeError('refine must be "gpu", "stage2" or None')
        return self

    # -- search (pilot_ann/layers/staged.py:191-228) ------------------------------
    @torch.no_grad()
    def search_candidates(self, query: torch.Tensor, ef_search: int, chunk_size: int = 0,
                          stage2: bool = False):
        """The GPU stage alone: raw host queries in, candidate handoff out.
        Returns ``(handoff_I [B, 4*ef] int64, handoff_D [B, 4*ef] f32, rotated
        [B, d_model] f32)`` as pinned CPU tensors -- exactly what upstream hands
        to ``traverse_refine`` (``extension/pipeline_cpu.cpp:110-117``); with
        ``stage2`` the rows after the sub-graph stage of the refinement (what
        upstream's stage 3, ``traverse_cpu``, starts from)."""
        assert query.dim() == 2 and self.stage is not None
        query = query.contiguous()
        rotated = torch.empty(query.shape, dtype=torch.float32, pin_memory=True)
        return self.stage.search_host(query, ef_search, chunk=chunk_size, rotated=rotated,
                                      stage2=stage2)

    @torch.no_grad()
    def search(self, query: torch.Tensor, k: int, ef_search: int, chunk_size: int = 128,
               refine=None):
        """``IndexStaged.search`` (``pilot_ann/layers/staged.py:191-228``): raw host
        queries in, ``(topk_I [B, k], topk_D [B, k])`` on the CPU out.

        Who refines the candidates: ``refine`` if given, else what
        :func:`pilotann_b200.set_refine` chose.  ``"gpu"`` finishes on the device
        (needs ``to(..., refine="gpu")``; ``chunk_size`` is not used then).  A callable with the signature of
        upstream's ``extension.traverse_refine`` runs on the host: chunks are
        submitted to the stage's slots and the callable refines one chunk while the
        GPU works on the next ones (upstream's overlap,
        ``extension/pipeline_cpu.cpp:99-141``)."""
        assert query.dim() == 2 and self.stage is not None
        consumer = refine if refine is not None else extension.get_refine()
        if consumer is None:
            raise RuntimeError("search: no consumer for the candidate handoff; pass refine=, call "
                               "pilotann_b200.set_refine, or use search_candidates()")
        query = query.contiguous()
        B = query.size(0)
        if consumer == "gpu":
            if not self.stage.has_full_graph:
                raise RuntimeError('search: the index was moved to the device without '
                                   'refine="gpu"; pass refine=<traverse_refine>')
            # nothing on the host to overlap with, so chunk_size plays no role: the
            # batch goes through in pieces as large as the stage takes
            cap = self.stage.max_batch
            if B <= cap:
                I, D, _ = self.stage.search_host(query, ef_search, k=k)
                return I, D
            I = torch.empty(B, k, dtype=torch.int64, pin_memory=True)
            D = torch.empty(B, k, dtype=torch.float32, pin_memory=True)
            for lo in range(0, B, cap):
                self.stage.search_host(query[lo:lo + cap], ef_search, out_I=I[lo:lo + cap],
                                       out_D=D[lo:lo + cap], k=k)
            return I, D
        stage = self.stage
        step = min(chunk_size if chunk_size > 0 else B, stage.slot_rows)
        chunks = [(lo, min(B, lo + step)) for lo in range(0, B, step)]
        topk_I = torch.empty(B, k, dtype=torch.int64)
        topk_D = torch.empty(B, k, dtype=torch.float32)
        sub = [self.subgraph.indptr, self.subgraph.indices]
        full = [self.fullgraph.indptr, self.fullgraph.indices]
        n_slots = stage.n_streams
        for i in range(len(chunks) + n_slots):
            slot = i % n_slots
            if i >= n_slots:
                lo, hi = chunks[i - n_slots]
                hI, hD, rot = stage.wait(slot)
                consumer(topk_I[lo:hi], topk_D[lo:hi], hI, hD, hI, hD, sub, full, self.storage,
                         rot, ef_search, self.d_principle)
            if i < len(chunks):
                lo, hi = chunks[i]
                stage.submit(slot, query[lo:hi], ef_search, want_rotated=True)
        return topk_I, topk_D
