"""Seeded small problems shared by the tests (CPU tensors, upstream layout)."""
from __future__ import annotations

import functools

import torch

from pilotann_b200 import utils


@functools.lru_cache(maxsize=32)
def make_problem(n: int = 4096, d: int = 64, n_nb: int = 32, ratio: float = 1.0,
                 batch: int = 64, n_init: int = 32, seed: int = 0, law: str = "fuzz",
                 exact_entries: bool = True, build_device: str = "cpu", graph: str = "nsw"):
    """A graph over n vectors of dim d (already 'reduced'), optionally sampled.
    Returns a dict of CPU tensors in the layout ``traverse_cuda`` takes
    (``extension/entry.cpp:32-38``)."""
    g = torch.Generator().manual_seed(seed)
    if law == "fuzz":
        x = 2.0 * (torch.rand(n, d, generator=g) - 0.5)
        q = 2.0 * (torch.rand(batch, d, generator=g) - 0.5)
    else:
        w = utils.WORKLOADS[{"powerlaw": 2, "powerlaw-ood": 3}.get(law, 1)]
        w = w.scaled(n, batch)
        w = type(w)(**{**w.__dict__, "d_model": d})
        x, q = utils.make_storage(w), utils.make_queries(w)
    dev = torch.device(build_device)
    indptr, indices = utils.graph_init(x.to(dev), graph, n_nb)
    full_indptr, full_indices = indptr, indices
    if ratio < 1.0:
        indptr, indices, nodelist, mapping = utils.subgraph_init(
            indptr, indices, x, graph, n_samples=int(ratio * n), n_neighbors=n_nb,
            generator=g, device=dev)
        storage = x[nodelist].contiguous()
    else:
        mapping = torch.arange(n)
        nodelist = torch.arange(n)
        storage = x
    initial_I = torch.randint(n, (batch, n_init), generator=g)
    diff = q.unsqueeze(1) - x[initial_I]
    initial_D = (diff * diff).sum(-1).contiguous()
    if not exact_entries:
        initial_D = initial_D * (1.0 + 0.01 * torch.rand(batch, n_init, generator=g))
    return dict(indptr=indptr, indices=indices, mapping=mapping, storage=storage, query=q,
                initial_I=initial_I, initial_D=initial_D, n_neighbors=n_nb, full=x,
                nodelist=nodelist, full_indptr=full_indptr, full_indices=full_indices)


def to_cuda(p: dict, device="cuda"):
    return {k: (v.to(device) if isinstance(v, torch.Tensor) else v) for k, v in p.items()}


def topk_ids(out_I: torch.Tensor, out_D: torch.Tensor, k: int):
    """Final top-k ids per query of a [B,4,ef] candidate buffer, by (distance, id)."""
    B = out_I.size(0)
    I = out_I.reshape(B, -1).cpu()
    D = out_D.reshape(B, -1).cpu().clone()
    D[I < 0] = float("inf")
    res = []
    for b in range(B):
        pairs = sorted(set(zip(D[b].tolist(), I[b].tolist())))
        res.append([i for _, i in pairs[:k]])
    return res
