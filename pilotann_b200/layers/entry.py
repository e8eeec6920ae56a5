"""Entry-point layer: counterpart of ``pilot_ann/layers/entry.py``."""
from __future__ import annotations

import torch
from torch import nn

from .. import extension, utils


class IndexEntry(nn.Module):
    """``method`` is ``'random<n>'`` (n shared random entries) or
    ``'router<r>x<l>'`` (two-level router: r routers with l leaves each), parsed
    as upstream does (``pilot_ann/layers/entry.py:39-56``)."""

    def __init__(self, d_model: int, method: str = "random32"):
        super().__init__()
        self.method = method
        self.d_model = d_model
        self.entry_nodes: torch.Tensor
        self.entry_vectors: torch.Tensor
        self.route_vectors: torch.Tensor
        self.register_buffer("entry_nodes", None)
        self.register_buffer("entry_vectors", None)
        self.register_buffer("route_vectors", None)

    def nodes(self):
        return self.entry_nodes.flatten().tolist()

    def train(self, storage: torch.Tensor, init_nodes: list | None = None,
              generator: torch.Generator | None = None):
        """``pilot_ann/layers/entry.py:26-62`` (``nn.Module.train`` is shadowed
        there too).  ``generator`` makes the draw reproducible."""
        assert isinstance(storage, torch.Tensor)
        if storage.dim() != 2 or storage.size(-1) != self.d_model:
            raise RuntimeError
        if self.entry_nodes is not None:
            return self
        if self.method.startswith("random"):
            n_entries = int(self.method.removeprefix("random"))
            entry_nodes = torch.randint(high=storage.size(0), size=[n_entries],
                                        dtype=torch.long, generator=generator)
            route_vectors = None
        elif self.method.startswith("router"):
            n_routers, n_leaves = [int(x) for x in self.method.removeprefix("router").split("x")]
            route_vectors, entry_nodes = utils.router_init(
                storage=storage, init_nodes=init_nodes, n_routers=n_routers,
                n_leaves=n_leaves, generator=generator)
        else:
            raise NotImplementedError
        self.register_buffer("entry_nodes", entry_nodes)
        self.register_buffer("entry_vectors", storage[entry_nodes].contiguous())
        self.register_buffer("route_vectors", route_vectors)
        return self

    @torch.no_grad()
    def search(self, query: torch.Tensor):
        """``pilot_ann/layers/entry.py:64-89``: returns ``(EP_I, EP_D)``, both
        ``[B, n_entries]``.  On a CUDA device both branches run the routing
        kernel of this package (one launch); on the CPU the 'random' branch is
        upstream's torch expression."""
        assert query.dim() == 2
        batch_size = query.size(0)
        if self.route_vectors is None:
            assert self.entry_vectors.dim() == 2
            if query.is_cuda:
                EP_D = extension.entry_distances(query, self.entry_vectors)
            else:
                EP_D = torch.square(torch.cdist(query, self.entry_vectors, p=2.0))
            EP_I = torch.tile(self.entry_nodes.unsqueeze(0), dims=[batch_size, 1])
        else:
            assert query.is_cuda is True
            assert self.entry_vectors.dim() == 3
            _, EP_D, EP_I = extension.routing_cuda(
                query, self.route_vectors, entry_nodes=self.entry_nodes,
                entry_vectors=self.entry_vectors, with_ids=True)
        return EP_I, EP_D
