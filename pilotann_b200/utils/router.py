"""Construction of the two-level entry router (build time).

Seeded counterpart of ``pilot_ann/utils/router.py:5-58``.  Layer 0: routers are
picked one at a time, each the candidate (out of ``n_routers`` random nodes)
with the largest summed distance to the routers chosen so far.  Layer 1: in each
of ``n_leaves`` rounds a fresh pool of ``min(1024, n_routers**2)`` unvisited
nodes is drawn (``init_nodes`` are consumed from the back first) and every
router takes the pool node nearest to it as a leaf.
"""
from __future__ import annotations

import torch


@torch.no_grad()
def router_init(storage: torch.Tensor, init_nodes: list | None, n_routers: int,
                n_leaves: int, generator: torch.Generator | None = None):
    assert storage.dim() == 2
    n_storage = storage.size(0)

    def rand_node() -> int:
        return int(torch.randint(n_storage, (1,), generator=generator).item())

    router = [rand_node()]
    chosen = set(router)
    while len(router) < n_routers:
        nodes = torch.randint(n_storage, (n_routers,), generator=generator).tolist()
        dists = torch.cdist(storage[nodes], storage[router], p=2.0)
        pick = nodes[int(torch.argmax(dists.sum(dim=-1)))]
        if pick not in chosen:
            chosen.add(pick)
            router.append(pick)
    route_vectors = storage[router].clone()

    init_nodes = list(init_nodes) if init_nodes else []
    visited: set[int] = set()
    entry_nodes: list[list[int]] = [[] for _ in range(n_routers)]
    pool_size = min(1024, n_routers ** 2)
    if n_storage < n_leaves * pool_size:
        # upstream draws without this check and would spin forever
        raise ValueError(f"router_init needs at least n_leaves * {pool_size} = "
                         f"{n_leaves * pool_size} vectors, got {n_storage}")
    for _ in range(n_leaves):
        pool: list[int] = []
        seen_here: set[int] = set()
        while len(pool) < pool_size:
            node = init_nodes.pop(-1) if init_nodes else rand_node()
            if node in visited or node in seen_here:
                continue
            seen_here.add(node)
            pool.append(node)
        visited |= seen_here
        dists = torch.cdist(route_vectors, storage[pool], p=2.0)
        nearest = torch.argmin(dists, dim=-1).tolist()
        for i in range(n_routers):
            entry_nodes[i].append(pool[nearest[i]])
    return route_vectors, torch.tensor(entry_nodes, dtype=torch.long)
