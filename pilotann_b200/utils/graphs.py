"""Proximity-graph construction and sub-graph sampling for the search stage.

Upstream builds its graphs with faiss (``pilot_ann/utils/graphs.py:6-93``:
``IndexHNSWFlat`` layer 0 for ``'nsw'``, ``IndexNSGFlat`` for ``'nsg'``), which is
an external dependency; this module is an independent builder that yields the
same *format* -- a padded CSR with ``indptr[i] = i * n_neighbors`` and ``-1``
padding at the tail of each row (``graphs.py:59-76``) -- and a graph of the same
family: nodes are inserted in batches, every new node takes its candidates from
an exact nearest-neighbour scan of the nodes inserted so far, selects up to
``n_neighbors`` of them with the HNSW diversity heuristic, and is linked back
from each selected neighbour (re-pruning lists that overflow); slots the
heuristic leaves free are filled with the nearest pruned candidates (the
"keep pruned connections" option of HNSW implementations).  Early nodes keep
the long-range links they acquired while the graph was small, which is what
makes the result navigable.  Everything is expressed in torch tensor ops and
runs on whichever device ``x`` lives on (a GPU for million-scale inputs).

``subgraph_init`` follows ``pilot_ann/utils/graphs.py:96-132`` and
``extension/sampling_cpu.cpp:5-65``: seeded random seeds plus their one-hop
closure until ``n_samples`` nodes are collected, a fresh graph over the sampled
vectors, ids mapped back to the global id space, CSR over the global id space
with empty rows for nodes outside the sample.

Build-time code: nothing here is on the timed search path.
"""
from __future__ import annotations

import torch


def _pairwise_sq(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Squared L2 between rows of a [.., m, d] and b [.., n, d] (clamped at 0)."""
    a2 = (a * a).sum(-1, keepdim=True)
    b2 = (b * b).sum(-1).unsqueeze(-2)
    return (a2 + b2 - 2.0 * a @ b.transpose(-1, -2)).clamp_min_(0.0)


def _select_diverse(cand: torch.Tensor, cand_d: torch.Tensor, x: torch.Tensor,
                    max_keep: int, keep_pruned: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
    """HNSW neighbour-selection heuristic, batched.

    cand [b, C] candidate ids sorted by ascending distance to the owner (``-1``
    = empty), cand_d [b, C] those distances.  A candidate is kept iff it is not
    closer to an already kept candidate than to the owner.  Returns ids and
    distances [b, max_keep], ``-1`` / ``inf`` padded, still ascending.
    """
    b, C = cand.shape
    valid = cand >= 0
    vecs = x[cand.clamp_min(0)]                                 # [b, C, d]
    pair = _pairwise_sq(vecs, vecs)                             # [b, C, C]
    kept = torch.zeros(b, C, dtype=torch.bool, device=cand.device)
    count = torch.zeros(b, dtype=torch.long, device=cand.device)
    for i in range(C):
        blocked = ((pair[:, i, :] < cand_d[:, i:i + 1]) & kept).any(dim=1)
        take = valid[:, i] & ~blocked & (count < max_keep)
        kept[:, i] = take
        count += take.long()
    if keep_pruned:
        # fill the free slots with the nearest pruned candidates (kept ones first)
        rank = torch.where(kept, 0, torch.where(valid, 1, 2)).to(torch.int8)
        order = torch.argsort(rank, dim=1, stable=True)[:, :max_keep]
        out_i = torch.gather(cand, 1, order)
        out_d = torch.gather(cand_d, 1, order)
        ok = torch.gather(valid, 1, order)
        out_i = torch.where(ok, out_i, torch.full_like(out_i, -1))
        out_d = torch.where(ok, out_d, torch.full_like(out_d, float("inf")))
        resort = torch.argsort(out_d, dim=1, stable=True)
        return torch.gather(out_i, 1, resort), torch.gather(out_d, 1, resort)
    # stable left-compaction of the kept candidates
    order = torch.argsort((~kept).to(torch.int8), dim=1, stable=True)[:, :max_keep]
    out_i = torch.gather(cand, 1, order)
    out_d = torch.gather(cand_d, 1, order)
    keep_mask = torch.gather(kept, 1, order)
    out_i = torch.where(keep_mask, out_i, torch.full_like(out_i, -1))
    out_d = torch.where(keep_mask, out_d, torch.full_like(out_d, float("inf")))
    return out_i, out_d


def _topk_candidates(x: torch.Tensor, lo: int, hi: int, n_cand: int,
                     chunk: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Exact n_cand nearest nodes among [0, hi) for every node in [lo, hi)."""
    base = x[:hi]
    base2 = (base * base).sum(-1)
    ids, dists = [], []
    k = min(n_cand, hi - 1)
    for s in range(lo, hi, chunk):
        e = min(hi, s + chunk)
        q = x[s:e]
        d = (q * q).sum(-1, keepdim=True) + base2.unsqueeze(0) - 2.0 * q @ base.T
        d[torch.arange(e - s, device=x.device), torch.arange(s, e, device=x.device)] = float("inf")
        dd, ii = torch.topk(d, k, dim=1, largest=False)
        ids.append(ii)
        dists.append(dd.clamp_min_(0.0))
    return torch.cat(ids), torch.cat(dists)


class _Cells:
    """Coarse partition of the vectors for candidate generation at large N: every
    node belongs to the cell of its nearest of ``n_cells`` sampled vectors, and
    looks for neighbours only among the members of the ``n_probe`` cells nearest to
    its own cell's centre -- the scan per node shrinks from N to about
    ``n_probe * N / n_cells`` vectors.  Members of a cell are kept in ascending id
    order, so "the members inserted so far" is a prefix of the cell."""

    def __init__(self, x: torch.Tensor, n_cells: int, n_probe: int, seed: int = 0,
                 chunk: int = 1 << 18):
        N = x.size(0)
        dev = x.device
        g = torch.Generator().manual_seed(seed)
        pick = torch.randperm(N, generator=g)[:n_cells].to(dev)
        self.centres = x[pick]
        c2 = (self.centres * self.centres).sum(-1)
        cell = torch.empty(N, dtype=torch.long, device=dev)
        for s in range(0, N, chunk):
            q = x[s:s + chunk]
            cell[s:s + chunk] = torch.argmin(c2.unsqueeze(0) - 2.0 * q @ self.centres.T, dim=1)
        self.n_cells, self.n_probe, self.N = n_cells, min(n_probe, n_cells), N
        self.order = torch.argsort(cell, stable=True)            # by cell, ids ascending inside
        self.key = cell[self.order] * N + self.order              # sorted
        self.probe = torch.topk(_pairwise_sq(self.centres, self.centres), self.n_probe, dim=1,
                                largest=False).indices            # [n_cells, n_probe], own cell first

    def bounds(self, limit: int) -> torch.Tensor:
        """Per cell: position in ``order`` of its first member with id >= limit."""
        cells = torch.arange(self.n_cells, device=self.key.device)
        return torch.searchsorted(self.key, cells * self.N + limit)

    def candidates(self, x: torch.Tensor, lo: int, hi: int, n_cand: int,
                   max_block: int = 1 << 28) -> tuple[torch.Tensor, torch.Tensor]:
        """``n_cand`` nearest nodes among [0, hi), probed cells only, for every node
        of [lo, hi): ids / distances [hi - lo, n_cand], ``-1`` / ``inf`` padded."""
        dev = x.device
        out_i = torch.full((hi - lo, n_cand), -1, dtype=torch.long, device=dev)
        out_d = torch.full((hi - lo, n_cand), float("inf"), dtype=x.dtype, device=dev)
        start = self.bounds(0).tolist()
        from_lo = self.bounds(lo).tolist()
        to_hi = self.bounds(hi).tolist()
        probe = self.probe.tolist()
        for c in range(self.n_cells):
            if to_hi[c] == from_lo[c]:
                continue
            mine = self.order[from_lo[c]:to_hi[c]]                # this cell's nodes in the batch
            cand = torch.cat([self.order[start[p]:to_hi[p]] for p in probe[c]])
            if cand.numel() == 0:
                continue
            base = x[cand]
            b2 = (base * base).sum(-1)
            k = min(n_cand, cand.numel())
            rows = max(1, max_block // max(1, cand.numel()))
            for s in range(0, mine.numel(), rows):
                ids = mine[s:s + rows]
                q = x[ids]
                d = (q * q).sum(-1, keepdim=True) + b2.unsqueeze(0) - 2.0 * q @ base.T
                d[cand.unsqueeze(0) == ids.unsqueeze(1)] = float("inf")
                dd, ii = torch.topk(d, k, dim=1, largest=False)
                found = cand[ii]
                found[torch.isinf(dd)] = -1
                out_i[ids - lo, :k] = found
                out_d[ids - lo, :k] = dd.clamp_min_(0.0)
        return out_i, out_d


#: above this many vectors the candidate scans are restricted to nearby cells
CELL_THRESHOLD = 1_500_000


@torch.no_grad()
def build_graph(x: torch.Tensor, n_neighbors: int, ef_construct: int = 80,
                first_batch: int = 1024, growth: float = 1.5,
                chunk_bytes: int = 1 << 30, keep_pruned: bool = False,
                cells: "_Cells | None | str" = "auto", exact_below: int = 200_000) -> torch.Tensor:
    """Returns the adjacency as an int64 tensor [N, n_neighbors], ``-1`` padded.

    ``cells``: ``"auto"`` restricts the candidate scans to nearby cells (see
    :class:`_Cells`) once N exceeds ``CELL_THRESHOLD``; ``None`` always scans
    exactly; batches whose scan covers fewer than ``exact_below`` vectors are
    always exact."""
    assert x.dim() == 2
    N, d = x.shape
    dev = x.device
    M = n_neighbors
    C = max(M, ef_construct)
    adj = torch.full((N, M), -1, dtype=torch.long, device=dev)
    adj_d = torch.full((N, M), float("inf"), dtype=x.dtype, device=dev)
    if N <= 1:
        return adj
    if isinstance(cells, str):
        cells = None
        if N > CELL_THRESHOLD:
            n_cells = max(64, int(round((N / 2400) / 64)) * 64)
            cells = _Cells(x, n_cells=n_cells, n_probe=8)
    # rows of distance matrix / gathered candidate vectors held at once
    prune_rows = max(64, chunk_bytes // (C * max(d, C) * 4 * 3))
    lo = 0
    hi = min(N, first_batch)
    while lo < N:
        scan_rows = max(64, chunk_bytes // (hi * 4 * 3))
        if cells is not None and hi > exact_below:
            cand, cand_d = cells.candidates(x, lo, hi, C)
        else:
            cand, cand_d = _topk_candidates(x, lo, hi, C, scan_rows)
        rev_src, rev_dst, rev_d = [], [], []
        for s in range(0, hi - lo, prune_rows):
            e = min(hi - lo, s + prune_rows)
            sel_i, sel_d = _select_diverse(cand[s:e], cand_d[s:e], x, M, keep_pruned)
            adj[lo + s:lo + e] = sel_i
            adj_d[lo + s:lo + e] = sel_d
            owner = torch.arange(lo + s, lo + e, device=dev).unsqueeze(1).expand_as(sel_i)
            m = sel_i >= 0
            rev_src.append(owner[m]); rev_dst.append(sel_i[m]); rev_d.append(sel_d[m])
        _add_reverse_links(adj, adj_d, x, torch.cat(rev_dst), torch.cat(rev_src),
                           torch.cat(rev_d), prune_rows, keep_pruned)
        lo = hi
        hi = min(N, max(hi + first_batch, int(hi * growth)))
    return adj


def _add_reverse_links(adj, adj_d, x, dst, src, dist, prune_rows: int,
                       keep_pruned: bool = False) -> None:
    """Give every ``dst`` node a link to ``src`` (distance ``dist``); lists that
    overflow are re-selected with the diversity heuristic over old + new."""
    M = adj.size(1)
    dev = adj.device
    if dst.numel() == 0:
        return
    # drop links that already exist
    exists = (adj[dst] == src.unsqueeze(1)).any(dim=1)
    dst, src, dist = dst[~exists], src[~exists], dist[~exists]
    if dst.numel() == 0:
        return
    # group incoming links by destination, nearest first, at most M per node
    key = torch.argsort(dist, stable=True)
    dst, src, dist = dst[key], src[key], dist[key]
    key = torch.argsort(dst, stable=True)
    dst, src, dist = dst[key], src[key], dist[key]
    uniq, counts = torch.unique_consecutive(dst, return_counts=True)
    starts = torch.cumsum(counts, 0) - counts
    rank = torch.arange(dst.numel(), device=dev) - torch.repeat_interleave(starts, counts)
    row = torch.repeat_interleave(torch.arange(uniq.numel(), device=dev), counts)
    ok = rank < M
    inc_i = torch.full((uniq.numel(), M), -1, dtype=torch.long, device=dev)
    inc_d = torch.full((uniq.numel(), M), float("inf"), dtype=adj_d.dtype, device=dev)
    inc_i[row[ok], rank[ok]] = src[ok]
    inc_d[row[ok], rank[ok]] = dist[ok]
    for s in range(0, uniq.numel(), prune_rows):
        e = min(uniq.numel(), s + prune_rows)
        nodes = uniq[s:e]
        all_i = torch.cat([adj[nodes], inc_i[s:e]], dim=1)          # [b, 2M]
        all_d = torch.cat([adj_d[nodes], inc_d[s:e]], dim=1)
        all_d = torch.where(all_i >= 0, all_d, torch.full_like(all_d, float("inf")))
        order = torch.argsort(all_d, dim=1, stable=True)
        all_i = torch.gather(all_i, 1, order)
        all_d = torch.gather(all_d, 1, order)
        fits = (all_i >= 0).sum(1) <= M
        new_i = all_i[:, :M].clone()
        new_d = all_d[:, :M].clone()
        if (~fits).any():
            sel_i, sel_d = _select_diverse(all_i[~fits], all_d[~fits], x, M, keep_pruned)
            new_i[~fits] = sel_i
            new_d[~fits] = sel_d
        adj[nodes] = new_i
        adj_d[nodes] = new_d


def graph_init(x: torch.Tensor, graph_type: str, n_neighbors: int,
               ef_construct: int = 80):
    """Counterpart of ``pilot_ann/utils/graphs.py:80-93``; returns int64 tensors
    ``(indptr [N+1], indices [N * n_neighbors])`` on the CPU.  ``'nsw'`` and
    ``'nsg'`` share the builder; the NSG flavour draws its candidates from a
    wider scan, as NSG does from its kNN graph."""
    if graph_type not in ("nsw", "nsg"):
        raise RuntimeError(graph_type)
    n_cand = ef_construct if graph_type == "nsw" else max(ef_construct, 3 * n_neighbors)
    chunk = (8 << 30) if x.is_cuda else (1 << 30)
    adj = build_graph(x, n_neighbors, ef_construct=n_cand, chunk_bytes=chunk, keep_pruned=True)
    N = x.size(0)
    indptr = torch.arange(N + 1, dtype=torch.long) * n_neighbors
    return indptr, adj.reshape(-1).cpu()


def graph_sampling(indptr: torch.Tensor, indices: torch.Tensor, n_samples: int,
                   n_hops: int = 1, generator: torch.Generator | None = None):
    """Seeded restatement of ``extension/sampling_cpu.cpp:5-65`` for one hop:
    random seeds and their neighbours are added until at least ``n_samples``
    nodes are in the sample.  Returns ``(nodelist sorted [n_s], mapping [N])``
    with ``mapping[u] = position of u in nodelist or -1``."""
    assert n_hops == 1
    n_nodes = indptr.numel() - 1
    n_samples = min(n_samples, n_nodes)
    chosen = torch.zeros(n_nodes, dtype=torch.bool)
    count = 0
    deg = max(1, int((indptr[1:] - indptr[:-1]).float().mean().item()))
    while count < n_samples:
        n_seeds = max(1, (n_samples - count) // (deg + 1))
        seeds = torch.randint(n_nodes, (n_seeds,), generator=generator)
        chosen[seeds] = True
        offs = indptr[seeds].unsqueeze(1) + torch.arange(deg).unsqueeze(0)
        inside = offs < indptr[seeds + 1].unsqueeze(1)
        nb = indices[offs.clamp_max(indices.numel() - 1)]
        nb = nb[inside & (nb >= 0)]
        chosen[nb] = True
        count = int(chosen.sum().item())
    nodelist = torch.nonzero(chosen).flatten()
    mapping = torch.full((n_nodes,), -1, dtype=torch.long)
    mapping[nodelist] = torch.arange(nodelist.numel())
    return nodelist, mapping


def subgraph_init(indptr: torch.Tensor, indices: torch.Tensor, storage: torch.Tensor,
                  graph_type: str, n_samples: int, n_neighbors: int, n_hops: int = 1,
                  generator: torch.Generator | None = None, device=None):
    """Counterpart of ``pilot_ann/utils/graphs.py:96-132``.  Returns
    ``(indptr [N+1], indices, nodelist, mapping)`` as int64 CPU tensors: a CSR
    over the global id space whose rows are empty for nodes outside the sample
    and hold global ids (``-1`` padded) for sampled ones."""
    nodelist, mapping = graph_sampling(indptr, indices, n_samples, n_hops, generator)
    sub_x = storage[nodelist]
    if device is not None:
        sub_x = sub_x.to(device)
    _, sg = graph_init(sub_x, graph_type, n_neighbors)
    sg = sg.reshape(-1, n_neighbors)
    glob = torch.where(sg >= 0, nodelist[sg.clamp_min(0)], torch.full_like(sg, -1))
    n_nodes = indptr.numel() - 1
    lengths = torch.zeros(n_nodes, dtype=torch.long)
    lengths[nodelist] = n_neighbors
    new_indptr = torch.zeros(n_nodes + 1, dtype=torch.long)
    torch.cumsum(lengths, 0, out=new_indptr[1:])
    return new_indptr, glob.reshape(-1).contiguous(), nodelist, mapping
