"""Query sharding across the GPUs of one node.

Upstream is single-GPU (its stream pool is a process-wide static bound to one
device, ``extension/pipeline_cpu.cpp:67-73``).  Queries are independent (one
CTA per query, ``extension/traverse_cuda.cu:54,288``), so the stage shards by
rows: every rank holds a replica of the packed index and searches a contiguous
slice of the batch; there is no collective on the data path.  The only exchange
is optional and comes after the search: an all-gather of the per-rank results
(final top-k, or the candidate handoff) when every rank needs all of them.
It goes through ``torch.distributed`` -- NCCL over NVLink for CUDA tensors, gloo
for CPU tensors -- with uneven shards padded to the largest one.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_bounds(n: int, world: int, rank: int) -> tuple[int, int]:
    """Rows ``[lo, hi)`` of rank ``rank`` when ``n`` rows are cut into ``world``
    contiguous, near-equal shards (the first ``n % world`` shards hold one more)."""
    if world <= 0 or not 0 <= rank < world or n < 0:
        raise ValueError("bad shard request")
    base, extra = divmod(n, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_sizes(n: int, world: int) -> list[int]:
    return [hi - lo for lo, hi in (shard_bounds(n, world, r) for r in range(world))]


def all_gather_rows(local: torch.Tensor, n_total: int, group=None) -> torch.Tensor:
    """Concatenates the row shards of all ranks (shard r = ``shard_bounds(n_total,
    world, r)``) into one ``[n_total, ...]`` tensor on every rank."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    sizes = shard_sizes(n_total, world)
    if local.size(0) != sizes[rank]:
        raise RuntimeError(f"rank {rank} holds {local.size(0)} rows, expected {sizes[rank]}")
    width = max(sizes)
    padded = local
    if local.size(0) < width:
        pad = local.new_zeros((width - local.size(0),) + tuple(local.shape[1:]))
        padded = torch.cat([local, pad])
    out = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(out, padded.contiguous(), group=group)
    return torch.cat([t[:s] for t, s in zip(out, sizes)])


class ShardedSearch:
    """Runs an index's GPU stage on this rank's slice of a batch.

    ``index`` is an ``IndexStaged`` already moved to this rank's device (every
    rank holds a replica).  ``search_candidates`` returns this rank's part of the
    handoff together with its row range; ``gather`` assembles per-rank results.
    """

    def __init__(self, index, group=None):
        self.index = index
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0

    def local_rows(self, n_queries: int) -> tuple[int, int]:
        return shard_bounds(n_queries, self.world, self.rank)

    def search_candidates(self, query: torch.Tensor, ef_search: int, chunk_size: int = 0):
        lo, hi = self.local_rows(query.size(0))
        I, D, rotated = self.index.search_candidates(query[lo:hi].contiguous(), ef_search,
                                                     chunk_size)
        return (lo, hi), I, D, rotated

    def gather(self, local: torch.Tensor, n_queries: int) -> torch.Tensor:
        if self.world == 1:
            return local
        return all_gather_rows(local, n_queries, self.group)
