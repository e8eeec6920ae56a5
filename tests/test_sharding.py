"""Host-side sharding logic, single process and two gloo ranks on the CPU."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from pilotann_b200 import sharding


def test_shard_bounds_cover_rows_exactly_once():
    for n in (0, 1, 7, 8, 1024, 1027, 16384):
        for world in (1, 2, 3, 4, 8):
            rows = []
            for r in range(world):
                lo, hi = sharding.shard_bounds(n, world, r)
                assert 0 <= lo <= hi <= n
                rows += list(range(lo, hi))
            assert rows == list(range(n))
            sizes = sharding.shard_sizes(n, world)
            assert max(sizes) - min(sizes) <= 1 and sum(sizes) == n
    with pytest.raises(ValueError):
        sharding.shard_bounds(10, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n_total, result_queue):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        lo, hi = sharding.shard_bounds(n_total, world, rank)
        # every rank "searches" its rows: ids encode (row, slot), distances the row
        ids = (torch.arange(lo, hi).unsqueeze(1) * 100 + torch.arange(10).unsqueeze(0)).long()
        dists = torch.arange(lo, hi, dtype=torch.float32).unsqueeze(1).repeat(1, 10)
        all_ids = sharding.all_gather_rows(ids, n_total)
        all_d = sharding.all_gather_rows(dists, n_total)
        ok = bool((all_ids[:, 0] == torch.arange(n_total) * 100).all()
                  and (all_d[:, 3] == torch.arange(n_total, dtype=torch.float32)).all()
                  and all_ids.shape == (n_total, 10))

        class FakeIndex:              # stands in for IndexStaged on a machine without a GPU
            def search_candidates(self, q, ef, chunk):
                return q[:, :1].long().repeat(1, 4 * ef), q[:, :1].repeat(1, 4 * ef), q

        sh = sharding.ShardedSearch(FakeIndex())
        q = torch.arange(n_total, dtype=torch.float32).unsqueeze(1).repeat(1, 8)
        (l2, h2), I, D, rot = sh.search_candidates(q, 4)
        full = sh.gather(I, n_total)
        ok = ok and (l2, h2) == (lo, hi) and bool((full[:, 0] == torch.arange(n_total)).all())
        # a rank holding the wrong number of rows is an error, not silent corruption
        try:
            sharding.all_gather_rows(ids[:-1], n_total) if hi - lo > 0 else None
            bad_detected = hi - lo == 0
        except RuntimeError:
            bad_detected = True
        result_queue.put((rank, ok, bad_detected))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n_total", [1024, 1027, 3])
def test_all_gather_rows_two_gloo_ranks(n_total):
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, n_total, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(r[0] for r in results) == [0, 1]
    assert all(r[1] for r in results), results
