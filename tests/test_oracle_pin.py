"""Pins the CPU oracle (oracle/pilot_oracle.c) to the upstream code.

* against the committed golden fixtures (tests/golden/golden_cpu.pt, produced by
  tests/golden/make_golden.py from the upstream module compiled in place);
* live against that module (oracle/_ref) when it is present: random heap
  operation traces, traverse_cpu and traverse_refine.
"""
from pathlib import Path

import pytest
import torch

GOLDEN = Path(__file__).parent / "golden" / "golden_cpu.pt"


@pytest.fixture(scope="module")
def golden():
    return torch.load(GOLDEN)


def _replay(oracle, trace):
    kind, hsize = trace["kind"], trace["hsize"]
    keys = torch.full((hsize,), float("inf") if kind == "open" else float("-inf"))
    vals = torch.full((hsize,), -1, dtype=torch.long)
    for op, k, v in trace["ops"]:
        if op == 0:
            oracle.heap_pop(keys, vals)
        elif op == 1:
            oracle.heap_replace(keys, vals, k, v)
        else:
            oracle.heap_pushpop(keys, vals, k, v)
    return keys, vals


def test_heap_traces_match_golden(oracle_lib, golden):
    assert len(golden["heap"]) == 18
    for trace in golden["heap"]:
        keys, vals = _replay(oracle_lib, trace)
        assert torch.equal(keys, trace["keys"]), (trace["hsize"], trace["kind"])
        assert torch.equal(vals, trace["values"]), (trace["hsize"], trace["kind"])


def test_search_cpu_matches_golden(oracle_lib, golden):
    p = golden["problem"]
    for ef, (gI, gD) in golden["search"].items():
        I, D = oracle_lib.search_cpu(p["initial_I"].clone(), p["initial_D"].clone(),
                                     p["full_indptr"], p["full_indices"], p["full"],
                                     p["query"], 10, ef)
        # upstream's host code is built with -ffast-math: ids agree, distances
        # to rounding
        assert (I == gI).float().mean().item() >= 0.995, ef
        assert torch.allclose(D, gD, rtol=1e-5, atol=1e-6)


def test_refine_matches_golden(oracle_lib, golden):
    p = golden["problem"]
    for ef, fx in golden["refine"].items():
        bI, bD = fx["cand_I"].clone(), fx["cand_D"].clone()
        I, D = oracle_lib.refine(bI, bD, [p["indptr"], p["indices"]],
                                 [p["full_indptr"], p["full_indices"]], p["full"], p["query"],
                                 10, ef, fx["d_principle"])
        assert (I == fx["out_I"]).float().mean().item() >= 0.995, ef
        assert torch.allclose(D, fx["out_D"], rtol=1e-5, atol=1e-6)
        # the handoff is rewritten in place: pads then the H best, ascending
        assert (bI == fx["buffer_I"]).float().mean().item() >= 0.995
        fin = torch.isfinite(fx["buffer_D"])
        assert torch.equal(fin, torch.isfinite(bD))
        assert torch.allclose(bD[fin], fx["buffer_D"][fin], rtol=1e-5, atol=1e-6)


def test_heap_random_traces_live(oracle_lib, ref_ext):
    g = torch.Generator().manual_seed(123)
    for trial in range(200):
        hsize = int(torch.randint(1, 300, (1,), generator=g))
        k_o = torch.full((hsize,), float("inf")); v_o = torch.full((hsize,), -1, dtype=torch.long)
        k_r, v_r = k_o.clone(), v_o.clone()
        ops = torch.randint(0, 3, (3 * hsize,), generator=g).tolist()
        ks = torch.rand(3 * hsize, generator=g)
        if trial % 3 == 0:
            ks = torch.round(ks * 16) / 16
        for i, (op, k) in enumerate(zip(ops, ks.tolist())):
            if op == 0:
                ref_ext.heapq_pop_cpu(k_r, v_r); oracle_lib.heap_pop(k_o, v_o)
            elif op == 1:
                ref_ext.heapq_replace_cpu(k_r, v_r, k, i); oracle_lib.heap_replace(k_o, v_o, k, i)
            else:
                ref_ext.heapq_pushpop_cpu(k_r, v_r, k, i); oracle_lib.heap_pushpop(k_o, v_o, k, i)
        assert torch.equal(k_o, k_r) and torch.equal(v_o, v_r), trial


def test_search_and_refine_live(oracle_lib, ref_ext, golden):
    p = golden["problem"]
    x, q = p["full"], p["query"]
    ef = 32
    I_r = torch.empty(q.size(0), 10, dtype=torch.long); D_r = torch.empty(q.size(0), 10)
    ref_ext.traverse_cpu(I_r, D_r, p["initial_I"].clone(), p["initial_D"].clone(),
                         p["full_indptr"], p["full_indices"], x, q, ef)
    I_o, D_o = oracle_lib.search_cpu(p["initial_I"].clone(), p["initial_D"].clone(),
                                     p["full_indptr"], p["full_indices"], x, q, 10, ef)
    assert (I_o == I_r).float().mean().item() >= 0.995
    assert torch.allclose(D_o, D_r, rtol=1e-5, atol=1e-6)


def test_bloom_known_answers(oracle_lib):
    """Hash restated independently in Python from extension/inc/bloom.cuh:9-16 and
    extension/traverse_cuda.cu:65-69."""
    def fnv(x, h):
        for i in range(4):
            h ^= (x >> (8 * i))
            h = (h * 0x01000193) & 0xFFFFFFFF
        return h
    for node in (0, 1, 2, 255, 256, 65535, 123456, 999_999, 2**31 - 1, 2**32 + 5):
        h, want = 0x811C9DC5, []
        for _ in range(4):
            h = fnv(node & 0xFFFFFFFF, h)
            want.append(h % 32768)
        assert oracle_lib.bloom_positions(node) == want
    assert oracle_lib.fnv1a_32(0, 0x811C9DC5) == fnv(0, 0x811C9DC5)


def test_heap_size_dispatch(oracle_lib):
    # extension/traverse_cuda.cu:302-315
    table = {1: 32, 16: 32, 32: 32, 33: 64, 64: 64, 65: 128, 128: 128, 129: 256, 256: 256,
             257: 256, 2048: 256, 2049: -1}
    for ef, h in table.items():
        assert oracle_lib.heap_size_for(ef) == h


def test_refine_in_the_kernels_summation_order_pinned_to_upstream(oracle_lib, ref_ext, golden):
    """``refine_ex(gpu_order=True)`` is what the refinement kernel is compared with
    bit for bit; this pins it to upstream's ``traverse_refine`` itself (AVX2 order,
    -ffast-math): same ids for >= 99.5 % of the entries, distances within 1e-5
    relative, and the same rewritten handoff.  ``gpu_order=False`` is ``refine``."""
    p = golden["problem"]
    x, q = p["full"], p["query"]
    g = torch.Generator().manual_seed(5)
    B, k = q.size(0), 10
    d_p = x.size(1) // 2 // 8 * 8
    sub = [p["indptr"], p["indices"]]
    full = [p["full_indptr"], p["full_indices"]]
    for ef in (16, 48, 128):
        n = 4 * ef
        ids = p["nodelist"][torch.randint(p["nodelist"].numel(), (B, n), generator=g)]
        ids[:, ::7] = -1                                          # pads inside the handoff
        dist = ((q.unsqueeze(1) - x[ids.clamp_min(0)])[:, :, :d_p] ** 2).sum(-1).contiguous()
        dist[ids < 0] = float("inf")
        u_I = torch.empty(B, k, dtype=torch.long); u_D = torch.empty(B, k)
        uI, uD = ids.clone(), dist.clone()
        ref_ext.traverse_refine(u_I, u_D, uI, uD, uI, uD, sub, full, x, q, ef, d_p)
        gI, gD = ids.clone(), dist.clone()
        o_I, o_D, st = oracle_lib.refine_ex(gI, gD, sub, full, x, q, k, ef, d_p, gpu_order=True,
                                            with_stats=True)
        assert (o_I == u_I).float().mean().item() >= 0.995, ef
        same = o_I == u_I
        assert ((o_D - u_D).abs() <= 1e-5 * u_D.abs() + 1e-7)[same].all()
        assert (gI == uI).float().mean().item() >= 0.995           # stage-2 rows
        assert (st[:, 0] <= 2).all() and (st[:, 2] <= 2 * ef).all()
        aI, aD = ids.clone(), dist.clone()
        a_I, a_D = oracle_lib.refine_ex(aI, aD, sub, full, x, q, k, ef, d_p, gpu_order=False)
        bI, bD = ids.clone(), dist.clone()
        b_I, b_D = oracle_lib.refine(bI, bD, sub, full, x, q, k, ef, d_p)
        assert torch.equal(a_I, b_I) and torch.equal(a_D, b_D) and torch.equal(aI, bI)
        # stage 2 alone leaves exactly the rows the two-stage call leaves in the buffer
        sI, sD = ids.clone(), dist.clone()
        oracle_lib.refine_ex(sI, sD, sub, full, x, q, k, ef, d_p, gpu_order=True, stages=2)
        assert torch.equal(sI, gI) and torch.equal(sD.view(torch.int32), gD.view(torch.int32))


def test_warp_order_distance(oracle_lib):
    g = torch.Generator().manual_seed(9)
    for d, off in ((768, 0), (768, 128), (96, 64), (200, 96), (64, 0), (132, 4)):
        q = torch.randn(d, generator=g)
        x = torch.randn(d, generator=g)
        want = ((q.double() - x.double())[off:] ** 2).sum().item()
        got = oracle_lib.warp_distance(q, x, off)
        assert abs(got - want) <= 2e-6 * max(want, 1e-30), (d, off)


def test_cpu_heap_sizes(oracle_lib):
    # extension/traverse_cpu.cpp:228-254
    table = {1: 16, 16: 16, 17: 32, 33: 48, 49: 64, 65: 96, 97: 128, 129: 192, 193: 256,
             257: 384, 385: 512, 513: 1024, 1025: 2048, 2049: -1}
    for ef, h in table.items():
        assert oracle_lib.cpu_heap_size_for(ef) == h
    from pilotann_b200 import _C
    for ef, h in table.items():
        assert _C.lib().pa_cpu_heap_size_for(ef) == h


def test_consumer_hook_validation():
    import pilotann_b200
    assert pilotann_b200.get_refine() == "gpu"
    with pytest.raises(RuntimeError):
        pilotann_b200.set_refine("cpu")
    f = lambda *a: None
    pilotann_b200.set_refine(f)
    assert pilotann_b200.get_refine() is f
    pilotann_b200.set_refine(None)
    assert pilotann_b200.get_refine() is None
    pilotann_b200.set_refine("gpu")


def test_heap_replace_properties_the_refinement_kernel_relies_on(oracle_lib):
    """Two facts about upstream's heap_replace (extension/inc/heapq.cuh:47-77, restated
    and pinned above) that let the refinement kernel skip serial heap work:
    (1) keys offered in strictly ascending order to an empty heap of 2H slots end at
    positions that depend on their rank only -- key 0 at index 0, keys 2t - 1 and 2t at
    the two rightmost nodes of level t -- and all later keys are dropped;
    (2) whatever the order, the two smallest keys offered so far are in the heap."""
    g = torch.Generator().manual_seed(9)

    def position(rank):
        if rank == 0:
            return 0
        level = (rank + 1) // 2
        return (1 << (level + 1)) - 3 + (0 if rank % 2 == 1 else 1)

    for H in (16, 32, 48, 64, 96, 128, 192, 256, 384, 512, 1024, 2048):
        cap = 2 * H
        for count in (0, 1, 2, 5, 9, 16, H // 2, H):
            keys = torch.rand(4 * H + 8, generator=g).unique()[:count].sort().values
            assert keys.numel() == count
            D = torch.full((cap,), float("inf"))
            I = torch.full((cap,), -1, dtype=torch.int64)
            for i in range(count):
                oracle_lib.heap_replace(D, I, float(keys[i]), i)
            want_D = torch.full((cap,), float("inf"))
            want_I = torch.full((cap,), -1, dtype=torch.int64)
            for rank in range(min(count, 64)):
                if position(rank) < cap:
                    want_D[position(rank)] = keys[rank]
                    want_I[position(rank)] = rank
            assert torch.equal(I, want_I) and torch.equal(D, want_D), (H, count)
    for H in (16, 24, 64, 128):
        cap = 2 * H
        for trial in range(20):
            n = int(torch.randint(1, 6 * cap, (1,), generator=g))
            keys = torch.rand(8 * cap, generator=g).unique()[:n]
            keys = keys[torch.randperm(keys.numel(), generator=g)]
            D = torch.full((cap,), float("inf"))
            I = torch.full((cap,), -1, dtype=torch.int64)
            for i in range(keys.numel()):
                oracle_lib.heap_replace(D, I, float(keys[i]), i)
                two = keys[: i + 1].sort().values[:2]
                assert all((D == k).any() for k in two), (H, trial, i)
            # ... and a pop returns the smallest of them
            k, v = oracle_lib.heap_pop(D, I)
            assert k == float(keys.min()) and v == int(keys.argmin())
