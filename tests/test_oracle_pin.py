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
