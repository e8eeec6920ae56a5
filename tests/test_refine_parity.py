"""The refinement kernel (``pa_refine``: stage 2 on the sub-graph, stage 3 on the
full graph, visited marks from the device pool) against

* the CPU oracle restating upstream ``traverse_refine`` with THIS kernel's
  summation order: ids, distance bits and per-stage counters identical;
* upstream's own ``traverse_refine`` (AVX2 order, built with -ffast-math, so no
  bit equality): top-k ids identical for at least 99.5 % of the queries,
  distances within 1e-5 relative.

The handoff both sides consume is produced by the traversal kernel of this
package on the same tensors.
"""
import pytest
import torch

from helpers import make_problem, to_cuda

pytestmark = pytest.mark.gpu


def _case(n=12000, d=96, d_p=32, ratio=0.5, batch=256, ef=48, law="powerlaw", seed=41,
          n_init=32):
    """Handoff [B, 4*ef] from the reduced-space traversal + everything the
    refinement needs, CPU and CUDA."""
    from pilotann_b200 import extension
    p = make_problem(n=n, d=d, ratio=ratio, batch=batch, n_init=n_init, seed=seed, law=law,
                     build_device="cuda")
    full = p["full"]
    reduced = p["storage"][:, :d_p].contiguous()              # rows of the sampled nodes
    q = p["query"]
    q_red = q[:, :d_p].contiguous()
    g = torch.Generator().manual_seed(seed)
    ids = p["nodelist"][torch.randint(p["nodelist"].numel(), (batch, n_init), generator=g)]
    diff = q_red.unsqueeze(1) - full[ids][:, :, :d_p]
    init_D = (diff * diff).sum(-1).contiguous()
    dev = "cuda"
    nbr, row_of = extension.pack_graph(p["indptr"].to(dev), p["indices"].to(dev),
                                       p["mapping"].to(dev), reduced.size(0), 32)
    oI = torch.empty(batch, 4, ef, dtype=torch.int64, device=dev)
    oD = torch.empty(batch, 4, ef, device=dev)
    extension.traverse_packed(oI, oD, nbr, row_of, reduced.to(dev), q_red.to(dev), ids.to(dev),
                              init_D.to(dev), 32)
    full_nbr = extension.pack_fullgraph(p["full_indptr"].to(dev), p["full_indices"].to(dev), 32)
    torch.cuda.synchronize()
    return dict(p=p, nbr=nbr, row_of=row_of, full_nbr=full_nbr, hand_I=oI, hand_D=oD,
                full=full, full_cuda=full.to(dev), q=q, q_cuda=q.to(dev), d_p=d_p, ef=ef)


@pytest.mark.parametrize("ef,d,d_p,law", [(16, 64, 32, "fuzz"), (48, 96, 32, "powerlaw"),
                                          (128, 200, 96, "powerlaw-ood"), (40, 64, 64, "mixture")])
def test_both_stages_bit_exact_vs_oracle(oracle_lib, ef, d, d_p, law):
    from pilotann_b200 import extension
    c = _case(d=d, d_p=d_p, ef=ef, law=law, batch=192)
    p = c["p"]
    k = 10
    pool = extension.VisitedPool(c["full"].size(0), 96)      # fewer slots than queries
    sub = [p["indptr"], p["indices"]]
    full = [p["full_indptr"], p["full_indices"]]
    hI = c["hand_I"].reshape(192, -1).cpu()
    hD = c["hand_D"].reshape(192, -1).cpu()
    # stage 2 alone: the rewritten handoff rows
    st = torch.zeros(192, 4, dtype=torch.int32, device="cuda")
    g_I, g_D = extension.refine(c["hand_I"], c["hand_D"], c["q_cuda"], c["full_cuda"], c["nbr"],
                                c["row_of"], None, pool, ef, d_p, k=None, stats=st)
    w_bI, w_bD = hI.clone(), hD.clone()
    _, _, w_st = oracle_lib.refine_ex(w_bI, w_bD, sub, full, c["full"], c["q"], k, ef, d_p,
                                      gpu_order=True, stages=2, with_stats=True)
    torch.cuda.synchronize()
    assert torch.equal(g_I.cpu(), w_bI)
    assert torch.equal(g_D.cpu().view(torch.int32), w_bD.view(torch.int32))
    assert torch.equal(st.cpu()[:, :2], w_st[:, :2])
    H = oracle_lib.cpu_heap_size_for(ef)
    assert (g_I[:, : 4 * ef - H] == -1).all() and (g_I[:, -1] >= 0).float().mean() > 0.9
    # both stages: top-k
    st.zero_()
    t_I, t_D = extension.refine(c["hand_I"], c["hand_D"], c["q_cuda"], c["full_cuda"], c["nbr"],
                                c["row_of"], c["full_nbr"], pool, ef, d_p, k=k, stats=st)
    w_I, w_D, w_st = oracle_lib.refine_ex(hI.clone(), hD.clone(), sub, full, c["full"], c["q"], k,
                                          ef, d_p, gpu_order=True, stages=3, with_stats=True)
    torch.cuda.synchronize()
    assert torch.equal(t_I.cpu(), w_I)
    assert torch.equal(t_D.cpu().view(torch.int32), w_D.view(torch.int32))
    assert torch.equal(st.cpu(), w_st)
    # the handoff itself was only read
    assert torch.equal(c["hand_I"].reshape(192, -1).cpu(), hI)
    # exact distances of what came back
    exact = (c["q"].unsqueeze(1) - c["full"][w_I]).square().sum(-1)
    assert torch.allclose(t_D.cpu(), exact, rtol=1e-4, atol=1e-6)


def test_against_upstream_traverse_refine(ref_ext):
    from pilotann_b200 import extension, utils
    ef, k = 64, 10
    c = _case(n=20000, d=128, d_p=32, ef=ef, law="powerlaw", batch=512, seed=43)
    p = c["p"]
    B = 512
    pool = extension.VisitedPool(c["full"].size(0), 1024)
    t_I, t_D = extension.refine(c["hand_I"], c["hand_D"], c["q_cuda"], c["full_cuda"], c["nbr"],
                                c["row_of"], c["full_nbr"], pool, ef, c["d_p"], k=k)
    torch.cuda.synchronize()
    hI = c["hand_I"].reshape(B, -1).cpu().clone()
    hD = c["hand_D"].reshape(B, -1).cpu().clone()
    u_I = torch.empty(B, k, dtype=torch.int64)
    u_D = torch.empty(B, k, dtype=torch.float32)
    ref_ext.traverse_refine(u_I, u_D, hI, hD, hI, hD, [p["indptr"], p["indices"]],
                            [p["full_indptr"], p["full_indices"]], c["full"], c["q"], ef, c["d_p"])
    same = (t_I.cpu() == u_I).all(dim=1).float().mean().item()
    print(f"top-{k} rows identical to upstream traverse_refine: {same:.4f}")
    assert same >= 0.995
    both = t_I.cpu() == u_I
    rel = ((t_D.cpu() - u_D).abs() / u_D.abs().clamp_min(1e-30))[both]
    assert rel.max().item() <= 1e-5
    truth = utils.ground_truth(c["q"], c["full"], k)
    assert abs(utils.recall(t_I.cpu(), truth) - utils.recall(u_I, truth)) <= 0.002
    # stage 2 alone, then upstream's full-graph search on its rows: what a caller
    # gets who keeps stage 3 on the CPU
    s_I, s_D = extension.refine(c["hand_I"], c["hand_D"], c["q_cuda"], c["full_cuda"], c["nbr"],
                                c["row_of"], None, pool, ef, c["d_p"], k=None)
    v_I = torch.empty(B, k, dtype=torch.int64)
    v_D = torch.empty(B, k, dtype=torch.float32)
    ref_ext.traverse_cpu(v_I, v_D, s_I.cpu(), s_D.cpu(), p["full_indptr"], p["full_indices"],
                         c["full"], c["q"], ef)
    assert abs(utils.recall(v_I, truth) - utils.recall(u_I, truth)) <= 0.005
    # after upstream's stage 2 the buffer holds exact full distances
    # (test/kernel/test_traverse_refine.py:89-95 checks the same of upstream)
    real = s_I.cpu() >= 0
    exact = (c["q"].unsqueeze(1) - c["full"][s_I.cpu().clamp_min(0)]).square().sum(-1)
    assert torch.allclose(s_D.cpu()[real], exact[real], rtol=1e-4, atol=1e-6)


def test_marker_wrap_and_slot_reuse(oracle_lib):
    """One slot serves 600 queries in a row: its marker passes 254 twice and the
    array is wiped in between; results stay those of the oracle."""
    from pilotann_b200 import extension
    ef, k, B = 16, 5, 600
    c = _case(n=6000, d=64, d_p=32, ef=ef, law="fuzz", batch=B, seed=47)
    p = c["p"]
    pool = extension.VisitedPool(c["full"].size(0), 1)
    t_I, t_D = extension.refine(c["hand_I"], c["hand_D"], c["q_cuda"], c["full_cuda"], c["nbr"],
                                c["row_of"], c["full_nbr"], pool, ef, c["d_p"], k=k)
    torch.cuda.synchronize()
    w_I, w_D = oracle_lib.refine_ex(c["hand_I"].reshape(B, -1).cpu().clone(),
                                    c["hand_D"].reshape(B, -1).cpu().clone(),
                                    [p["indptr"], p["indices"]],
                                    [p["full_indptr"], p["full_indices"]], c["full"], c["q"], k,
                                    ef, c["d_p"], gpu_order=True, stages=3)
    assert torch.equal(t_I.cpu(), w_I)
    assert torch.equal(t_D.cpu().view(torch.int32), w_D.view(torch.int32))


def test_ragged_rows_pads_duplicates_and_sparse_handoff(oracle_lib):
    """Rows cut short by -1, a repeated id inside a row, queries whose handoff is
    mostly pads, ids outside the sample: the cases upstream's loops guard against
    (traverse_cpu.cpp:47-49, 109-116)."""
    from pilotann_b200 import extension
    ef, k, B = 32, 10, 64
    c = _case(n=6000, d=64, d_p=32, ef=ef, law="fuzz", batch=B, seed=53)
    p = c["p"]
    n = c["full"].size(0)
    g = torch.Generator().manual_seed(9)
    full_indices = p["full_indices"].clone().reshape(n, 32)
    cut = torch.randint(n, (n // 3,), generator=g)
    full_indices[cut, 20:] = -1                              # rows ending early
    full_indices[cut[:500], 7] = full_indices[cut[:500], 3]  # a repeated id
    full_indices = full_indices.reshape(-1).contiguous()
    full_nbr = extension.pack_fullgraph(p["full_indptr"].cuda(), full_indices.cuda(), 32)
    hI = c["hand_I"].reshape(B, -1).clone()
    hD = c["hand_D"].reshape(B, -1).clone()
    hI[:8, 5:] = -1                                          # almost empty handoffs
    hD[:8, 5:] = float("inf")
    hI[8:12] = -1                                            # nothing at all
    pool = extension.VisitedPool(n, 16)
    t_I, t_D = extension.refine(hI, hD, c["q_cuda"], c["full_cuda"], c["nbr"], c["row_of"],
                                full_nbr, pool, ef, c["d_p"], k=k)
    torch.cuda.synchronize()
    w_I, w_D = oracle_lib.refine_ex(hI.cpu().clone(), hD.cpu().clone(),
                                    [p["indptr"], p["indices"]],
                                    [p["full_indptr"], full_indices], c["full"], c["q"], k, ef,
                                    c["d_p"], gpu_order=True, stages=3)
    assert torch.equal(t_I.cpu(), w_I)
    assert torch.equal(t_D.cpu().view(torch.int32), w_D.view(torch.int32))
    assert (t_I[8:12] == -1).all()


def test_rejections():
    from pilotann_b200 import _C
    lib = _C.lib()
    # stages must be 2 or 3
    rc = lib.pa_refine(0, 0, 0, 0, 0, 0, 0, 0, 32, 0, 32, 4, 100, 64, 32, 64, 16, 10, 1, 0, 0, 0)
    assert rc == _C.PA_ERR_ARG and b"stages" in lib.pa_last_error()
    # k larger than the candidate row
    rc = lib.pa_refine(0, 0, 0, 0, 0, 0, 0, 0, 32, 0, 32, 4, 100, 64, 32, 64, 16, 100, 3, 0, 0, 0)
    assert rc == _C.PA_ERR_ARG and b"k must" in lib.pa_last_error()
    # d_principle > d_model
    rc = lib.pa_refine(0, 0, 0, 0, 0, 0, 0, 0, 32, 0, 32, 4, 100, 64, 96, 64, 16, 10, 3, 0, 0, 0)
    assert rc == _C.PA_ERR_ARG
    # a pool for fewer nodes is refused at creation of the call, and n_slots <= 0 at creation
    import ctypes
    h = ctypes.c_void_p()
    assert lib.pa_visited_pool_create(ctypes.byref(h), 100, 0) == _C.PA_ERR_ARG
    assert lib.pa_visited_pool_bytes(1000, 4) == 4 * 1008 + 32


def test_large_ef_and_wide_rows(oracle_lib):
    """ef_search 1024: heaps of 1024 / 2048 entries and a 4096-entry handoff row (more
    shared memory than a CTA gets by default, so the launch opts in), the traversal
    pads the handoff beyond its 256-entry heaps with (-1, -inf); and a degree-64
    sub-graph (two 32-slot chunks per adjacency row)."""
    from pilotann_b200 import extension
    from helpers import make_problem
    k = 10
    for ef, n_nb in ((1024, 32), (64, 64)):
        B, d, d_p = 48, 64, 32
        p = make_problem(n=6000, d=d, n_nb=n_nb, ratio=0.5, batch=B, n_init=32, seed=61)
        full = p["full"]
        reduced = p["storage"][:, :d_p].contiguous()
        q = p["query"]
        g = torch.Generator().manual_seed(3)
        ids = p["nodelist"][torch.randint(p["nodelist"].numel(), (B, 32), generator=g)]
        init_D = ((q[:, :d_p].unsqueeze(1) - full[ids][:, :, :d_p]) ** 2).sum(-1).contiguous()
        nbr, row_of = extension.pack_graph(p["indptr"].cuda(), p["indices"].cuda(),
                                           p["mapping"].cuda(), reduced.size(0), n_nb)
        hI = torch.empty(B, 4, ef, dtype=torch.int64, device="cuda")
        hD = torch.empty(B, 4, ef, device="cuda")
        extension.traverse_packed(hI, hD, nbr, row_of, reduced.cuda(), q[:, :d_p].contiguous().cuda(),
                                  ids.cuda(), init_D.cuda(), n_nb)
        full_nbr = extension.pack_fullgraph(p["full_indptr"].cuda(), p["full_indices"].cuda(), n_nb)
        pool = extension.VisitedPool(full.size(0), 16)
        st = torch.zeros(B, 4, dtype=torch.int32, device="cuda")
        t_I, t_D = extension.refine(hI, hD, q.cuda(), full.cuda(), nbr, row_of, full_nbr, pool, ef,
                                    d_p, k=k, stats=st)
        torch.cuda.synchronize()
        w_I, w_D, w_st = oracle_lib.refine_ex(hI.reshape(B, -1).cpu(), hD.reshape(B, -1).cpu(),
                                              [p["indptr"], p["indices"]],
                                              [p["full_indptr"], p["full_indices"]], full, q, k, ef,
                                              d_p, gpu_order=True, with_stats=True)
        assert torch.equal(t_I.cpu(), w_I), (ef, n_nb)
        assert torch.equal(t_D.cpu().view(torch.int32), w_D.view(torch.int32))
        assert torch.equal(st.cpu(), w_st)


def test_shape_sweep_vs_oracle(oracle_lib):
    """Odd shapes: dimensions that are not multiples of 128 (or of 32), d_principle
    anywhere up to d, ef 1 (a 4-entry handoff under 16-entry heaps), heaps that are
    not powers of two, k from 1 to the whole row -- all bit for bit."""
    from pilotann_b200 import extension
    from helpers import make_problem
    g = torch.Generator().manual_seed(77)
    shapes = [(8, 4, 1, 1), (8, 8, 3, 5), (20, 12, 16, 10), (64, 16, 17, 1), (100, 64, 33, 40),
              (132, 128, 100, 25), (256, 64, 300, 50), (36, 36, 40, 160)]
    for d, d_p, ef, k in shapes:
        B = 24
        p = make_problem(n=3000, d=d, ratio=0.5, batch=B, n_init=32, seed=80 + d)
        full, q = p["full"], p["query"]
        ids = p["nodelist"][torch.randint(p["nodelist"].numel(), (B, 4 * ef), generator=g)]
        ids[torch.rand(B, 4 * ef, generator=g) < 0.15] = -1
        dist = ((q[:, :d_p].unsqueeze(1) - full[ids.clamp_min(0)][:, :, :d_p]) ** 2).sum(-1)
        dist[ids < 0] = float("inf")
        dist = dist.contiguous()
        reduced = p["storage"][:, :d_p].contiguous()
        nbr, row_of = extension.pack_graph(p["indptr"].cuda(), p["indices"].cuda(),
                                           p["mapping"].cuda(), reduced.size(0), 32)
        full_nbr = extension.pack_fullgraph(p["full_indptr"].cuda(), p["full_indices"].cuda(), 32)
        pool = extension.VisitedPool(full.size(0), 7)
        st = torch.zeros(B, 4, dtype=torch.int32, device="cuda")
        t_I, t_D = extension.refine(ids.cuda(), dist.cuda(), q.cuda(), full.cuda(), nbr, row_of,
                                    full_nbr, pool, ef, d_p, k=k, stats=st)
        torch.cuda.synchronize()
        w_I, w_D, w_st = oracle_lib.refine_ex(ids.clone(), dist.clone(), [p["indptr"], p["indices"]],
                                              [p["full_indptr"], p["full_indices"]], full, q, k, ef,
                                              d_p, gpu_order=True, with_stats=True)
        assert torch.equal(t_I.cpu(), w_I), (d, d_p, ef, k)
        assert torch.equal(t_D.cpu().view(torch.int32), w_D.view(torch.int32)), (d, d_p, ef, k)
        assert torch.equal(st.cpu(), w_st), (d, d_p, ef, k)


def test_three_warp_ctas_for_short_rows(oracle_lib):
    """Rows of at most 128 floats and more queries than nine per SM: the kernel runs
    with a heap warp and two gather warps (twelve CTAs per SM) instead of three or four.
    Same bits as the oracle, and as the same queries refined in small batches (which
    take the wider CTAs)."""
    from pilotann_b200 import extension
    from helpers import make_problem
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    B, d, d_p, ef, k = 9 * sms + 170, 64, 32, 24, 10
    g = torch.Generator().manual_seed(5)
    p = make_problem(n=3000, d=d, ratio=0.5, batch=B, n_init=32, seed=91)
    full, q = p["full"], p["query"]
    ids = p["nodelist"][torch.randint(p["nodelist"].numel(), (B, 4 * ef), generator=g)]
    dist = ((q[:, :d_p].unsqueeze(1) - full[ids][:, :, :d_p]) ** 2).sum(-1).contiguous()
    nbr, row_of = extension.pack_graph(p["indptr"].cuda(), p["indices"].cuda(), p["mapping"].cuda(),
                                       p["storage"].size(0), 32)
    full_nbr = extension.pack_fullgraph(p["full_indptr"].cuda(), p["full_indices"].cuda(), 32)
    assert extension.refine_wave(d) == 12 * sms and extension.refine_wave(768) == 7 * sms
    pool = extension.VisitedPool(full.size(0), B)
    st = torch.zeros(B, 4, dtype=torch.int32, device="cuda")
    args = (full.cuda(), nbr, row_of, full_nbr, pool, ef, d_p)
    t_I, t_D = extension.refine(ids.cuda(), dist.cuda(), q.cuda(), *args, k=k, stats=st)
    torch.cuda.synchronize()
    w_I, w_D, w_st = oracle_lib.refine_ex(ids.clone(), dist.clone(), [p["indptr"], p["indices"]],
                                          [p["full_indptr"], p["full_indices"]], full, q, k, ef,
                                          d_p, gpu_order=True, with_stats=True)
    assert torch.equal(t_I.cpu(), w_I)
    assert torch.equal(t_D.cpu().view(torch.int32), w_D.view(torch.int32))
    assert torch.equal(st.cpu(), w_st)
    s_I, s_D = extension.refine(ids[:200].cuda(), dist[:200].cuda(), q[:200].cuda(), *args, k=k)
    assert torch.equal(s_I, t_I[:200]) and torch.equal(s_D.view(torch.int32), t_D[:200].view(torch.int32))


def test_equal_distances_take_upstreams_sequence(oracle_lib):
    """Vectors on a coarse grid, many of them identical: equal distances everywhere.
    The shortcuts of the kernel (two-expansion stage without the open heap, seeds
    merged by selection and sort) give way to upstream's heap sequence wherever two
    keys that matter are equal -- same bits as the oracle, statistics included."""
    from pilotann_b200 import extension
    from helpers import make_problem
    g = torch.Generator().manual_seed(123)
    for d, d_p, ef, k, levels, dup in [(64, 32, 24, 10, 2.0, 6), (96, 32, 48, 10, 1.0, 3),
                                       (200, 64, 16, 5, 4.0, 10), (768, 128, 32, 10, 1.0, 4)]:
        B = 48
        p = make_problem(n=3000, d=d, ratio=0.5, batch=B, n_init=32, seed=300 + d)
        full = torch.round(p["full"] * levels) / levels
        full[torch.randperm(3000, generator=g)] = full.repeat_interleave(dup, 0)[:3000]
        full = full.contiguous()
        q = (torch.round(p["query"] * levels) / levels).contiguous()
        ids = p["nodelist"][torch.randint(p["nodelist"].numel(), (B, 4 * ef), generator=g)]
        ids[torch.rand(B, 4 * ef, generator=g) < 0.1] = -1
        dist = ((q[:, :d_p].unsqueeze(1) - full[ids.clamp_min(0)][:, :, :d_p]) ** 2).sum(-1)
        dist[ids < 0] = float("inf")
        dist = dist.contiguous()
        nbr, row_of = extension.pack_graph(p["indptr"].cuda(), p["indices"].cuda(), p["mapping"].cuda(),
                                           p["storage"].size(0), 32)
        full_nbr = extension.pack_fullgraph(p["full_indptr"].cuda(), p["full_indices"].cuda(), 32)
        pool = extension.VisitedPool(full.size(0), 16)
        graphs = ([p["indptr"], p["indices"]], [p["full_indptr"], p["full_indices"]])
        for stages_k in (None, k):
            st = torch.zeros(B, 4, dtype=torch.int32, device="cuda")
            t_I, t_D = extension.refine(ids.cuda(), dist.cuda(), q.cuda(), full.cuda(), nbr, row_of,
                                        full_nbr if stages_k else None, pool, ef, d_p, k=stages_k,
                                        stats=st)
            torch.cuda.synchronize()
            w_bI, w_bD = ids.clone(), dist.clone()
            w_I, w_D, w_st = oracle_lib.refine_ex(w_bI, w_bD, *graphs, full, q, k, ef, d_p, gpu_order=True,
                                                  stages=3 if stages_k else 2, with_stats=True)
            if stages_k is None:
                w_I, w_D, w_st = w_bI, w_bD, w_st[:, :2]
                st = st[:, :2]
            assert torch.equal(t_I.cpu(), w_I), (d, ef, stages_k)
            assert torch.equal(t_D.cpu().view(torch.int32), w_D.view(torch.int32)), (d, ef, stages_k)
            assert torch.equal(st.cpu(), w_st), (d, ef, stages_k)
        # the case is what it claims to be: equal distances among a query's candidates
        row = dist[0][ids[0] >= 0]
        assert row.unique().numel() < row.numel()


def test_replay_of_upstream_fixtures():
    """Outputs of upstream ``traverse_refine`` recorded by tests/golden/make_golden.py
    (CPU, no GPU involved), replayed through the refinement kernel without the
    upstream module: top-k, and the handoff rows the sub-graph stage leaves."""
    from pathlib import Path
    from pilotann_b200 import extension
    gold = torch.load(Path(__file__).parent / "golden" / "golden_cpu.pt")
    p = gold["problem"]
    n = p["full"].size(0)
    d_sub = p["storage"].size(1)
    nbr, row_of = extension.pack_graph(p["indptr"].cuda(), p["indices"].cuda(), p["mapping"].cuda(),
                                       p["storage"].size(0), 32)
    full_nbr = extension.pack_fullgraph(p["full_indptr"].cuda(), p["full_indices"].cuda(), 32)
    pool = extension.VisitedPool(n, 8)
    assert d_sub == p["full"].size(1)
    for ef, fx in gold["refine"].items():
        k = fx["out_I"].size(1)
        args = (fx["cand_I"].cuda(), fx["cand_D"].cuda(), p["query"].cuda(), p["full"].cuda(), nbr,
                row_of)
        t_I, t_D = extension.refine(*args, full_nbr, pool, ef, fx["d_principle"], k=k)
        s_I, s_D = extension.refine(*args, None, pool, ef, fx["d_principle"], k=None)
        torch.cuda.synchronize()
        assert (t_I.cpu() == fx["out_I"]).float().mean().item() >= 0.995, ef
        assert torch.allclose(t_D.cpu(), fx["out_D"], rtol=1e-5, atol=1e-6)
        assert (s_I.cpu() == fx["buffer_I"]).float().mean().item() >= 0.995
        fin = torch.isfinite(fx["buffer_D"])
        assert torch.equal(fin, torch.isfinite(s_D.cpu()))
        assert torch.allclose(s_D.cpu()[fin], fx["buffer_D"][fin], rtol=1e-5, atol=1e-6)
