"""Side-by-side parity with the UPSTREAM CUDA kernels (compiled in place into
oracle/_ref): identical graph, projection, entries and queries go to both.

Gates: router ids and leaf ids bit-exact; reduced-space distances within 1e-5
relative; recall@k within +-0.002; final top-k ids identical for at least
99.5 % of queries -- or, where the upstream kernel does not reproduce ITSELF at
that level, for at least as many queries as two runs of the upstream kernel on
the same inputs agree on (plus a small margin).  The upstream traversal kernel
is not deterministic: its warps race on the bloom filter and the filter is
cleared without a barrier before the entries are inserted, so nodes get visited
twice or not at all depending on timing; the test measures that run-to-run
mismatch first.  The deterministic, bit-exact comparison is the one against the
CPU oracle (test_traverse_parity.py), which fixes one legal interleaving."""
import pytest
import torch

from helpers import make_problem, to_cuda, topk_ids

pytestmark = pytest.mark.gpu


def _ours(c, ef, n_nb, packed):
    from pilotann_b200 import extension
    B = c["query"].size(0)
    oI = torch.empty(B, 4, ef, dtype=torch.int64, device="cuda")
    oD = torch.empty(B, 4, ef, device="cuda")
    if packed:
        nbr, row_of = extension.pack_graph(c["indptr"], c["indices"], c["mapping"],
                                           c["storage"].size(0), n_nb)
        extension.traverse_packed(oI, oD, nbr, row_of, c["storage"], c["query"],
                                  c["initial_I"], c["initial_D"], n_nb)
    else:
        extension.traverse_cuda(oI, oD, c["indptr"], c["indices"], c["mapping"], c["storage"],
                                c["query"], c["initial_I"], c["initial_D"], n_nb)
    torch.cuda.synchronize()
    return oI.cpu(), oD.cpu()


def _theirs(ref_ext, c, ef, n_nb):
    B = c["query"].size(0)
    oI = torch.empty(B, 4, ef, dtype=torch.int64, device="cuda")
    oD = torch.empty(B, 4, ef, device="cuda")
    ref_ext.traverse_cuda(oI, oD, c["indptr"], c["indices"], c["mapping"], c["storage"],
                          c["query"], c["initial_I"], c["initial_D"], n_nb)
    torch.cuda.synchronize()
    return oI.cpu(), oD.cpu()


def _recall(top, truth):
    hit = sum(len(set(a) & set(b)) for a, b in zip(top, truth))
    return hit / sum(len(b) for b in truth)


# (law, d, sample ratio, ef, entries per query, k, graph flavour); the last two rows
# are the reduced-size shapes of the 96-d L2 configuration (shared random entries:
# 32 of them, heaps of 32) and of the 200-d out-of-distribution one (d_principle 96,
# half the nodes sampled, 32 leaves per router, top-100, ef 128, NSG-style graph)
CASES = [("fuzz", 64, 1.0, 64, 64, 10, "nsw"), ("powerlaw", 128, 0.25, 32, 64, 10, "nsw"),
         ("mixture", 64, 0.25, 32, 64, 10, "nsw"), ("powerlaw", 128, 0.25, 128, 64, 10, "nsw"),
         ("mixture", 64, 0.25, 32, 32, 10, "nsw"), ("powerlaw-ood", 96, 0.5, 128, 32, 100, "nsg")]


@pytest.mark.parametrize("law,d,ratio,ef,n_init,k,graph", CASES)
def test_traversal_vs_upstream_kernel(ref_ext, law, d, ratio, ef, n_init, k, graph):
    p = make_problem(n=20000, d=d, ratio=ratio, batch=512, n_init=n_init, seed=21, law=law,
                     build_device="cuda", graph=graph)
    c = to_cuda(p)
    # Upstream's kernel is racy: its own runs disagree with each other.  Five runs
    # give its run-to-run mismatch rate (mean over the ten pairs); the deterministic
    # kernel must look like one more such run: its mean mismatch against the five
    # stays within 1.5 x that rate plus four standard deviations of a rate estimated
    # on this many queries, and never less than the 0.5 % gate -- which is the whole
    # gate wherever upstream reproduces itself (rate 0, deviation 0).
    # 1.5 x: upstream's runs share their timing habits and sit closer to each other
    # than to any other legal interleaving (measured: 0.14 against 0.095 on the
    # uniform-random workload, where revisits are most frequent; equal elsewhere).
    runs = [_theirs(ref_ext, c, ef, 32) for _ in range(5)]
    tops = [topk_ids(*r, k) for r in runs]
    n_q = len(tops[0])

    def mismatch(a, b):
        return sum(x != y for x, y in zip(a, b)) / n_q

    pairs = [(i, j) for i in range(5) for j in range(i + 1, 5)]
    jitter = sum(mismatch(tops[i], tops[j]) for i, j in pairs) / len(pairs)
    sigma = (jitter * (1.0 - jitter) / n_q) ** 0.5
    theirs, t_top = runs[0], tops[0]
    truth = p["nodelist"][__import__("pilotann_b200").utils.ground_truth(
        p["query"], p["full"][p["nodelist"]], k)].tolist()
    t_recall = sum(_recall(tp, truth) for tp in tops) / 5
    for packed in (False, True):
        ours = _ours(c, ef, 32, packed)
        o_top = topk_ids(*ours, k)
        miss = sum(mismatch(o_top, tp) for tp in tops) / 5
        print(f"{law} d={d} ef={ef} packed={packed}: mismatch against upstream {miss:.4f} "
              f"(upstream run-to-run {jitter:.4f}, sigma {sigma:.4f})")
        assert miss <= max(0.005, 1.5 * jitter + 4.0 * sigma)
        # recall: never worse than upstream beyond +-0.002 (+ upstream's own noise: a
        # query whose top-k differs typically differs in about one of its k ids).  It
        # may be better by up to the mismatch rate: upstream's races insert some nodes
        # twice, which costs it heap slots and recall; the fixed schedule does not.
        delta = _recall(o_top, truth) - t_recall
        assert -(0.002 + (jitter + 4.0 * sigma) / k) <= delta <= 0.002 + jitter + 4.0 * sigma
        # distances of ids both sides report, within 1e-5 relative
        for b in range(0, len(t_top), 17):
            mine = dict(zip(ours[0][b].flatten().tolist(), ours[1][b].flatten().tolist()))
            for i, dist in zip(theirs[0][b].flatten().tolist(), theirs[1][b].flatten().tolist()):
                if i >= 0 and i in mine:
                    assert abs(mine[i] - dist) <= 1e-5 * abs(dist)


def test_routing_vs_upstream_kernel(ref_ext):
    from pilotann_b200 import extension
    g = torch.Generator().manual_seed(2)
    n, d = 20000, 128
    x = torch.nn.functional.normalize(torch.randn(n, d, generator=g), dim=-1)
    q = torch.nn.functional.normalize(torch.randn(777, d, generator=g), dim=-1).cuda()
    for n_r, n_l in ((16, 32), (64, 64)):
        rv = x[torch.randint(n, (n_r,), generator=g)].contiguous().cuda()
        en = torch.randint(n, (n_r, n_l), generator=g).cuda()
        ev = x[en.cpu()].contiguous().cuda()
        t_router, t_dist = ref_ext.routing_cuda(q, rv, en, ev)
        o_router, o_dist, o_ids = extension.routing_cuda(q, rv, en, ev, with_ids=True)
        torch.cuda.synchronize()
        assert torch.equal(o_router, t_router)
        assert torch.equal(o_ids, torch.index_select(en, 0, t_router))   # entry.py:86-88
        assert torch.allclose(o_dist, t_dist, rtol=1e-5, atol=0.0)


def test_golden_gpu_fixtures():
    """Outputs of the upstream kernels recorded on a B200
    (tests/golden/make_golden.py --gpu), replayed without the upstream module."""
    from pathlib import Path
    from pilotann_b200 import extension
    gdir = Path(__file__).parent / "golden"
    if not (gdir / "golden_gpu.pt").is_file():
        pytest.skip("golden_gpu.pt not recorded yet")
    fx = torch.load(gdir / "golden_gpu.pt")
    p = torch.load(gdir / "golden_cpu.pt")["problem"]
    c = {k: v.cuda() for k, v in p.items()}
    for ef, (tI, tD) in fx["traverse"].items():
        ours = _ours(c, ef, 32, packed=True)
        same = sum(a == b for a, b in zip(topk_ids(*ours, 10), topk_ids(tI, tD, 10)))
        assert same >= 0.95 * tI.size(0)       # 24 queries: at most one may differ
    for (n_r, n_l), r in fx["routing"].items():
        ev = p["full"][r["entry_nodes"]].contiguous()
        router, dist = extension.routing_cuda(c["query"], r["route_vectors"].cuda(),
                                              r["entry_nodes"].cuda(), ev.cuda())
        assert torch.equal(router.cpu(), r["router"])
        assert torch.allclose(dist.cpu(), r["distances"], rtol=1e-5, atol=0.0)


def test_pipeline_drop_in_vs_upstream_pipeline(ref_ext):
    """kernels.pipeline of this package, fed upstream's own traverse_refine as the
    consumer, against upstream's whole `pipeline` (extension/pipeline_cpu.cpp:32-145)
    on the same tensors: same recall within +-0.005, exact distances, and mostly
    the same ids (the GPU halves differ only through upstream's races)."""
    from pilotann_b200 import kernels, utils
    k, ef, chunk = 10, 64, 128
    p = make_problem(n=20000, d=96, ratio=0.25, batch=512, n_init=64, seed=33, law="powerlaw",
                     build_device="cuda")
    full_indptr, full_indices = utils.graph_init(p["full"].cuda(), "nsw", 32)
    c = to_cuda(p)
    graph = [full_indptr, full_indices]
    subgraph = [p["indptr"], p["indices"]]
    sub_cuda = [c["indptr"], c["indices"], c["mapping"]]
    d_p = 96      # no reduction in this test: the whole vector is "principal"
    args = dict(storage=p["full"], storage_cuda=c["storage"], query=p["query"],
                query_cuda=c["query"], initial_I=c["initial_I"], initial_D=c["initial_D"])
    import pilotann_b200
    try:
        pilotann_b200.set_refine(ref_ext.traverse_refine)     # upstream's own CPU consumer
        ours_I, ours_D = kernels.pipeline(graph=graph, subgraph=subgraph, subgraph_cuda=sub_cuda,
                                          n_neighbors=32, k=k, ef_search=ef, d_principle=d_p,
                                          chunk_size=chunk, **args)
    finally:
        pilotann_b200.set_refine("gpu")
    # and with this package's own consumer (the refinement kernel): the whole search
    # on the device
    gpu_I, gpu_D = kernels.pipeline(graph=graph, subgraph=subgraph, subgraph_cuda=sub_cuda,
                                    n_neighbors=32, k=k, ef_search=ef, d_principle=d_p,
                                    chunk_size=chunk, **args)
    def upstream():
        return ref_ext.pipeline(graph, subgraph, sub_cuda, args["storage"], args["storage_cuda"],
                                args["query"], args["query_cuda"], args["initial_I"],
                                args["initial_D"], 32, ef, d_p, k, chunk)

    def mismatch(a, b):
        return 1.0 - (a.sort(dim=1).values == b.sort(dim=1).values).all(dim=1).float().mean().item()

    # upstream's GPU half is racy: four runs give its own run-to-run mismatch; this
    # stage must look like one more run (see test_traversal_vs_upstream_kernel)
    theirs = [upstream()[0] for _ in range(4)]
    pairs = [(i, j) for i in range(4) for j in range(i + 1, 4)]
    jitter = sum(mismatch(theirs[i], theirs[j]) for i, j in pairs) / len(pairs)
    sigma = (jitter * (1.0 - jitter) / ours_I.size(0)) ** 0.5
    miss = sum(mismatch(ours_I, th) for th in theirs) / 4
    truth = utils.ground_truth(p["query"], p["full"], k)
    r_ours = utils.recall(ours_I, truth)
    r_theirs = sum(utils.recall(th, truth) for th in theirs) / 4
    print(f"pipeline recall ours {r_ours:.4f} upstream {r_theirs:.4f}, top-{k} mismatch {miss:.4f} "
          f"(upstream run-to-run {jitter:.4f}, sigma {sigma:.4f})")
    assert abs(r_ours - r_theirs) <= 0.005
    assert miss <= max(0.005, 1.5 * jitter + 4.0 * sigma)
    # GPU refinement against CPU refinement on the same (deterministic) handoff
    same = 1.0 - mismatch(gpu_I, ours_I)
    print(f"GPU-refined top-{k} rows equal to CPU-refined ones: {same:.4f}")
    assert same >= 0.995
    assert abs(utils.recall(gpu_I, truth) - r_ours) <= 0.002
    exact = torch.cdist(p["query"].unsqueeze(1), p["full"][ours_I]).squeeze(1).square()
    assert torch.allclose(ours_D, exact, atol=1e-3)
