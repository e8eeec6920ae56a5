"""Reduced-size versions of the other benchmark configurations, end to end on a
GPU: config 1 (clustered 96-d, 'random32' entries, top-10) and config 3 (200-d,
out-of-distribution queries, NSG-style graph, 50 % sample, router32x32, top-100).
The handoff must equal the oracle's bit for bit; recall is measured through the
oracle's restatement of the CPU refinement."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _build(cfg, n, n_q, **over):
    from pilotann_b200 import layers, utils
    w = utils.WORKLOADS[cfg].scaled(n, n_q)
    w = type(w)(**{**w.__dict__, **over})
    x = utils.make_storage(w, device="cuda")
    g = torch.Generator().manual_seed(4000 + cfg)
    index = layers.IndexStaged(w.d_model, w.d_principle, w.sample_ratio, w.graph_method,
                               w.entry_method)
    index.train(x, generator=g, build_device="cuda")
    index.to("cuda", max_batch=n_q, max_ef=256)
    return index, x.cpu(), utils.make_queries(w), w


def _refine_with(oracle_lib):
    def refine(out_I, out_D, buf_I, buf_D, ini_I, ini_D, subgraph, fullgraph, storage, query,
               ef_search, d_principle):
        I, D = oracle_lib.refine(buf_I, buf_D, subgraph, fullgraph, storage, query.contiguous(),
                                 out_I.size(1), ef_search, d_principle)
        out_I.copy_(I); out_D.copy_(D)
    return refine


@pytest.mark.parametrize("cfg,ef,k,floor", [(1, 32, 10, 0.85), (3, 128, 100, 0.80)])
def test_config_end_to_end(oracle_lib, cfg, ef, k, floor):
    from pilotann_b200 import extension, utils
    index, x, q, w = _build(cfg, 30000 if cfg == 1 else 40000, 256)
    assert w.top_k == k
    hI, hD, rot = index.search_candidates(q, ef)
    # handoff == oracle on the stage's own projection and entries
    red = rot[:, :w.d_principle].contiguous().cuda()
    EP_I, EP_D = index.entry.search(red)
    want = oracle_lib.traverse(index.subgraph.indptr, index.subgraph.indices, index.mapping,
                               index.storage_cuda.cpu(), red.cpu(), EP_I.cpu(), EP_D.cpu(),
                               index.n_neighbors, ef)
    assert torch.equal(hI.view(-1, 4, ef), want[0]) and torch.equal(hD.view(-1, 4, ef), want[1])
    # config 1 uses one shared entry list for every query (entry.py:70-77)
    if w.entry_method.startswith("random"):
        assert (EP_I == EP_I[0]).all() and EP_I.size(1) == 32
    I, D = index.search(q, k=k, ef_search=ef, chunk_size=64, refine=_refine_with(oracle_lib))
    truth = utils.ground_truth(q, x, k)
    assert utils.recall(I, truth) >= floor
    exact = torch.cdist(q.unsqueeze(1), x[I]).squeeze(1).square()
    assert torch.allclose(D, exact, atol=1e-3)
    # the same search finished on the device (refinement kernel): the oracle's
    # restatement in that kernel's summation order, bit for bit, and the recall of
    # the CPU-refined run
    gI, gD = index.search(q, k, ef)
    w_I, w_D = oracle_lib.refine_ex(hI.clone(), hD.clone(),
                                    [index.subgraph.indptr, index.subgraph.indices],
                                    [index.fullgraph.indptr, index.fullgraph.indices],
                                    index.storage, rot.clone(), k, ef, w.d_principle, gpu_order=True)
    assert torch.equal(gI, w_I) and torch.equal(gD.view(torch.int32), w_D.view(torch.int32))
    assert abs(utils.recall(gI, truth) - utils.recall(I, truth)) <= 0.002
