"""The stage at the benchmark's shapes (1024 queries, d_principle 128, degree 32,
router entries, ef up to 256) on a graph small enough to build in seconds:
bit-exact parity with the oracle plus the size-independent properties that are
also checked where the oracle is too slow."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def big():
    from pilotann_b200 import layers, utils
    w = utils.WORKLOADS[2].scaled(60000, 1024)
    w = type(w)(**{**w.__dict__, "d_model": 256, "d_principle": 128, "entry_method": "router32x32"})
    x = utils.make_storage(w, device="cuda")
    g = torch.Generator().manual_seed(9)
    index = layers.IndexStaged(w.d_model, w.d_principle, w.sample_ratio, w.graph_method,
                               w.entry_method)
    index.train(x, generator=g, build_device="cuda")
    index.to("cuda", max_batch=1024, max_ef=256)
    return index, utils.make_queries(w), w


@pytest.mark.parametrize("ef", [128, 256])
def test_bench_shape_parity_and_properties(big, oracle_lib, ef):
    from pilotann_b200 import extension, _C
    index, q, w = big
    rot = extension.project(q.cuda(), index.VT_cuda)
    red = rot[:, :w.d_principle].contiguous()
    EP_I, EP_D = index.entry.search(red)
    B = q.size(0)
    oI = torch.empty(B, 4, ef, dtype=torch.int64, device="cuda")
    oD = torch.empty(B, 4, ef, device="cuda")
    st = torch.zeros(B, 4, dtype=torch.int32, device="cuda")
    extension.traverse_packed(oI, oD, index.packed_nbr, index.row_of, index.storage_cuda, red,
                              EP_I, EP_D, index.n_neighbors, stats=st)
    assert _C.lib().pa_device_status(1) == 0
    I, D = oI.cpu(), oD.cpu()
    wI, wD, wS = oracle_lib.traverse(index.subgraph.indptr, index.subgraph.indices, index.mapping,
                                     index.storage_cuda.cpu(), red.cpu(), EP_I.cpu(), EP_D.cpu(),
                                     index.n_neighbors, ef, with_stats=True)
    assert torch.equal(I, wI) and torch.equal(D, wD) and torch.equal(st.cpu(), wS)
    # properties that need no oracle
    valid = I >= 0
    assert (I[valid] < index.mapping.numel()).all()
    Dm = torch.where(valid, D, torch.full_like(D, float("inf")))
    assert (Dm[:, :, :-1] >= Dm[:, :, 1:]).all()              # each beam: worst -> best
    flat = I.reshape(B, -1)
    for b in range(0, B, 37):                                  # a node is reported once
        ids = flat[b][flat[b] >= 0]
        entries = EP_I[b].cpu()
        dup_budget = entries.numel() - entries.unique().numel()
        assert ids.numel() - ids.unique().numel() <= dup_budget
    # reported distances are the reduced-space distances of the reported ids
    rows = index.mapping[flat.clamp_min(0)]
    has_vec = (flat >= 0) & (rows >= 0)
    vec = index.storage_cuda.cpu()[rows.clamp_min(0)]
    exact = ((red.cpu().unsqueeze(1).double() - vec.double()) ** 2).sum(-1)
    got = D.reshape(B, -1).double()
    rel = ((got - exact).abs() / exact.clamp_min(1e-12))[has_vec]
    assert rel.max().item() <= 1e-5
