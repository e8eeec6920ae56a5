"""GPU parity of the traversal kernels (both index layouts) against the CPU
oracle: ids, distances, per-query counters and bloom occupancy must be equal
bit for bit, on seeded inputs the oracle finishes in seconds."""
import pytest
import torch

from helpers import make_problem, to_cuda

pytestmark = pytest.mark.gpu


def run_gpu(p, ef, layout, stats=True):
    from pilotann_b200 import extension
    c = to_cuda(p)
    B = c["query"].size(0)
    oI = torch.full((B, 4, ef), -7, dtype=torch.int64, device="cuda")
    oD = torch.full((B, 4, ef), -7.0, device="cuda")
    st = torch.zeros(B, 4, dtype=torch.int32, device="cuda") if stats else None
    if layout == "csr":
        extension.traverse_cuda(oI, oD, c["indptr"], c["indices"], c["mapping"], c["storage"],
                                c["query"], c["initial_I"], c["initial_D"], p["n_neighbors"],
                                stats=st)
    else:
        nbr, row_of = extension.pack_graph(c["indptr"], c["indices"], c["mapping"],
                                           c["storage"].size(0), p["n_neighbors"])
        extension.traverse_packed(oI, oD, nbr, row_of, c["storage"], c["query"],
                                  c["initial_I"], c["initial_D"], p["n_neighbors"], stats=st)
    torch.cuda.synchronize()
    return oI.cpu(), oD.cpu(), None if st is None else st.cpu()


def run_oracle(oracle, p, ef):
    return oracle.traverse(p["indptr"], p["indices"], p["mapping"], p["storage"], p["query"],
                           p["initial_I"], p["initial_D"], p["n_neighbors"], ef, with_stats=True)


def assert_same(got, want):
    gI, gD, gS = got
    wI, wD, wS = want
    assert torch.equal(gI, wI), f"{(gI != wI).any(-1).any(-1).sum().item()} queries differ in ids"
    assert torch.equal(gD.view(torch.int32), wD.view(torch.int32)), "distance bits differ"
    if gS is not None:
        assert torch.equal(gS, wS), "rounds / expansions / evaluations / bloom bits differ"


@pytest.mark.parametrize("layout", ["csr", "packed"])
@pytest.mark.parametrize("ef", [1, 16, 32, 48, 64, 100, 128, 256, 300])
def test_unsampled_graph(oracle_lib, layout, ef):
    p = make_problem(n=4096, d=64, batch=96, n_init=32, seed=1)
    assert_same(run_gpu(p, ef, layout), run_oracle(oracle_lib, p, ef))


@pytest.mark.parametrize("layout", ["csr", "packed"])
@pytest.mark.parametrize("d,ef", [(32, 32), (96, 32), (128, 64), (200, 16), (768, 32)])
def test_sampled_graph_dims(oracle_lib, layout, d, ef):
    # 25 % sample: most random entries fall outside the sample (empty rows)
    p = make_problem(n=6000, d=d, ratio=0.25, batch=64, n_init=64, seed=2)
    assert_same(run_gpu(p, ef, layout), run_oracle(oracle_lib, p, ef))


@pytest.mark.parametrize("layout", ["csr", "packed"])
def test_degree_64(oracle_lib, layout):
    p = make_problem(n=3000, d=64, n_nb=64, ratio=0.5, batch=48, n_init=32, seed=3)
    for ef in (32, 128):
        assert_same(run_gpu(p, ef, layout), run_oracle(oracle_lib, p, ef))


@pytest.mark.parametrize("layout", ["csr", "packed"])
def test_entries_with_pads_duplicates_and_inexact_distances(oracle_lib, layout):
    p = dict(make_problem(n=4096, d=64, ratio=0.5, batch=64, n_init=40, seed=4,
                          exact_entries=False))
    I = p["initial_I"].clone()
    I[:, 3] = -1                     # pad entry
    I[:, 5] = I[:, 4]                # duplicate entry
    I[7, :] = -1                     # a query with no entry at all
    I[9, 1:] = -1                    # a query with a single entry
    p["initial_I"] = I
    D = p["initial_D"].clone()
    D[11, 0] = float("inf")          # an entry that can never be admitted
    p["initial_D"] = D
    for ef in (16, 64):
        assert_same(run_gpu(p, ef, layout), run_oracle(oracle_lib, p, ef))


@pytest.mark.parametrize("layout", ["csr", "packed"])
def test_ragged_and_empty_rows(oracle_lib, layout):
    """General CSR: rows shorter than n_neighbors, rows holding only pads, and
    sampled nodes with an empty row."""
    base = make_problem(n=2048, d=32, batch=32, n_init=32, seed=5)
    n_nb = 32
    adj = base["indices"].view(-1, n_nb).clone()
    g = torch.Generator().manual_seed(9)
    lengths = torch.randint(0, n_nb + 1, (adj.size(0),), generator=g)
    lengths[::5] = n_nb
    adj[1::7] = -1                                     # rows of pads only (kept full length)
    lengths[1::7] = n_nb
    rows = [adj[u, :lengths[u]] for u in range(adj.size(0))]
    indptr = torch.zeros(adj.size(0) + 1, dtype=torch.long)
    indptr[1:] = torch.cumsum(lengths, 0)
    p = dict(base)
    p["indptr"], p["indices"] = indptr, torch.cat(rows).contiguous()
    for ef in (16, 40):
        assert_same(run_gpu(p, ef, layout), run_oracle(oracle_lib, p, ef))


def test_few_entries_and_tiny_batches(oracle_lib):
    for batch, n_init in ((1, 1), (3, 2), (5, 7)):
        p = make_problem(n=2048, d=64, batch=batch, n_init=n_init, seed=6)
        for layout in ("csr", "packed"):
            assert_same(run_gpu(p, 32, layout), run_oracle(oracle_lib, p, 32))


def test_empty_batch_and_rejections():
    from pilotann_b200 import extension
    p = to_cuda(make_problem(n=2048, d=64, batch=4, n_init=8, seed=6))
    oI = torch.empty(0, 4, 16, dtype=torch.int64, device="cuda")
    oD = torch.empty(0, 4, 16, device="cuda")
    extension.traverse_cuda(oI, oD, p["indptr"], p["indices"], p["mapping"], p["storage"],
                            p["query"][:0], p["initial_I"][:0], p["initial_D"][:0], 32)
    oI = torch.empty(4, 4, 16, dtype=torch.int64, device="cuda")
    oD = torch.empty(4, 4, 16, device="cuda")
    args = (p["indptr"], p["indices"], p["mapping"], p["storage"], p["query"], p["initial_I"],
            p["initial_D"])
    with pytest.raises(RuntimeError):      # traverse_cuda.cu:281
        extension.traverse_cuda(oI, oD, *args, 48)
    with pytest.raises(RuntimeError):      # traverse_cuda.cu:280
        extension.traverse_cuda(oI, oD, *args, 96)
    with pytest.raises(RuntimeError):      # traverse_cuda.cu:276
        extension.traverse_cuda(oI[:, :2].contiguous(), oD[:, :2].contiguous(), *args, 32)
    with pytest.raises(RuntimeError):      # CHECK_CUDA dtype
        extension.traverse_cuda(oI.int(), oD, *args, 32)
    big_I = torch.empty(4, 4, 2049, dtype=torch.int64, device="cuda")
    with pytest.raises(RuntimeError):      # traverse_cuda.cu:313
        extension.traverse_cuda(big_I, torch.empty(4, 4, 2049, device="cuda"), *args, 32)


def test_ef_beyond_256_pads_tail(oracle_lib):
    p = make_problem(n=4096, d=64, batch=16, n_init=32, seed=1)
    gI, gD, _ = run_gpu(p, 300, "packed")
    assert (gI[:, :, 256:] == -1).all() and torch.isinf(gD[:, :, 256:]).all()
    assert (gD[:, :, 256:] < 0).all()      # (-1, -inf) tail


def test_unpackable_graph_is_refused():
    from pilotann_b200 import extension
    p = make_problem(n=2048, d=32, batch=4, n_init=8, seed=5)
    mapping = p["mapping"].clone()
    mapping[0] = -1                        # node 0 keeps its neighbours but loses its row
    with pytest.raises(RuntimeError):
        extension.pack_graph(p["indptr"].cuda(), p["indices"].cuda(), mapping.cuda(),
                             p["storage"].size(0), 32)


def test_repeatable():
    p = make_problem(n=4096, d=64, ratio=0.5, batch=64, n_init=32, seed=8)
    a = run_gpu(p, 64, "packed")
    b = run_gpu(p, 64, "packed")
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1]) and torch.equal(a[2], b[2])


def test_drop_in_call_switches_to_the_packed_form(oracle_lib):
    """``traverse_cuda`` with the same graph tensors again: packed on the second
    call, identical results on every call, CSR again after an in-place change."""
    from pilotann_b200 import extension
    p = make_problem(n=3000, d=64, batch=32, ratio=0.5, seed=77)
    c = to_cuda(p)
    want = run_oracle(oracle_lib, p, 48)
    extension._pack_cache.clear()
    outs = []
    for call in range(3):
        oI = torch.full((32, 4, 48), -7, dtype=torch.int64, device="cuda")
        oD = torch.full((32, 4, 48), -7.0, device="cuda")
        st = torch.zeros(32, 4, dtype=torch.int32, device="cuda")
        extension.traverse_cuda(oI, oD, c["indptr"], c["indices"], c["mapping"], c["storage"],
                                c["query"], c["initial_I"], c["initial_D"], 32, stats=st)
        torch.cuda.synchronize()
        outs.append((oI.cpu(), oD.cpu(), st.cpu()))
        entry = next(iter(extension._pack_cache.values()))
        assert (entry["packed"] is not None) == (call >= 1)
    for got in outs:
        assert_same(got, want)
    c["indices"].add_(0)                       # in-place op: version counter moves
    oI = torch.empty(32, 4, 48, dtype=torch.int64, device="cuda")
    oD = torch.empty(32, 4, 48, device="cuda")
    extension.traverse_cuda(oI, oD, c["indptr"], c["indices"], c["mapping"], c["storage"],
                            c["query"], c["initial_I"], c["initial_D"], 32)
    assert next(iter(extension._pack_cache.values()))["packed"] is None
    torch.cuda.synchronize()
    assert torch.equal(oI.cpu(), want[0])
