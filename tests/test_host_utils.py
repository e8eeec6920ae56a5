"""Host-side build helpers (CPU): seeded workloads, SVD rotation, graph builder,
sampling, router tables, recall.  Small sizes; everything here runs without a GPU."""
import pytest
import torch

from pilotann_b200 import utils


def test_workloads_are_seeded_and_unit_norm():
    for cfg in (1, 2, 3):
        w = utils.WORKLOADS[cfg].scaled(2000, 64)
        a, b = utils.make_storage(w), utils.make_storage(w)
        assert torch.equal(a, b) and a.shape == (2000, w.d_model) and a.dtype == torch.float32
        assert torch.allclose(a.norm(dim=1), torch.ones(2000), atol=1e-5)
        q = utils.make_queries(w)
        assert q.shape == (64, w.d_model) and torch.equal(q, utils.make_queries(w))
        assert not torch.equal(q[:8], a[:8])          # queries are fresh draws
    assert utils.WORKLOADS[2].d_principle == 128 and utils.WORKLOADS[2].entry_method == "router64x64"
    assert utils.WORKLOADS[3].ood and utils.WORKLOADS[3].top_k == 100


def test_powerlaw_spectrum_decays():
    w = utils.WORKLOADS[2].scaled(4000, 8)
    x = utils.make_storage(w).double()
    ev = torch.linalg.eigvalsh(x.T @ x / x.size(0)).flip(0)
    assert ev[0] > 5 * ev[63] > 5 * ev[511] * 0.5      # ~1/i decay under the rotation


def test_svd_rotation_is_orthogonal_and_ordered():
    g = torch.Generator().manual_seed(3)
    x = torch.randn(3000, 24, generator=g) * torch.linspace(3.0, 0.1, 24)
    xr, V = utils.svd(x)
    assert torch.allclose(V.T @ V, torch.eye(24), atol=1e-4)
    assert torch.allclose(xr, x @ V, atol=1e-4)
    var = xr.var(dim=0)
    assert torch.all(var[:-1] >= var[1:] * 0.999)     # principal axes first


def test_ground_truth_and_recall():
    g = torch.Generator().manual_seed(4)
    x = torch.randn(500, 16, generator=g)
    q = x[:10] + 1e-3
    truth = utils.ground_truth(q, x, 5)
    assert torch.equal(truth[:, 0], torch.arange(10))
    assert utils.recall(truth, truth) == 1.0
    half = truth.clone()
    half[:, 1::2] = -1
    assert abs(utils.recall(half, truth) - 0.6) < 1e-6


def test_graph_builder_rows_are_valid_and_reach_true_neighbours():
    g = torch.Generator().manual_seed(5)
    x = torch.nn.functional.normalize(torch.randn(1500, 16, generator=g), dim=1)
    indptr, indices = utils.graph_init(x, "nsw", 32)
    assert indptr.dtype == indices.dtype == torch.int64
    assert torch.equal(indptr, torch.arange(1501) * 32)
    rows = indices.view(1500, 32)
    assert rows.max() < 1500 and rows.min() >= -1
    assert not (rows == torch.arange(1500).unsqueeze(1)).any()          # no self loops
    for r in rows[:50]:                                                   # no duplicates in a row
        v = r[r >= 0]
        assert v.unique().numel() == v.numel()
    nearest = utils.ground_truth(x, x, 2)[:, 1]                           # true nearest neighbour
    assert ((rows == nearest.unsqueeze(1)).any(dim=1)).float().mean() > 0.95


def test_sampling_and_subgraph_layout():
    g = torch.Generator().manual_seed(6)
    x = torch.nn.functional.normalize(torch.randn(2000, 16, generator=g), dim=1)
    indptr, indices = utils.graph_init(x, "nsw", 32)
    sub_indptr, sub_indices, nodelist, mapping = utils.subgraph_init(
        indptr, indices, x, "nsw", n_samples=500, n_neighbors=32, generator=g)
    assert 500 <= nodelist.numel() < 900 and torch.equal(nodelist, nodelist.sort().values)
    assert torch.equal(mapping[nodelist], torch.arange(nodelist.numel()))
    assert (mapping >= 0).sum() == nodelist.numel()
    lengths = sub_indptr[1:] - sub_indptr[:-1]
    assert torch.all(lengths[nodelist] == 32) and lengths.sum() == 32 * nodelist.numel()
    ids = sub_indices[sub_indices >= 0]
    assert torch.all(mapping[ids] >= 0)                                   # neighbours are sampled nodes


def test_router_tables_shapes_and_guard():
    g = torch.Generator().manual_seed(7)
    x = torch.nn.functional.normalize(torch.randn(3000, 16, generator=g), dim=1)
    out = utils.router_init(x, None, 4, 32, generator=g)
    route_vectors, entry_nodes = out[0], out[1]
    assert route_vectors.shape == (4, 16) and entry_nodes.shape == (4, 32)
    assert entry_nodes.min() >= 0 and entry_nodes.max() < 3000
    for leaves in entry_nodes:                                            # no repeats within a router
        assert leaves.unique().numel() == 32
    with pytest.raises(ValueError):
        utils.router_init(x[:100], None, 4, 32, generator=g)              # too few vectors
