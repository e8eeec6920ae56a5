"""GPU parity of entry routing and query projection against the CPU oracle."""
import pytest
import torch

pytestmark = pytest.mark.gpu

RTOL = 1e-5     # reduced-space distances: 1e-5 relative


def _tables(n, d, n_r, n_l, seed):
    g = torch.Generator().manual_seed(seed)
    x = 2.0 * (torch.rand(n, d, generator=g) - 0.5)
    rv = x[torch.randint(n, (n_r,), generator=g)].contiguous()
    en = torch.randint(n, (n_r, n_l), generator=g)
    return x, rv, en, x[en].contiguous()


@pytest.mark.parametrize("n_r,n_l,d,B", [(8, 32, 64, 1), (16, 64, 96, 333), (32, 32, 96, 512),
                                         (64, 64, 128, 1024), (64, 64, 200, 257)])
def test_routing_matches_oracle(oracle_lib, n_r, n_l, d, B):
    from pilotann_b200 import extension
    x, rv, en, ev = _tables(20000, d, n_r, n_l, seed=n_r + d)
    g = torch.Generator().manual_seed(B)
    q = 2.0 * (torch.rand(B, d, generator=g) - 0.5)
    router, dist, ids = extension.routing_cuda(q.cuda(), rv.cuda(), en.cuda(), ev.cuda(),
                                               with_ids=True)
    w_router, w_dist, w_ids = oracle_lib.route(q, rv, en, ev)
    assert torch.equal(router.cpu(), w_router)              # FES entry ids: bit-exact
    assert torch.equal(ids.cpu(), w_ids)
    assert torch.allclose(dist.cpu(), w_dist, rtol=RTOL, atol=0.0)


def test_routing_near_ties_resolved_exactly(oracle_lib):
    """Routers that are (almost) equidistant from the query: the choice must be
    the exact-arithmetic one, ties to the lowest index."""
    from pilotann_b200 import extension
    d, n_r, n_l = 64, 16, 32
    g = torch.Generator().manual_seed(0)
    q = torch.randn(200, d, generator=g)
    rv = torch.randn(n_r, d, generator=g)
    rv[5] = rv[2]                                # exact duplicate -> tie
    rv[9] = rv[2] + 1e-7 * torch.randn(d, generator=g)
    q[:50] = rv[2] + 0.1 * torch.randn(50, d, generator=g)
    en = torch.randint(1000, (n_r, n_l), generator=g)
    ev = torch.randn(n_r, n_l, d, generator=g)
    router, _, _ = extension.routing_cuda(q.cuda(), rv.cuda(), en.cuda(), ev.cuda(), with_ids=True)
    assert torch.equal(router.cpu(), oracle_lib.route(q, rv, en, ev)[0])


def test_routing_against_torch_reference():
    """The check upstream's own test makes (test/kernel/test_routing.py:70-85)."""
    from pilotann_b200 import extension
    x, rv, en, ev = _tables(30000, 128, 16, 64, seed=5)
    q = 2.0 * (torch.rand(700, 128, generator=torch.Generator().manual_seed(1)) - 0.5)
    router, dist = extension.routing_cuda(q.cuda(), rv.cuda(), en.cuda(), ev.cuda())
    indices = torch.argmin(torch.cdist(q, rv, p=2.0), dim=-1)
    target = torch.cdist(q.unsqueeze(1), x[en[indices]]).square().squeeze(1)
    assert torch.equal(router.cpu(), indices)
    assert torch.allclose(dist.cpu(), target, atol=1e-3)


def test_routing_rejections():
    from pilotann_b200 import extension
    x, rv, en, ev = _tables(1000, 64, 8, 48, seed=1)
    q = torch.rand(4, 64)
    with pytest.raises(RuntimeError):          # routing_cuda.cu:90
        extension.routing_cuda(q.cuda(), rv.cuda(), en.cuda(), ev.cuda())
    with pytest.raises(RuntimeError):          # CHECK_CUDA
        extension.routing_cuda(q, rv.cuda(), en.cuda(), ev.cuda())


def test_random_entries_match_oracle(oracle_lib):
    from pilotann_b200 import extension
    x, _, en, ev = _tables(5000, 96, 1, 64, seed=2)
    q = 2.0 * (torch.rand(100, 96, generator=torch.Generator().manual_seed(4)) - 0.5)
    dist = extension.entry_distances(q.cuda(), ev[0].contiguous().cuda())
    _, want, _ = oracle_lib.route(q, ev[0, :1].contiguous(), en, ev)
    assert torch.allclose(dist.cpu(), want, rtol=RTOL, atol=0.0)


@pytest.mark.parametrize("B,d,d_out", [(1, 64, 64), (100, 96, 64), (1024, 768, 768),
                                       (513, 200, 96), (64, 768, 128)])
def test_projection_matches_oracle(oracle_lib, B, d, d_out):
    from pilotann_b200 import extension
    g = torch.Generator().manual_seed(B + d)
    q = torch.nn.functional.normalize(torch.randn(B, d, generator=g), dim=-1)
    V, _ = torch.linalg.qr(torch.randn(d, d, generator=g, dtype=torch.float64))
    VT = V.T.float().contiguous()
    got = extension.project(q.cuda(), VT.cuda(), d_out).cpu()
    want = oracle_lib.project(q, VT, d_out)
    # coordinates of a unit vector in an orthonormal basis: absolute error
    # relative to the row norm (1.0)
    assert (got - want).abs().max().item() <= 2e-6
    # what matters downstream: reduced-space distances within 1e-5 relative
    x = torch.nn.functional.normalize(torch.randn(50, d, generator=g), dim=-1) @ VT.T[:, :d_out]
    dg = torch.cdist(got.double(), x.double()).square()
    dw = torch.cdist(want.double(), x.double()).square()
    assert ((dg - dw).abs() / dw).max().item() <= RTOL
