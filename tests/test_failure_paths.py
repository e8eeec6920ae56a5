"""Failure paths that must leave the GPU usable: a bounded wait that runs out,
and queries holding NaN / Inf.  Nothing here faults, traps or hangs the device:
the wait under test polls sixteen times on a barrier phase nobody completes and
returns; the NaN queries only exercise index clamping."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _routing_case(seed=3, n=5000, d=128, n_r=16, n_l=32, batch=200):
    g = torch.Generator().manual_seed(seed)
    x = torch.nn.functional.normalize(torch.randn(n, d, generator=g), dim=-1)
    q = torch.nn.functional.normalize(torch.randn(batch, d, generator=g), dim=-1)
    rv = x[torch.randint(n, (n_r,), generator=g)].contiguous()
    en = torch.randint(n, (n_r, n_l), generator=g)
    ev = x[en].contiguous()
    return q, rv, en, ev


def test_bounded_wait_runs_out_sets_the_status_and_the_device_stays_usable(oracle_lib):
    from pilotann_b200 import _C, extension
    lib = _C.lib()
    lib.pa_device_status(1)
    assert lib.pa_device_status(0) == 0
    _C.check(lib.pa_selftest_bounded_wait(0))
    assert lib.pa_device_status(0) == 1          # reported, not reset
    # while the word is set, routing distrusts tensor-core scores and measures every
    # router exactly: same answer as always
    q, rv, en, ev = _routing_case()
    router, dist, ids = extension.routing_cuda(q.cuda(), rv.cuda(), en.cuda(), ev.cuda(),
                                               with_ids=True)
    w_router, w_dist, w_ids = oracle_lib.route(q, rv, en, ev)
    assert torch.equal(router.cpu(), w_router) and torch.equal(ids.cpu(), w_ids)
    assert torch.equal(dist.cpu(), w_dist)
    assert lib.pa_device_status(1) == 1          # read and reset
    assert lib.pa_device_status(0) == 0
    # the tensor-core projection runs as before
    g = torch.Generator().manual_seed(0)
    V, _ = torch.linalg.qr(torch.randn(128, 128, generator=g, dtype=torch.float64))
    VT = V.T.float().contiguous()
    rot = extension.project(q.cuda(), VT.cuda())
    assert (rot.cpu() - oracle_lib.project(q, VT)).abs().max().item() < 1e-5
    assert lib.pa_device_status(0) == 0


def test_nan_and_inf_queries_route_to_a_valid_router():
    """Upstream picks the router with argmin, which returns an index in range
    whatever the distances are; here a query without any finite distance goes to
    router 0.  The ids gathered for it are that router's leaves."""
    from pilotann_b200 import extension
    q, rv, en, ev = _routing_case(seed=4)
    q[3, 7] = float("nan")
    q[11] = float("inf")
    q[12, 0] = float("-inf")
    for with_ws in (True, False):
        if with_ws:
            router, dist, ids = extension.routing_cuda(q.cuda(), rv.cuda(), en.cuda(), ev.cuda(),
                                                       with_ids=True)
        else:       # a single implicit router: the 'random' entry method
            dist = extension.entry_distances(q.cuda(), ev[0].contiguous().cuda())
            router = torch.zeros(q.size(0), dtype=torch.int64)
            ids = None
        torch.cuda.synchronize()
        router = router.cpu()
        assert ((router >= 0) & (router < rv.size(0))).all()
        if ids is not None:
            assert torch.equal(ids.cpu(), en[router])
            assert router[3] == 0 and router[11] == 0 and router[12] == 0
        bad = torch.tensor([3, 11, 12])
        assert not torch.isfinite(dist.cpu()[bad]).any()
        good = torch.ones(q.size(0), dtype=torch.bool)
        good[bad] = False
        assert torch.isfinite(dist.cpu()[good]).all()
