"""The allocation-free entry point ``pa_search_reduced_noalloc``.

It exists for callers that cannot allocate device memory -- a process whose
memory pool owns the whole GPU, or a thread that must not stall the device with
an allocation -- and keeps its intermediates in a static device array.  This
test calls it through the C ABI twice in a row with different inputs and checks
each result, bit for bit, against the two existing entry points it combines
(``pa_route`` then ``pa_traverse_packed``); the second call would expose
anything left behind in the shared array by the first.  Collected last on
purpose (file name), so a failure here cannot hide the other tests.
"""
import pytest
import torch

from helpers import make_problem, to_cuda

pytestmark = pytest.mark.gpu


def _tables(p, n_r, n_l, seed):
    g = torch.Generator().manual_seed(seed)
    n = p["full"].size(0)
    rv = p["full"][torch.randint(n, (n_r,), generator=g)].contiguous().cuda()
    en = torch.randint(n, (n_r, n_l), generator=g)
    ev = p["full"][en].contiguous().cuda()
    return rv, en.cuda(), ev


def _expected(c, nbr, row_of, rv, en, ev, query, ef):
    from pilotann_b200 import extension
    _, EP_D, EP_I = extension.routing_cuda(query, rv, en, ev, with_ids=True)
    oI = torch.empty(query.size(0), 4, ef, dtype=torch.int64, device="cuda")
    oD = torch.empty(query.size(0), 4, ef, device="cuda")
    extension.traverse_packed(oI, oD, nbr, row_of, c["storage"], query, EP_I, EP_D, 32)
    torch.cuda.synchronize()
    return oI, oD


def test_two_calls_in_a_row_match_the_allocating_path():
    from pilotann_b200 import extension
    p = make_problem(n=6000, d=64, ratio=0.5, batch=200, n_init=32, seed=31)
    c = to_cuda(p)
    nbr, row_of = extension.pack_graph(c["indptr"], c["indices"], c["mapping"],
                                       c["storage"].size(0), 32)
    # first call: 200 queries, 16 routers x 64 leaves, ef 48
    # second call: fewer queries, other tables, other ef -> other scratch extent
    calls = [(c["query"], _tables(p, 16, 64, 1), 48),
             (c["query"][50:170].contiguous(), _tables(p, 8, 32, 2), 32)]
    outputs = []
    for query, (rv, en, ev), ef in calls:                 # the two calls, back to back
        oI = torch.full((query.size(0), 4, ef), -9, dtype=torch.int64, device="cuda")
        oD = torch.full((query.size(0), 4, ef), -9.0, device="cuda")
        extension.search_reduced_noalloc(oI, oD, nbr, row_of, c["storage"], query, rv, en, ev, 32)
        outputs.append((oI, oD))
    torch.cuda.synchronize()
    for (query, (rv, en, ev), ef), (oI, oD) in zip(calls, outputs):
        wI, wD = _expected(c, nbr, row_of, rv, en, ev, query, ef)
        assert torch.equal(oI, wI)
        assert torch.equal(oD.view(torch.int32), wD.view(torch.int32))
        assert (oI[:, :, -1] >= 0).all()                   # real results, not fill values


def test_shared_entry_list_variant():
    from pilotann_b200 import extension
    p = make_problem(n=6000, d=64, ratio=0.5, batch=64, n_init=32, seed=31)
    c = to_cuda(p)
    nbr, row_of = extension.pack_graph(c["indptr"], c["indices"], c["mapping"],
                                       c["storage"].size(0), 32)
    g = torch.Generator().manual_seed(3)
    en = torch.randint(6000, (32,), generator=g)
    ev = p["full"][en].contiguous().cuda()
    oI = torch.empty(64, 4, 16, dtype=torch.int64, device="cuda")
    oD = torch.empty(64, 4, 16, device="cuda")
    extension.search_reduced_noalloc(oI, oD, nbr, row_of, c["storage"], c["query"], None,
                                     en.cuda(), ev, 32)
    EP_D = extension.entry_distances(c["query"], ev)
    EP_I = en.cuda().unsqueeze(0).repeat(64, 1).contiguous()
    wI = torch.empty_like(oI); wD = torch.empty_like(oD)
    extension.traverse_packed(wI, wD, nbr, row_of, c["storage"], c["query"], EP_I, EP_D, 32)
    torch.cuda.synchronize()
    assert torch.equal(oI, wI) and torch.equal(oD, wD)


def test_sizes_beyond_the_static_scratch_are_refused():
    from pilotann_b200 import extension
    p = make_problem(n=6000, d=64, ratio=0.5, batch=64, n_init=32, seed=31)
    c = to_cuda(p)
    nbr, row_of = extension.pack_graph(c["indptr"], c["indices"], c["mapping"],
                                       c["storage"].size(0), 32)
    rv, en, ev = _tables(p, 4, 64, 5)
    big = extension.NOALLOC_MAX_BATCH + 1
    q = c["query"][:1].repeat(big, 1).contiguous()
    oI = torch.empty(big, 4, 16, dtype=torch.int64, device="cuda")
    oD = torch.empty(big, 4, 16, device="cuda")
    with pytest.raises(RuntimeError, match="PA_NOALLOC_MAX_BATCH"):
        extension.search_reduced_noalloc(oI, oD, nbr, row_of, c["storage"], q, rv, en, ev, 32)
    rv, en, ev = _tables(p, 4, 96, 6)
    with pytest.raises(RuntimeError, match="PA_NOALLOC_MAX_LEAVES"):
        extension.search_reduced_noalloc(oI[:8], oD[:8], nbr, row_of, c["storage"],
                                         c["query"][:8].contiguous(), rv, en, ev, 32)


def test_mismatched_shapes_are_refused_on_the_host_and_nothing_is_allocated():
    """Shapes that would make the kernels read past a table are turned down by
    the wrapper before anything is enqueued; a good call leaves torch's
    allocation counter where it was."""
    from pilotann_b200 import extension
    p = make_problem(n=6000, d=64, ratio=0.5, batch=64, n_init=32, seed=31)
    c = to_cuda(p)
    nbr, row_of = extension.pack_graph(c["indptr"], c["indices"], c["mapping"],
                                       c["storage"].size(0), 32)
    rv, en, ev = _tables(p, 4, 64, 7)
    q = c["query"]
    oI = torch.empty(64, 4, 16, dtype=torch.int64, device="cuda")
    oD = torch.empty(64, 4, 16, device="cuda")
    bad = [
        dict(ev=ev[:, :, :32].contiguous()),          # leaf vectors of another dimension
        dict(ev=ev[:3].contiguous()),                 # fewer routers than route_vectors
        dict(ev=ev[:, :32].contiguous()),             # fewer leaves than entry_nodes
        dict(rv=rv[:, :32].contiguous()),             # router vectors of another dimension
        dict(en=en[:2].contiguous()),                 # entry_nodes for fewer routers
        dict(nbr=nbr[:-1].contiguous()),              # packed rows != storage rows
        dict(n_nb=64),                                # degree other than the packed one
    ]
    launches = extension.launch_count()
    for change in bad:
        a = dict(rv=rv, en=en, ev=ev, nbr=nbr, n_nb=32)
        a.update(change)
        with pytest.raises(RuntimeError):
            extension.search_reduced_noalloc(oI, oD, a["nbr"], row_of, c["storage"], q, a["rv"],
                                             a["en"], a["ev"], a["n_nb"])
    assert extension.launch_count() == launches           # nothing was enqueued
    torch.cuda.synchronize()
    extension.search_reduced_noalloc(oI, oD, nbr, row_of, c["storage"], q, rv, en, ev, 32)  # set-up
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    extension.search_reduced_noalloc(oI, oD, nbr, row_of, c["storage"], q, rv, en, ev, 32)
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
