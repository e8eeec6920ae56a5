"""The stage object and the index layers, end to end on a GPU."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def small_index():
    from pilotann_b200 import layers, utils
    w = utils.WORKLOADS[2].scaled(12000, 256)
    w = type(w)(**{**w.__dict__, "d_model": 192, "d_principle": 64,
                   "entry_method": "router16x32"})
    x = utils.make_storage(w)
    g = torch.Generator().manual_seed(5000 + w.cfg)
    index = layers.IndexStaged(w.d_model, w.d_principle, w.sample_ratio, w.graph_method,
                               w.entry_method)
    index.train(x, generator=g, build_device="cuda")
    index.to("cuda", max_batch=256, max_ef=128)
    q = utils.make_queries(w)
    return index, x, q, w


def test_stage_equals_composition_of_ops(small_index, oracle_lib):
    """search_candidates == project -> route -> traverse, each checked against
    the oracle: the handoff ids / distances are those of the oracle run on the
    projected queries and entries the stage itself produced."""
    from pilotann_b200 import extension
    index, x, q, w = small_index
    ef = 32
    I, D, rotated = index.search_candidates(q, ef, chunk_size=64)
    qc = q.cuda()
    rot = extension.project(qc, index.VT_cuda)
    assert torch.equal(rot.cpu(), rotated)
    red = rot[:, :w.d_principle].contiguous()
    EP_I, EP_D = index.entry.search(red)
    want = oracle_lib.traverse(index.subgraph.indptr, index.subgraph.indices, index.mapping,
                               index.storage_cuda.cpu(), red.cpu(), EP_I.cpu(), EP_D.cpu(),
                               index.n_neighbors, ef)
    assert torch.equal(I.view(-1, 4, ef), want[0])
    assert torch.equal(D.view(-1, 4, ef), want[1])
    # chunking and stream count do not change the result
    I2, D2, _ = index.search_candidates(q, ef, chunk_size=0)
    assert torch.equal(I, I2) and torch.equal(D, D2)


def test_end_to_end_recall_with_cpu_refine(small_index, oracle_lib):
    """GPU stage -> CPU refinement (oracle restatement of traverse_refine):
    recall@10 against brute force, as upstream's test/module/test_staged.py:42."""
    from pilotann_b200 import utils
    index, x, q, w = small_index

    def refine(out_I, out_D, buf_I, buf_D, ini_I, ini_D, subgraph, fullgraph, storage, query,
               ef_search, d_principle):
        I, D = oracle_lib.refine(buf_I, buf_D, subgraph, fullgraph, storage,
                                 query.contiguous(), out_I.size(1), ef_search, d_principle)
        out_I.copy_(I); out_D.copy_(D)

    I, D = index.search(q, k=10, ef_search=32, chunk_size=64, refine=refine)
    truth = utils.ground_truth(q, x, 10)
    assert utils.recall(I, truth) > 0.90
    exact = torch.cdist(q.unsqueeze(1), x[I]).squeeze(1).square()
    assert torch.allclose(D, exact, atol=1e-3)


def test_device_resident_variant_matches_host_variant(small_index):
    index, x, q, w = small_index
    ef = 48
    I, D, _ = index.search_candidates(q, ef)
    st = torch.zeros(q.size(0), 4, dtype=torch.int32, device="cuda")
    dI, dD = index.stage.search_device(q.cuda(), ef, stats=st)
    index.stage.synchronize()
    assert torch.equal(dI.cpu().view(-1, 4 * ef), I) and torch.equal(dD.cpu().view(-1, 4 * ef), D)
    assert (st[:, 0] > 0).all() and (st[:, 2] >= st[:, 1]).all()


def test_stage_rejects_oversized_calls(small_index):
    index, x, q, w = small_index
    with pytest.raises(RuntimeError):
        index.stage.search_host(torch.zeros(257, w.d_model), 32)
    with pytest.raises(RuntimeError):
        index.stage.search_host(q, 129)


def test_dump_load_roundtrip(small_index):
    from pilotann_b200 import layers
    index, x, q, w = small_index
    again = layers.IndexStaged.load(index.dump())
    again.to("cuda", max_batch=256, max_ef=64)
    a = index.search_candidates(q[:32], 32)
    b = again.search_candidates(q[:32], 32)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])


def test_pipeline_wrapper_matches_upstream_signature(small_index, oracle_lib):
    """kernels.pipeline with upstream's keyword set (kernels/__init__.py:106-124)."""
    from pilotann_b200 import kernels, extension, utils
    index, x, q, w = small_index
    rot = extension.project(q.cuda(), index.VT_cuda)
    red = rot[:, :w.d_principle].contiguous()
    EP_I, EP_D = index.entry.search(red)

    def refine(out_I, out_D, buf_I, buf_D, ini_I, ini_D, subgraph, fullgraph, storage, query,
               ef_search, d_principle):
        I, D = oracle_lib.refine(buf_I, buf_D, subgraph, fullgraph, storage,
                                 query.contiguous(), out_I.size(1), ef_search, d_principle)
        out_I.copy_(I); out_D.copy_(D)

    import pilotann_b200
    # the call of pilot_ann/layers/staged.py:207-227, keyword for keyword
    call = dict(
        graph=[index.fullgraph.indptr, index.fullgraph.indices], storage=index.storage,
        subgraph=[index.subgraph.indptr, index.subgraph.indices],
        subgraph_cuda=[index.subgraph_cuda.indptr, index.subgraph_cuda.indices,
                       index.mapping_cuda],
        storage_cuda=index.storage_cuda, query=rot.cpu(), query_cuda=red, initial_I=EP_I,
        initial_D=EP_D, k=10, n_neighbors=32, ef_search=32, d_principle=w.d_principle)
    truth = utils.ground_truth(q, x, 10)
    try:
        pilotann_b200.set_refine(refine)           # a CPU consumer, overlapped with the GPU
        I, D = kernels.pipeline(chunk_size=64, **call)
        assert utils.recall(I, truth) > 0.90
        with pytest.raises(RuntimeError):          # pipeline_cpu.cpp:58
            kernels.pipeline(chunk_size=100, **call)
        pilotann_b200.set_refine(None)
        with pytest.raises(RuntimeError, match="set_refine"):
            kernels.pipeline(chunk_size=64, **call)
    finally:
        pilotann_b200.set_refine("gpu")
    # default consumer: the refinement kernel; the same answer as the oracle's
    # restatement of traverse_refine in that kernel's summation order, fed the same
    # handoff, bit for bit -- twice (the second call reuses every buffer)
    hI = torch.empty(q.size(0), 4, 32, dtype=torch.int64, device="cuda")
    hD = torch.empty(q.size(0), 4, 32, device="cuda")
    extension.traverse_cuda(hI, hD, index.subgraph_cuda.indptr, index.subgraph_cuda.indices,
                            index.mapping_cuda, index.storage_cuda, red, EP_I, EP_D, 32)
    torch.cuda.synchronize()
    w_I, w_D = oracle_lib.refine_ex(hI.view(q.size(0), -1).cpu(), hD.view(q.size(0), -1).cpu(),
                                    call["subgraph"], call["graph"], index.storage, rot.cpu(), 10,
                                    32, w.d_principle, gpu_order=True)
    for _ in range(2):
        gI, gD = kernels.pipeline(chunk_size=64, **call)
        assert gI.device.type == "cpu" and gI.shape == (q.size(0), 10)
        assert torch.equal(gI, w_I) and torch.equal(gD.view(torch.int32), w_D.view(torch.int32))
    assert utils.recall(gI, truth) > 0.90
    # positional order of extension/entry.cpp:48-56
    pI, pD = extension.pipeline(call["graph"], call["subgraph"], call["subgraph_cuda"],
                                call["storage"], call["storage_cuda"], call["query"],
                                call["query_cuda"], EP_I, EP_D, 32, 32, w.d_principle, 10, 128)
    assert torch.equal(pI, w_I)


def test_search_finishes_on_the_gpu_by_default(small_index, oracle_lib):
    """IndexStaged.search with upstream's signature and nothing else: top-k from
    the device, equal to the oracle's traverse_refine (kernel summation order) on
    the stage's own handoff; the stage-2 rows likewise."""
    from pilotann_b200 import utils
    index, x, q, w = small_index
    k, ef = 10, 32
    I, D = index.search(q, k, ef, 64)
    assert I.shape == (q.size(0), k) and I.device.type == "cpu"
    hI, hD, rot = index.search_candidates(q, ef)
    sub = [index.subgraph.indptr, index.subgraph.indices]
    full = [index.fullgraph.indptr, index.fullgraph.indices]
    bI, bD = hI.clone(), hD.clone()
    w_I, w_D = oracle_lib.refine_ex(bI, bD, sub, full, index.storage, rot.clone(), k, ef,
                                    w.d_principle, gpu_order=True)
    assert torch.equal(I, w_I) and torch.equal(D.view(torch.int32), w_D.view(torch.int32))
    s_I, s_D, _ = index.search_candidates(q, ef, stage2=True)
    assert torch.equal(s_I, bI) and torch.equal(s_D.view(torch.int32), bD.view(torch.int32))
    assert utils.recall(I, utils.ground_truth(q, x, k)) > 0.90
    # device-resident variant
    dI, dD = index.stage.search_device(q.cuda(), ef, k=k)
    index.stage.synchronize()
    assert torch.equal(dI.cpu(), I)
    # more queries than the stage takes at once
    more_I, more_D = index.search(torch.cat([q, q[:100]]), k, ef)
    assert torch.equal(more_I[:256], I) and torch.equal(more_I[256:], I[:100])
    assert torch.equal(more_D[256:], D[:100])


def test_submit_wait_slots(small_index):
    """Chunks in flight on the stage's slots: same rows as the blocking call,
    pinned buffers that persist, and the state errors."""
    index, x, q, w = small_index
    stage = index.stage
    ef = 32
    assert stage.slot_rows == 128                      # max_batch 256 over two streams
    want_I, want_D, want_rot = index.search_candidates(q, ef)
    stage.submit(0, q[:128].contiguous(), ef, want_rotated=True)
    stage.submit(1, q[128:256].contiguous(), ef, want_rotated=True)
    with pytest.raises(RuntimeError, match="still holds"):
        stage.submit(1, q[:8].contiguous(), ef)
    a = stage.wait(0)
    b = stage.wait(1)
    assert torch.equal(a[0], want_I[:128]) and torch.equal(b[0], want_I[128:])
    assert torch.equal(a[1], want_D[:128]) and torch.equal(b[2], want_rot[128:])
    with pytest.raises(RuntimeError, match="holds no chunk"):
        stage.wait(0)
    with pytest.raises(RuntimeError):
        stage.submit(0, torch.zeros(129, w.d_model), ef)
    addr = a[0].data_ptr()
    stage.submit(0, q[:64].contiguous(), ef, k=10)     # top-k through the same slot
    c = stage.wait(0)
    assert c[0].shape == (64, 10) and c[0].data_ptr() == addr
    top_I, _ = index.search(q[:64], 10, ef)
    assert torch.equal(c[0], top_I)


def test_ragged_chunks_and_empty_submit(small_index):
    index, x, q, w = small_index
    stage = index.stage
    ef, k = 32, 7
    want_I, want_D, _ = stage.search_host(q, ef, k=k)
    got_I, got_D, _ = stage.search_host(q, ef, chunk=100, k=k)        # 100 + 100 + 56
    assert torch.equal(want_I, got_I) and torch.equal(want_D, got_D)
    h_I, _, _ = stage.search_host(q, ef, chunk=96)
    h2_I, _, _ = stage.search_host(q, ef)
    assert torch.equal(h_I, h2_I)
    stage.submit(1, q[:0].contiguous(), ef, k=k)                       # nothing to do
    out = stage.wait(1)
    assert out[0].shape == (0, k)
    with pytest.raises(RuntimeError):                                  # k beyond the row
        stage.search_host(q, ef, k=4 * ef + 1)
