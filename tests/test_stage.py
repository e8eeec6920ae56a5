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

    I, D = kernels.pipeline(
        graph=[index.fullgraph.indptr, index.fullgraph.indices], storage=index.storage,
        subgraph=[index.subgraph.indptr, index.subgraph.indices],
        subgraph_cuda=[index.subgraph_cuda.indptr, index.subgraph_cuda.indices,
                       index.mapping_cuda],
        storage_cuda=index.storage_cuda, query=rot.cpu(), query_cuda=red, initial_I=EP_I,
        initial_D=EP_D, k=10, n_neighbors=32, ef_search=32, d_principle=w.d_principle,
        chunk_size=64, refine=refine)
    assert utils.recall(I, utils.ground_truth(q, x, 10)) > 0.90
    with pytest.raises(RuntimeError):          # pipeline_cpu.cpp:58
        kernels.pipeline(
            graph=[index.fullgraph.indptr, index.fullgraph.indices], storage=index.storage,
            subgraph=[index.subgraph.indptr, index.subgraph.indices],
            subgraph_cuda=[index.subgraph_cuda.indptr, index.subgraph_cuda.indices,
                           index.mapping_cuda],
            storage_cuda=index.storage_cuda, query=rot.cpu(), query_cuda=red, initial_I=EP_I,
            initial_D=EP_D, k=10, n_neighbors=32, ef_search=32, d_principle=w.d_principle,
            chunk_size=100, refine=refine)
