"""The packed index (``pa_pack_graph``): ids, storage rows and the precomputed
bloom probes of every neighbour slot against a host restatement -- hash
positions from the oracle's FNV chain, elections by the rule "first slot of its
32-slot chunk to touch that bit in that hash step".  Integer work: bit-exact."""
import numpy as np
import pytest
import torch

from helpers import make_problem, to_cuda

pytestmark = pytest.mark.gpu


def _expected(p, n_nb, oracle):
    indptr, indices, mapping = (p[k].numpy() for k in ("indptr", "indices", "mapping"))
    n_storage = p["storage"].size(0)
    want = np.empty((n_storage, n_nb, 4), dtype=np.int64)
    want[..., 0], want[..., 1], want[..., 2], want[..., 3] = -1, -1, 0, 0
    want[:, 0, 0] = -2                      # rows without adjacency keep the tag
    for u in range(len(mapping)):
        row, lo, hi = mapping[u], indptr[u], indptr[u + 1]
        if row < 0 or hi == lo:
            continue
        ids = np.full(n_nb, -1, dtype=np.int64)
        ids[: min(hi - lo, n_nb)] = indices[lo: lo + min(hi - lo, n_nb)]
        for c in range(0, n_nb, 32):        # one chunk of 32 slots
            pos = np.array([oracle.bloom_positions(int(v)) if v >= 0 else [0] * 4
                            for v in ids[c:c + 32]], dtype=np.int64)
            elected = np.zeros((32, 4), dtype=np.int64)
            for s in range(4):
                seen = set()
                for lane in range(32):
                    if ids[c + lane] >= 0 and pos[lane, s] not in seen:
                        elected[lane, s] = 1
                        seen.add(pos[lane, s])
            valid = ids[c:c + 32] >= 0
            w0 = pos[:, 0] | (pos[:, 1] << 15) | ((elected[:, 0] | (elected[:, 1] << 1)) << 30)
            w1 = pos[:, 2] | (pos[:, 3] << 15) | ((elected[:, 2] | (elected[:, 3] << 1)) << 30)
            want[row, c:c + 32, 0] = ids[c:c + 32]
            want[row, c:c + 32, 1] = np.where(valid, mapping[np.maximum(ids[c:c + 32], 0)], -1)
            want[row, c:c + 32, 2] = w0
            want[row, c:c + 32, 3] = w1
    return want


@pytest.mark.parametrize("n_nb", [32, 64])
def test_packed_slots_match_host_restatement(oracle_lib, n_nb):
    from pilotann_b200 import extension
    p = make_problem(n=600, d=32, n_nb=n_nb, batch=2, seed=31 + n_nb, ratio=0.6, n_init=32)
    c = to_cuda(p)
    nbr, row_of = extension.pack_graph(c["indptr"], c["indices"], c["mapping"],
                                       c["storage"].size(0), n_nb)
    assert nbr.shape == (p["storage"].size(0), n_nb, 4) and nbr.dtype == torch.int32
    got = nbr.cpu().numpy().astype(np.int64)
    want = _expected(p, n_nb, oracle_lib)
    # ids and rows as they are; probe words compared as unsigned 32-bit patterns
    assert np.array_equal(got[..., :2], want[..., :2])
    valid = want[..., 0] >= 0
    assert np.array_equal(got[..., 2:][valid] & 0xffffffff, want[..., 2:][valid] & 0xffffffff)
    # slots without a node are never elected
    assert np.all(((got[..., 2] >> 30) & 3)[~valid] == 0) and np.all(((got[..., 3] >> 30) & 3)[~valid] == 0)
    assert torch.equal(row_of.cpu().long(), torch.where(p["mapping"] < 0, -1, p["mapping"]))


def test_same_bit_collision_elects_the_first_slot(oracle_lib):
    """A row holding the same id twice: the second copy must not be elected in any step."""
    from pilotann_b200 import extension
    n = 40
    indptr = torch.zeros(n + 1, dtype=torch.int64)
    indptr[1:] = 32                              # only node 0 has neighbours
    row = torch.arange(1, 33, dtype=torch.int64)
    row[7] = row[3]                              # duplicate id inside the chunk
    mapping = torch.arange(n, dtype=torch.int64)
    nbr, _ = extension.pack_graph(indptr.cuda(), row.cuda(), mapping.cuda(), n, 32)
    w = nbr[0].cpu().numpy().astype(np.int64) & 0xffffffff
    el = ((w[:, 2] >> 30) & 3) | (((w[:, 3] >> 30) & 3) << 2)
    assert el[3] == 0xF and el[7] == 0
