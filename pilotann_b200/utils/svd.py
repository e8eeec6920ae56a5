"""SVD rotation of the base vectors (build time).

Counterpart of ``pilot_ann/utils/svd.py:4-21``: returns ``(x @ V, V)`` where the
columns of ``V`` are the right singular vectors ordered by decreasing singular
value.  Upstream calls ``torch.svd`` on the whole matrix (or on a 10M-row
sample); here ``V`` comes from the eigen-decomposition of the d x d Gram matrix
accumulated in float64, which is the same subspace basis and needs one pass
over the rows instead of an N x d factorisation.
"""
from __future__ import annotations

import torch


@torch.no_grad()
def svd(x: torch.Tensor, max_size: int = 10_000_000, chunk: int = 1 << 18,
        generator: torch.Generator | None = None):
    assert x.dim() == 2
    n, d = x.shape
    if n > max_size:
        rows = torch.randint(n, (max_size,), generator=generator).to(x.device)
    else:
        rows = None
    gram = torch.zeros(d, d, dtype=torch.float64, device=x.device)
    total = n if rows is None else max_size
    for s in range(0, total, chunk):
        blk = x[s:s + chunk] if rows is None else x[rows[s:s + chunk]]
        blk = blk.double()
        gram += blk.T @ blk
    evals, evecs = torch.linalg.eigh(gram)
    V = evecs.flip(-1).to(x.dtype).contiguous()          # descending eigenvalues
    out = torch.empty_like(x)
    for s in range(0, n, chunk):
        out[s:s + chunk] = x[s:s + chunk] @ V
    return out, V
