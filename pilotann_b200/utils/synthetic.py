"""Seeded synthetic workloads standing in for the public datasets upstream
evaluates on (DEEP d=96, Text2Image d=200, LAION / Wiki d=768; see
``pilot_ann/utils/loader.py:97-204``), which are not available offline.  Only
shapes, sizes and the broad character of the value distributions are taken
from them; no dataset item is reproduced.

* ``mixture``  -- Gaussian mixture: centres ~ N(0, I), points = centre + sigma *
  N(0, I), rows L2-normalised (clustered, low-dimensional: the DEEP-like case);
* ``powerlaw`` -- anisotropic Gaussian with covariance spectrum lambda_i ~ 1/i
  under a seeded random rotation, rows L2-normalised (the cosine / inner-product
  embedding case); ``ood=True`` shifts the *queries* by 0.5 sigma_j along the top
  eight principal axes before normalisation (out-of-distribution queries).

Because the rows are unit-norm, L2, cosine and inner-product order coincide
(upstream implements squared L2 only, ``extension/traverse_cuda.cu:31-32``).

``fuzz`` reproduces the law of upstream's own unit-test data: uniform(-1, 1)
(``pilot_ann/utils/loader.py:9-41``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, replace

import torch


@dataclass(frozen=True)
class Workload:
    cfg: int                 # seed family
    name: str
    n_storage: int
    d_model: int
    law: str                 # 'mixture' | 'powerlaw' | 'fuzz'
    n_centres: int = 0
    sigma: float = 0.3
    ood: bool = False
    graph_method: str = "nsw32"
    sample_ratio: float = 0.25
    d_principle: int = 64
    entry_method: str = "random32"
    top_k: int = 10
    n_queries: int = 1024

    def scaled(self, n_storage: int, n_queries: int | None = None) -> "Workload":
        """Same law at a smaller size (parity tests); centres scale with n."""
        centres = max(8, self.n_centres * n_storage // self.n_storage) if self.n_centres else 0
        return replace(self, n_storage=n_storage, n_centres=centres,
                       n_queries=n_queries or self.n_queries,
                       name=f"{self.name}@{n_storage}")


WORKLOADS = {
    1: Workload(1, "c1-1m-96-l2", 1_000_000, 96, "mixture", n_centres=1024,
                graph_method="nsw32", sample_ratio=0.25, d_principle=64,
                entry_method="random32", top_k=10, n_queries=1024),
    2: Workload(2, "c2-1m-768-cos", 1_000_000, 768, "powerlaw",
                graph_method="nsw32", sample_ratio=0.25, d_principle=128,
                entry_method="router64x64", top_k=10, n_queries=1024),
    3: Workload(3, "c3-1m-200-ip-ood", 1_000_000, 200, "powerlaw", ood=True,
                graph_method="nsg32", sample_ratio=0.5, d_principle=96,
                entry_method="router32x32", top_k=100, n_queries=1024),
    4: Workload(4, "c4-10m-96-l2", 10_000_000, 96, "mixture", n_centres=10_000,
                graph_method="nsw32", sample_ratio=0.25, d_principle=64,
                entry_method="router64x64", top_k=10, n_queries=16384),
    5: Workload(5, "c5-100m-96-l2", 100_000_000, 96, "mixture", n_centres=100_000,
                graph_method="nsw32", sample_ratio=0.25, d_principle=64,
                entry_method="router64x64", top_k=10, n_queries=65536),
}


def _gen(seed: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return g


def _rotation(w: Workload, device) -> torch.Tensor:
    g = _gen(3000 + w.cfg)
    a = torch.randn(w.d_model, w.d_model, generator=g, dtype=torch.float64)
    q, r = torch.linalg.qr(a)
    q = q * torch.sign(torch.diagonal(r)).unsqueeze(0)
    return q.float().to(device)


def _draw(w: Workload, n: int, g: torch.Generator, device, queries: bool,
          chunk: int = 1 << 16) -> torch.Tensor:
    out = torch.empty(n, w.d_model, dtype=torch.float32, device=device)
    if w.law == "mixture":
        cg = _gen(3000 + w.cfg)
        centres = torch.randn(w.n_centres, w.d_model, generator=cg).to(device)
    elif w.law == "powerlaw":
        rot = _rotation(w, device)
        scale = torch.rsqrt(torch.arange(1, w.d_model + 1, dtype=torch.float32)).to(device)
    for s in range(0, n, chunk):
        m = min(chunk, n - s)
        if w.law == "fuzz":
            blk = (2.0 * (torch.rand(m, w.d_model, generator=g) - 0.5)).to(device)
            out[s:s + m] = blk
            continue
        z = torch.randn(m, w.d_model, generator=g).to(device)
        if w.law == "mixture":
            which = torch.randint(w.n_centres, (m,), generator=g).to(device)
            blk = centres[which] + w.sigma * z
        else:
            z = z * scale
            if queries and w.ood:
                z[:, :8] += 0.5 * scale[:8]
            blk = z @ rot.T
        out[s:s + m] = torch.nn.functional.normalize(blk, dim=-1)
    return out


def make_storage(w: Workload, device="cpu") -> torch.Tensor:
    return _draw(w, w.n_storage, _gen(1000 + w.cfg), device, queries=False)


def make_queries(w: Workload, device="cpu", n_queries: int | None = None) -> torch.Tensor:
    return _draw(w, n_queries or w.n_queries, _gen(2000 + w.cfg), device, queries=True)


@torch.no_grad()
def ground_truth(query: torch.Tensor, storage: torch.Tensor, k: int,
                 chunk_bytes: int = 1 << 30) -> torch.Tensor:
    """Exact top-k ids by squared L2 (brute force, tiled); int64 [B, k]."""
    n = storage.size(0)
    s2 = (storage * storage).sum(-1)
    rows = max(1, chunk_bytes // (n * 4 * 2))
    out = []
    for s in range(0, query.size(0), rows):
        q = query[s:s + rows]
        d = s2.unsqueeze(0) - 2.0 * q @ storage.T
        out.append(torch.topk(d, k, dim=1, largest=False).indices)
    return torch.cat(out)


def fuzz_workload(n_storage: int, d_model: int, seed: int = 0, n_queries: int = 256,
                  **kw) -> Workload:
    return Workload(100 + seed, f"fuzz-{n_storage}x{d_model}", n_storage, d_model, "fuzz",
                    n_queries=n_queries, **kw)
