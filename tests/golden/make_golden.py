"""Generates the golden fixtures in this directory by running the UPSTREAM code
(compiled in place into oracle/_ref by oracle/build_ref.py) on seeded inputs.

    python tests/golden/make_golden.py            # CPU fixtures (no GPU needed)
    python tests/golden/make_golden.py --gpu OUT  # GPU fixtures, on a CUDA box

CPU fixtures (golden_cpu.pt): heap operation traces through upstream's
heapq.cuh (extension.heapq_*_cpu), and traverse_cpu / traverse_refine outputs
on a small graph.  GPU fixtures (golden_gpu.pt): outputs of upstream's
traverse_cuda and routing_cuda kernels on the same small inputs.  The inputs
are stored inside the fixtures, so nothing has to be regenerated to use them.
"""
from __future__ import annotations

import sys
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parents[1]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

from oracle import build_ref  # noqa: E402


def heap_traces(ext, seed=7):
    g = torch.Generator().manual_seed(seed)
    traces = []
    for hsize in (1, 2, 3, 7, 32, 48, 64, 100, 256):
        for kind in ("open", "result"):
            keys = torch.full((hsize,), float("inf") if kind == "open" else float("-inf"))
            vals = torch.full((hsize,), -1, dtype=torch.long)
            ops = []
            n_ops = 4 * hsize + 16
            opcodes = torch.randint(0, 4, (n_ops,), generator=g).tolist()
            ks = torch.rand(n_ops, generator=g)
            ks = torch.round(ks * 64) / 64 if hsize % 2 else ks    # some traces full of ties
            for i, (op, k) in enumerate(zip(opcodes, ks.tolist())):
                if kind == "result":
                    k = -k
                if op == 0:
                    ext.heapq_pop_cpu(keys, vals)
                    ops.append((0, 0.0, 0))
                elif op in (1, 3) and kind == "open":
                    ext.heapq_replace_cpu(keys, vals, k, i)
                    ops.append((1, k, i))
                else:
                    ext.heapq_pushpop_cpu(keys, vals, k, i)
                    ops.append((2, k, i))
            traces.append(dict(hsize=hsize, kind=kind, ops=ops, keys=keys.clone(),
                               values=vals.clone()))
    return traces


def small_problem():
    from helpers import make_problem
    p = make_problem(n=1024, d=32, n_nb=32, ratio=0.5, batch=24, n_init=32, seed=11)
    full_indptr, full_indices = __import__("pilotann_b200").utils.graph_init(p["full"], "nsw", 32)
    out = {k: v for k, v in p.items() if isinstance(v, torch.Tensor)}
    out["full_indptr"], out["full_indices"] = full_indptr, full_indices
    return out


def cpu_fixtures(ext):
    p = small_problem()
    fx = dict(heap=heap_traces(ext), problem=p, search={}, refine={})
    x, q = p["full"], p["query"]
    for ef in (16, 40, 64):
        I = torch.empty(q.size(0), 10, dtype=torch.long)
        D = torch.empty(q.size(0), 10)
        ext.traverse_cpu(I, D, p["initial_I"].clone(), p["initial_D"].clone(),
                         p["full_indptr"], p["full_indices"], x, q, ef)
        fx["search"][ef] = (I, D)
    # refine: handoff = 4*ef candidates among the sampled nodes with distances
    # over the first 16 of 32 dims (d_principle = 16)
    g = torch.Generator().manual_seed(5)
    for ef in (16, 32):
        nb = 4 * ef
        cand = p["nodelist"][torch.randint(p["nodelist"].numel(), (q.size(0), nb), generator=g)]
        cand[:, ::7] = -1
        dp = 16
        diff = q[:, None, :dp] - x[cand.clamp_min(0)][:, :, :dp]
        cand_D = (diff * diff).sum(-1)
        cand_D[cand < 0] = float("inf")
        bI, bD = cand.clone(), cand_D.clone()
        I = torch.empty(q.size(0), 10, dtype=torch.long)
        D = torch.empty(q.size(0), 10)
        ext.traverse_refine(I, D, bI, bD, bI, bD, [p["indptr"], p["indices"]],
                            [p["full_indptr"], p["full_indices"]], x, q, ef, dp)
        fx["refine"][ef] = dict(cand_I=cand, cand_D=cand_D, out_I=I, out_D=D,
                                buffer_I=bI, buffer_D=bD, d_principle=dp)
    return fx


def gpu_fixtures(ext, cpu_fx):
    p = cpu_fx["problem"]
    dev = "cuda"
    fx = dict(traverse={}, routing={})
    for ef in (16, 32, 48, 100):
        B = p["query"].size(0)
        oI = torch.empty(B, 4, ef, dtype=torch.long, device=dev)
        oD = torch.empty(B, 4, ef, device=dev)
        ext.traverse_cuda(oI, oD, p["indptr"].to(dev), p["indices"].to(dev),
                          p["mapping"].to(dev), p["storage"].to(dev), p["query"].to(dev),
                          p["initial_I"].to(dev), p["initial_D"].to(dev), 32)
        torch.cuda.synchronize()
        fx["traverse"][ef] = (oI.cpu(), oD.cpu())
    g = torch.Generator().manual_seed(3)
    x = p["full"]
    for n_r, n_l in ((8, 32), (16, 64)):
        rv = x[torch.randint(x.size(0), (n_r,), generator=g)].contiguous()
        en = torch.randint(x.size(0), (n_r, n_l), generator=g)
        ev = x[en].contiguous()
        router, dist = ext.routing_cuda(p["query"].to(dev), rv.to(dev), en.to(dev), ev.to(dev))
        torch.cuda.synchronize()
        fx["routing"][(n_r, n_l)] = dict(route_vectors=rv, entry_nodes=en, router=router.cpu(),
                                         distances=dist.cpu())
    return fx


def main():
    build_ref.build()
    ext = build_ref.load()
    assert ext is not None, "upstream module not built"
    if "--gpu" in sys.argv:
        out = Path(sys.argv[sys.argv.index("--gpu") + 1])
        cpu_fx = torch.load(HERE / "golden_cpu.pt")
        torch.save(gpu_fixtures(ext, cpu_fx), out)
        print("wrote", out)
    else:
        torch.save(cpu_fixtures(ext), HERE / "golden_cpu.pt")
        print("wrote", HERE / "golden_cpu.pt")


if __name__ == "__main__":
    main()
