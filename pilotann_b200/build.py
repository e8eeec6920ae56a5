"""In-tree build of the C-ABI library ``pilotann_b200/_lib/libpilotann_b200.so``.

Every ``csrc/*.cu`` is compiled with nvcc for sm_100a only
(``-gencode arch=compute_100a,code=sm_100a``) and linked into one shared
library that depends on nothing but the CUDA runtime (linked statically) and
the driver; no torch headers are involved.  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
LIB_DIR = PKG / "_lib"
LIB = LIB_DIR / "libpilotann_b200.so"
NVCC = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr", "-Xcompiler",
         "-fPIC,-Wall,-Wno-unknown-pragmas", "-I", str(ROOT / "include"), "-I", str(CSRC)]


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def stale() -> bool:
    if not LIB.is_file():
        return True
    deps = list(CSRC.glob("*")) + [ROOT / "include" / "pilotann_b200.h", Path(__file__)]
    return any(d.stat().st_mtime > LIB.stat().st_mtime for d in deps)


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    if not force and not stale():
        return LIB
    obj_dir = LIB_DIR / "obj"
    obj_dir.mkdir(parents=True, exist_ok=True)
    extra = ["-Xptxas", "-v"] if ptxas_info else []
    # build parameters of the kernels (e.g. PA_MIN_CTAS=8), space separated NAME=VALUE
    extra += ["-D" + d for d in os.environ.get("PILOTANN_B200_DEFINES", "").split()]

    def compile_one(src: Path) -> tuple[Path, str]:
        obj = obj_dir / (src.stem + ".o")
        cmd = [NVCC, "-c", str(src), "-o", str(obj)] + ARCH + FLAGS + extra
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed: %s\n%s" % (" ".join(cmd), r.stdout))
        return obj, r.stdout

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        results = list(pool.map(compile_one, sources()))
    if verbose or ptxas_info:
        for _, out in results:
            if out.strip():
                print(out)
    cmd = [NVCC, "-shared", "-o", str(LIB)] + [str(o) for o, _ in results] + ARCH
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError("link failed: %s\n%s" % (" ".join(cmd), r.stdout))
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True, ptxas_info="--ptxas" in sys.argv))
