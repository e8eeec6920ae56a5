"""Compile the upstream PilotANN extension, unmodified, into ``oracle/_ref/``.

TEST INFRASTRUCTURE ONLY.  The upstream sources are compiled where they lie
(the checkout named by ``$PILOTANN_REFERENCE``, else a ``reference`` directory beside this
repository); nothing is copied into this
repository and the upstream build system (``setup.py``) is not run: this file
is the whole recipe -- one ``g++``/``nvcc`` command per translation unit listed
in the upstream ``setup.py:28-37`` and one link step.  The host flags are the
ones the upstream build uses (``setup.py:39-44``); the device code is built for
sm_100a.

The result, ``oracle/_ref/extension.so``, is a pybind11 module with the eleven
functions of the upstream ``extension/entry.cpp:65-86``.  It is used

* by the tests, to pin the C restatement in ``oracle/pilot_oracle.c`` against
  the upstream heap / traversal code, and (on a GPU) as the parity target for
  the CUDA kernels of this package;
* by ``bench.py`` as the timed CPU baseline (``traverse_cpu`` /
  ``traverse_refine``).

No product code may import it.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
SOURCES = [
    "entry.cpp", "ops_cpu.cpp", "sampling_cpu.cpp", "traverse_cpu.cpp",
    "pipeline_cpu.cpp", "traverse_cuda.cu", "routing_cuda.cu",
]


def reference_root() -> Path | None:
    root = Path(os.environ.get("PILOTANN_REFERENCE", HERE.parent.parent / "reference"))
    return root if (root / "extension" / "entry.cpp").is_file() else None


def target() -> Path:
    return OUT / "extension.so"


def build(force: bool = False, verbose: bool = False) -> Path | None:
    """Build ``oracle/_ref/extension.so``; returns its path, or the prebuilt one
    when the upstream sources are not present, or None if neither exists."""
    root = reference_root()
    so = target()
    if root is None:
        return so if so.is_file() else None
    srcs = [root / "extension" / s for s in SOURCES]
    deps = srcs + list((root / "extension" / "inc").glob("*")) + [Path(__file__)]
    if so.is_file() and not force:
        if all(so.stat().st_mtime >= d.stat().st_mtime for d in deps):
            return so

    import torch  # noqa: F401  (header / library locations)
    import pybind11
    tdir = Path(torch.__file__).resolve().parent
    cuda = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
    incs = [
        tdir / "include", tdir / "include/torch/csrc/api/include",
        cuda / "include", Path(sysconfig.get_paths()["include"]),
        Path(pybind11.get_include()),
    ]
    inc_flags = [f"-I{p}" for p in incs] + [f"-I{root / 'extension'}"]
    defs = ["-DTORCH_EXTENSION_NAME=extension", "-DTORCH_API_INCLUDE_EXTENSION_H",
            "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI)]
    host = ["-O3", "-fPIC", "-std=c++17", "-mavx2", "-mfma", "-fopenmp",
            "-ffast-math", "-funroll-loops", "-w"]
    obj_dir = OUT / "obj"
    obj_dir.mkdir(parents=True, exist_ok=True)
    cmds, objs = [], []
    for src in srcs:
        obj = obj_dir / (src.name + ".o")
        objs.append(obj)
        if src.suffix == ".cu":
            cmds.append([
                str(cuda / "bin/nvcc"), "-c", str(src), "-o", str(obj), "-O3",
                "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a",
                "-lineinfo", "--expt-relaxed-constexpr", "--expt-extended-lambda",
                "-Xcompiler", "-fPIC,-w", "-w",
                "-D__CUDA_NO_HALF_OPERATORS__", "-D__CUDA_NO_HALF_CONVERSIONS__",
                "-D__CUDA_NO_HALF2_OPERATORS__",
                "-D__CUDA_NO_BFLOAT16_CONVERSIONS__"] + defs + inc_flags)
        else:
            cmds.append(["g++", "-c", str(src), "-o", str(obj)] + host + defs
                        + inc_flags)
    procs = [subprocess.Popen(c, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                              text=True) for c in cmds]
    for c, p in zip(cmds, procs):
        out, _ = p.communicate()
        if p.returncode != 0:
            raise RuntimeError("reference build failed:\n%s\n%s" % (" ".join(c), out))
        if verbose and out.strip():
            print(out)
    link = ["g++", "-shared", "-o", str(so)] + [str(o) for o in objs] + [
        f"-L{tdir / 'lib'}", f"-L{cuda / 'lib64'}", f"-Wl,-rpath,{tdir / 'lib'}",
        f"-Wl,-rpath,{cuda / 'lib64'}", "-lc10", "-lc10_cuda", "-ltorch_cpu",
        "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart", "-lgomp"]
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError("reference link failed:\n" + r.stdout)
    shutil.rmtree(obj_dir, ignore_errors=True)
    return so


def load():
    """Import the built module (``import torch`` first: it needs libtorch)."""
    so = target()
    if not so.is_file():
        return None
    import importlib.util
    import torch  # noqa: F401
    spec = importlib.util.spec_from_file_location("extension", so)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose=True)
    print(path if path else "reference sources not found and no prebuilt module")
