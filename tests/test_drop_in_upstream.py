"""Upstream's own Python call sites bound to this package.

``pilot_ann/kernels/__init__.py`` is a file of thin wrappers that call
``pilot_ann.extension.<name>(...)`` POSITIONALLY, so a drop-in extension has to
take the same arguments in the same order.  These tests import upstream's
unmodified ``pilot_ann.kernels`` / ``pilot_ann.layers`` with
``pilot_ann.extension`` replaced by a shim made of this package's three hot names
(``traverse_cuda``, ``routing_cuda``, ``pipeline``) plus upstream's CPU functions.

* CPU part: every upstream wrapper is called with sentinel objects and the shim
  checks, through the signature of this package's function, that each sentinel
  arrives in the parameter of the same meaning.
* GPU part: upstream's ``IndexStaged.load`` / ``.to`` / ``.search`` run as they
  are on a checkpoint written by this package and return what this package's own
  ``IndexStaged.search`` returns.

Both need the upstream Python sources next to the repository (they are never
copied into it) and are skipped where those are absent.
"""
import importlib
import inspect
import os
import sys
import types

import pytest
import torch

from oracle import build_ref

_root = build_ref.reference_root()
REFERENCE = str(_root) if _root is not None else ""


def _import_upstream(extension_module):
    """Upstream's package with ``pilot_ann.extension`` = ``extension_module``."""
    if not REFERENCE or not os.path.isdir(os.path.join(REFERENCE, "pilot_ann")):
        pytest.skip("upstream sources not present")
    saved = {k: v for k, v in sys.modules.items() if k == "faiss" or k.startswith("pilot_ann")}
    for k in [m for m in sys.modules if m.startswith("pilot_ann")]:
        del sys.modules[k]
    sys.modules.setdefault("faiss", types.ModuleType("faiss"))   # only graph_init needs it
    sys.path.insert(0, REFERENCE)
    pkg = types.ModuleType("pilot_ann")
    pkg.__path__ = [os.path.join(REFERENCE, "pilot_ann")]
    sys.modules["pilot_ann"] = pkg
    sys.modules["pilot_ann.extension"] = extension_module
    pkg.extension = extension_module
    for sub in ("kernels", "utils", "layers"):
        setattr(pkg, sub, importlib.import_module("pilot_ann." + sub))

    def restore():
        sys.path.remove(REFERENCE)
        for k in [m for m in sys.modules if m.startswith("pilot_ann")]:
            del sys.modules[k]
        if "faiss" not in saved:
            sys.modules.pop("faiss", None)
        sys.modules.update(saved)
    return pkg, restore


def _shim(ours, upstream_ext):
    shim = types.ModuleType("extension")
    for name in dir(upstream_ext or object()):
        if not name.startswith("_"):
            setattr(shim, name, getattr(upstream_ext, name))
    for name in ("traverse_cuda", "routing_cuda", "pipeline"):
        setattr(shim, name, getattr(ours, name))
    return shim


class _Named:
    def __init__(self, name):
        self.name = name


def test_upstream_wrappers_bind_to_this_packages_signatures():
    from pilotann_b200 import extension
    seen = {}

    def recorder(name):
        sig = inspect.signature(getattr(extension, name))

        def call(*args):
            seen[name] = sig.bind(*args).arguments
            return [None, None]
        return call

    shim = types.ModuleType("extension")
    for name in ("traverse_cuda", "routing_cuda", "pipeline"):
        setattr(shim, name, recorder(name))
    pkg, restore = _import_upstream(shim)
    try:
        kernels = pkg.kernels
        for fn_name in ("traverse_cuda", "routing_cuda", "pipeline"):
            fn = getattr(kernels, fn_name)
            params = list(inspect.signature(fn).parameters)
            fn(**{p: _Named(p) for p in params})          # upstream's keywords, by name
            got = seen[fn_name]
            assert set(got) >= set(params), (fn_name, set(params) - set(got))
            for p in params:                              # ... arrive under the same name
                assert got[p].name == p, (fn_name, p, got[p].name)
    finally:
        restore()


@pytest.mark.gpu
def test_upstream_index_searches_unmodified_through_this_package(tmp_path):
    import pilotann_b200
    from pilotann_b200 import extension, layers
    pkg, restore = _import_upstream(_shim(extension, build_ref.load()))
    try:
        g = torch.Generator().manual_seed(11)
        x = torch.nn.functional.normalize(torch.randn(8000, 96, generator=g), dim=-1)
        q = torch.nn.functional.normalize(torch.randn(256, 96, generator=g), dim=-1)
        ours = layers.IndexStaged(d_model=96, d_principle=32, graph_method="nsw32",
                                  entry_method="router8x32", sample_ratio=0.5)
        ours.train(x, generator=g, build_device="cuda")
        path = tmp_path / "index.ckpt"
        torch.save(ours.dump(), path)
        theirs = pkg.layers.IndexStaged.load(str(path))
        theirs.to("cuda")                                  # upstream's own .to
        t_I, t_D = theirs.search(q, k=10, ef_search=32, chunk_size=64)   # and .search
        ours.to("cuda", max_batch=256, max_ef=64)
        o_I, o_D = ours.search(q, 10, 32, 64)
        # upstream rotates the queries with a CPU matmul, this package on the tensor
        # cores: the two agree to ~1e-6, so a few near-ties may fall the other way
        assert (t_I == o_I).all(dim=1).float().mean().item() >= 0.98
        assert torch.allclose(t_D, o_D, rtol=1e-4, atol=1e-6) or \
            ((t_D - o_D).abs() > 1e-4).float().mean().item() < 0.02
        # with upstream's CPU consumer behind the same unmodified call sites
        pilotann_b200.set_refine(build_ref.load().traverse_refine)
        c_I, _ = theirs.search(q, k=10, ef_search=32, chunk_size=64)
        assert (c_I == t_I).all(dim=1).float().mean().item() >= 0.995
    finally:
        pilotann_b200.set_refine("gpu")
        restore()
