"""Checkpoint compatibility with upstream (pilot_ann/layers/staged.py:59-122):
an index dumped by this package loads with upstream's ``IndexStaged.load`` and
the other way round, tensor for tensor.  Needs the upstream Python sources
(imported from the reference checkout when it is present; skipped otherwise)."""
import os
import sys
import types

import pytest
import torch

from oracle import build_ref

_root = build_ref.reference_root()        # $PILOTANN_REFERENCE, else ../reference beside the repo
REFERENCE = str(_root) if _root is not None else ""


@pytest.fixture(scope="module")
def upstream_layers():
    if not REFERENCE or not os.path.isdir(os.path.join(REFERENCE, "pilot_ann")):
        pytest.skip("upstream sources not present")
    ext = build_ref.load()
    if ext is None:
        pytest.skip("oracle/_ref/extension.so not built")
    saved = {k: sys.modules.get(k) for k in ("faiss", "pilot_ann", "pilot_ann.extension")}
    sys.modules.setdefault("faiss", types.ModuleType("faiss"))   # only graph_init needs it
    sys.path.insert(0, REFERENCE)
    try:
        pkg = types.ModuleType("pilot_ann")
        pkg.__path__ = [os.path.join(REFERENCE, "pilot_ann")]
        sys.modules["pilot_ann"] = pkg
        sys.modules["pilot_ann.extension"] = ext
        pkg.extension = ext
        import importlib
        for sub in ("kernels", "utils", "layers"):
            setattr(pkg, sub, importlib.import_module("pilot_ann." + sub))
        yield pkg.layers
    finally:
        sys.path.remove(REFERENCE)
        for k in [m for m in sys.modules if m == "pilot_ann" or m.startswith("pilot_ann.")]:
            del sys.modules[k]
        for k, v in saved.items():
            if v is not None:
                sys.modules[k] = v
            elif k == "faiss":
                sys.modules.pop("faiss", None)


def _small_index():
    from pilotann_b200 import layers
    g = torch.Generator().manual_seed(5)
    x = torch.nn.functional.normalize(torch.randn(3000, 48, generator=g), dim=-1)
    index = layers.IndexStaged(d_model=48, d_principle=16, graph_method="nsw32",
                               entry_method="router4x32", sample_ratio=0.5)
    return index.train(x, generator=g)


def test_our_dump_loads_upstream_and_back(upstream_layers, tmp_path):
    from pilotann_b200 import layers
    ours = _small_index()
    path = tmp_path / "index.ckpt"
    torch.save(ours.dump(), path)
    theirs = upstream_layers.IndexStaged.load(str(path))
    want = ours.dump()["state_dict"]
    got = theirs.state_dict()
    assert set(got) == set(want)
    for key, value in want.items():
        assert got[key].dtype == value.dtype and torch.equal(got[key], value), key
    assert (theirs.d_model, theirs.d_principle, theirs.graph_method, theirs.entry_method) == \
           (ours.d_model, ours.d_principle, ours.graph_method, ours.entry_method)
    # and back: what upstream dumps is what this package loads
    path2 = tmp_path / "again.ckpt"
    torch.save(theirs.dump(), path2)
    again = layers.IndexStaged.load(str(path2))
    for key, value in want.items():
        assert torch.equal(again.state_dict()[key], value), key
