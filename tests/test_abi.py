"""The C-ABI library loads on a machine without a GPU, exports every symbol the
header declares, and rejects bad arguments before touching CUDA."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def declared_symbols():
    text = (ROOT / "include" / "pilotann_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pa_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from pilotann_b200 import _C
    lib = _C.lib()
    names = declared_symbols()
    assert len(names) >= 15
    for name in names:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    assert set(names) == set(_C.SYMBOLS)
    assert lib.pa_version() >= 100


def test_no_torch_types_in_the_header():
    text = (ROOT / "include" / "pilotann_b200.h").read_text()
    assert "torch" not in re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    assert "at::" not in text and "#include <stdint.h>" in text


def test_heap_size_dispatch_matches_upstream_launcher():
    from pilotann_b200 import _C
    lib = _C.lib()
    table = {0: -1, 1: 32, 32: 32, 33: 64, 64: 64, 65: 128, 128: 128, 129: 256, 2048: 256,
             2049: -1}
    for ef, h in table.items():
        assert lib.pa_heap_size_for(ef) == h


def test_argument_errors_come_back_as_codes_and_messages():
    from pilotann_b200 import _C
    lib = _C.lib()
    # n_neighbors = 48 is not a multiple of 32 (extension/traverse_cuda.cu:281)
    rc = lib.pa_traverse_csr(0, 0, 0, 0, 0, 0, 0, 0, 0, 4, 100, 100, 64, 48, 8, 16, 0, 0)
    assert rc == _C.PA_ERR_ARG and b"multiple of 32" in lib.pa_last_error()
    # 4 * n_neighbors > 256 (:280)
    rc = lib.pa_traverse_csr(0, 0, 0, 0, 0, 0, 0, 0, 0, 4, 100, 100, 64, 96, 8, 16, 0, 0)
    assert rc == _C.PA_ERR_ARG
    # ef_search > 2048 (:313)
    rc = lib.pa_traverse_packed(0, 0, 0, 0, 0, 0, 0, 0, 4, 100, 100, 64, 32, 8, 4096, 0, 0)
    assert rc == _C.PA_ERR_ARG and b"ef_search" in lib.pa_last_error()
    # n_leaves % 32 (extension/routing_cuda.cu:90)
    rc = lib.pa_route(0, 0, 0, 0, 0, 0, 0, 4, 64, 8, 48, 0)
    assert rc == _C.PA_ERR_ARG and b"n_leaves" in lib.pa_last_error()
    # the allocation-free entry point states its limit
    rc = lib.pa_search_reduced_noalloc(0, 0, 0, 0, 0, 0, 0, 0, 0, 5000, 100, 100, 64, 32, 8, 32, 16, 0)
    assert rc == _C.PA_ERR_ARG and b"PA_NOALLOC_MAX_BATCH" in lib.pa_last_error()
    with pytest.raises(RuntimeError, match="pilotann_b200"):
        _C.check(rc)


def test_python_ops_reject_cpu_tensors_like_check_cuda():
    import torch
    from pilotann_b200 import extension
    q = torch.zeros(4, 64)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        extension.routing_cuda(q, q, torch.zeros(2, 32, dtype=torch.long), torch.zeros(2, 32, 64))
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        extension.project(q, torch.zeros(64, 64))


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from pilotann_b200 import _C
    monkeypatch.setattr(_C, "_lib", None)
    monkeypatch.setattr(_C, "LIB_PATH", tmp_path / "nope.so")
    with pytest.raises(ImportError, match="no CPU fallback"):
        _C.lib()
