"""CPU-only: the C-ABI library loads and exports every symbol include/flash_sinkhorn_b200.h declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "flash_sinkhorn_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fs_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from flash_sinkhorn_b200 import _lib
    if not os.path.exists(_lib.library_path()):
        import __graft_entry__
        __graft_entry__.build()
    lib = ctypes.CDLL(_lib.library_path())
    names = declared_symbols()
    assert len(names) >= 13
    for name in names:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    assert set(names) == set(_lib.SIGNATURES), "ctypes signature table and header disagree"


def test_no_compute_without_gpu_but_metadata_calls_work():
    from flash_sinkhorn_b200 import _lib
    lib = _lib.load()
    assert lib.fs_version() >= 100
    assert lib.fs_workspace_bytes(_lib.OP_SOLVE_SYMMETRIC, 1000, 900, 64, _lib.PREC_SIMT) > 0
    assert lib.fs_last_error() is not None


def test_product_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "flash_sinkhorn_b200")
    for dirpath, _, files in os.walk(pkg):
        for fn in files:
            if fn.endswith((".py", ".cu", ".cuh", ".h")):
                src = open(os.path.join(dirpath, fn)).read()
                assert "oracle" not in src.replace("no CPU or PyTorch fallback", ""), f"{fn} mentions the oracle"


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from flash_sinkhorn_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "_LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(ImportError):
        _lib.load()
