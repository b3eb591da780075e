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


def test_label_cost_descriptor_validation_and_workspace():
    """Host logic of the label-cost arguments (no GPU): the reference's activation rule and errors
    (kernels/sinkhorn_flashstyle_sqeuclid.py:1183-1208), the ctypes mirror of fs_label_cost, and the
    class-count argument of the workspace query."""
    import torch
    from flash_sinkhorn_b200 import _lib
    cpu = torch.device("cpu")
    lx, ly, W = torch.tensor([0, 2, 1]), torch.tensor([1, 1]), torch.rand(3, 3)
    mk = lambda **kw: _lib.LabelCost.make(kw.get("lx", lx), kw.get("ly", ly), kw.get("W", W), kw.get("lam_x", 1.0),
                                          kw.get("lam_y", 1.0), 3, 2, cpu)
    assert mk(lam_y=0.0) is None and mk(W=None) is None and mk(lx=None) is None
    lc = mk()
    assert lc.V == 3 and lc.label_x.dtype == torch.int32 and lc.table.dtype == torch.float32
    assert lc.struct.V == 3 and lc.struct.label_x == lc.label_x.data_ptr() and lc.struct.lambda_y == 1.0
    assert ctypes.sizeof(_lib.LabelCostStruct) == 3 * ctypes.sizeof(ctypes.c_void_p) + 12 + 4  # padded to 8
    for bad in (dict(lx=torch.tensor([0, 1])), dict(ly=torch.tensor([0, 3])), dict(W=torch.rand(3, 2)),
                dict(W=torch.rand(3)), dict(lx=torch.tensor([0, -1, 1])), dict(lam_x=0.0)):
        with pytest.raises(ValueError):
            mk(**bad)
    lib = _lib.load()
    plain = lib.fs_workspace_bytes(_lib.OP_SOLVE_SYMMETRIC, 5000, 4000, 64, _lib.PREC_TF32)
    labelled = lib.fs_workspace_bytes_labels(_lib.OP_SOLVE_SYMMETRIC, 5000, 4000, 64, _lib.PREC_TF32, 10)
    assert labelled > plain == lib.fs_workspace_bytes_labels(_lib.OP_SOLVE_SYMMETRIC, 5000, 4000, 64, _lib.PREC_TF32, 0)
    # exact-fp32 mode: the label block is staged once (K = 3*64 + 3*5 + 3), so this stays on the tensor-core engine
    exact = lib.fs_workspace_bytes_labels(_lib.OP_SOLVE_SYMMETRIC, 5000, 4000, 64, _lib.PREC_FP32, 5)
    assert exact > lib.fs_workspace_bytes(_lib.OP_SOLVE_SYMMETRIC, 5000, 4000, 64, _lib.PREC_SIMT)
    assert lib.fs_set_reserved_sms(3) == 0 and lib.fs_set_reserved_sms(0) == 3


def test_workspace_sizes_at_the_largest_shapes():
    """Host-side size logic only. The tcgen05 kernel numbers its (row block, column tile) items with 32-bit
    integers, so problems with about 1.7e13 entries or more must be planned for the CUDA-core engine (no staged
    operands: a far smaller workspace); sizes must never wrap around 2^32 or come out zero."""
    from flash_sinkhorn_b200 import _lib
    lib = _lib.load()
    big = lib.fs_workspace_bytes(_lib.OP_LSE, 4_000_000, 4_000_000, 64, _lib.PREC_TF32)
    over = lib.fs_workspace_bytes(_lib.OP_LSE, 4_300_000, 4_300_000, 64, _lib.PREC_TF32)
    assert big > 2 * 4_000_000 * 64 * 4  # staged operands of both clouds
    assert 0 < over < big // 10  # one vector of scratch, no staging
    # a long thin problem stays on the tensor-core engine whichever side is long
    for n, m in ((16_000_000, 1000), (1000, 16_000_000)):
        assert lib.fs_workspace_bytes(_lib.OP_LSE, n, m, 64, _lib.PREC_TF32) > 16_000_000 * 64 * 4
    # config 3 of the benchmark list (1e6 x 1e6, d = 3) and config 5 (d = 2048) have non-zero plans in every op
    for op in range(9):
        assert lib.fs_workspace_bytes(op, 1_000_000, 1_000_000, 3, _lib.PREC_TF32) > 0
        assert lib.fs_workspace_bytes(op, 16384, 16384, 2048, _lib.PREC_FP32) > 0
    assert lib.fs_workspace_bytes(_lib.OP_LSE, 0, 5, 3, 0) == 0 and lib.fs_workspace_bytes(_lib.OP_LSE, 5, 5, 0, 0) == 0
