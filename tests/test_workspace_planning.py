"""Host-side planning of the CUDA library, checked without a GPU: workspace sizes reported by
`fs_workspace_bytes` cover what the entry points carve, and the CTA split of a streaming pass respects its bounds."""
import os

import pytest

from flash_sinkhorn_b200 import _lib

pytestmark = pytest.mark.skipif(not os.path.exists(_lib.library_path()), reason="the CUDA library has not been built")


@pytest.mark.parametrize("prec", [_lib.PREC_TF32, _lib.PREC_FP32])
def test_apply_mat_never_carves_more_than_the_reported_workspace(prec):
    """fs_apply_mat may be called with any matrix width dv <= d; the size query has no dv argument, so it must
    cover the largest need over all widths (the tensor-core scratch of a narrow matrix can exist where the one
    of a d-wide matrix does not fit shared memory)."""
    lib = _lib.load()
    n, m = 700, 900
    for d in range(1, 261):
        reported = lib.fs_workspace_bytes(_lib.OP_APPLY_MAT, n, m, d, prec)
        assert reported > 0
        for dv in sorted({1, 3, 32, 33, 64, 96, 128, d}):
            if dv > d:
                continue
            carved = lib.fs_apply_mat_plan_bytes(n, m, d, dv, prec)
            assert 0 < carved <= reported, (d, dv, carved, reported)


def test_large_feature_dimensions_report_the_streamed_scratch():
    lib = _lib.load()
    n = m = 4096
    small = lib.fs_workspace_bytes(_lib.OP_GRAD, n, m, 64, _lib.PREC_TF32)
    big = lib.fs_workspace_bytes(_lib.OP_GRAD, n, m, 2048, _lib.PREC_TF32)
    # scores / weights of a chunk of rows plus the transposed matrix: at least n*m + d*m floats
    assert big > small and big >= 4 * (n * m + 2048 * m)
    assert lib.fs_engine(n, m, 64, _lib.PREC_TF32) == 1
    assert lib.fs_engine(n, m, 2048, _lib.PREC_TF32) == 2
    assert lib.fs_engine(n, m, 128, _lib.PREC_FP32) == 2
    assert lib.fs_engine(n, m, 64, _lib.PREC_SIMT) == 0


def _pieces(nblk, ntiles, g):
    """Largest number of CTAs sharing one row block when nblk*ntiles items are cut into g equal contiguous ranges."""
    total = nblk * ntiles
    first = lambda c: (total * c) // g
    def owner(t):
        c = (t * g) // total
        while c + 1 < g and first(c + 1) <= t:
            c += 1
        while c > 0 and first(c) > t:
            c -= 1
        return c
    return max(owner((b + 1) * ntiles - 1) - owner(b * ntiles) + 1 for b in range(nblk))


@pytest.mark.parametrize("sms", [148, 132, 74, 16])
def test_cta_split_respects_the_sm_count_and_the_partial_slots(sms):
    lib = _lib.load()
    for nblk, ntiles in [(1, 1), (1, 391), (25, 391), (196, 391), (64, 64), (7813, 7813), (3, 5000), (2, 2)]:
        for reserved in (0, 2):
            for limit in (0, 1, 7):
                g = lib.fs_plan_ctas(nblk, ntiles, sms, reserved, limit)
                assert 1 <= g <= max(1, sms - reserved)
                assert g <= nblk * ntiles
                if limit:
                    assert g <= limit
                if nblk * ntiles <= 200000:  # the check walks every row block
                    assert _pieces(nblk, ntiles, g) <= 16
    assert lib.fs_plan_ctas(0, 5, sms, 0, 0) == 0


@pytest.mark.parametrize("sms", [148, 132, 16])
def test_matrix_pass_column_shares_fit_the_scratch(sms):
    """Column shares of the plan-times-matrix kernel: never more raw output tiles than the scratch was sized for
    (sized from the larger cloud, used for any row range of it), at least 8 column tiles per share, none for
    small clouds, and a better SM fill than without shares whenever shares are used."""
    import ctypes
    lib = _lib.load()
    for prec, bn in ((0, 128), (1, 64)):
        for n, m in [(50000, 50000), (6250, 50000), (50000, 6250), (4096, 4096), (1000, 900), (300, 9000), (128, 128),
                     (100000, 80000), (1, 1), (200000, 200000)]:
            slots = ctypes.c_int(-1)
            s = lib.fs_plan_pv_split(n, m, prec, sms, ctypes.byref(slots))
            nblk, ntiles = (n + 127) // 128, (m + bn - 1) // bn
            assert 1 <= s <= 8
            if s > 1:
                assert nblk * s <= slots.value
                assert ntiles // s >= 8
                fill = lambda k: nblk * k / (-(-nblk * k // sms) * sms)
                assert fill(s) > fill(1)
            # a row shard of the same problem must fit the slots sized for the whole problem
            full = ctypes.c_int(-1)
            lib.fs_plan_pv_split(max(n, m), max(n, m), prec, sms, ctypes.byref(full))
            assert slots.value == full.value
            if -(-max(n, m) // bn) < 16:  # fewer than 16 column tiles: no shares
                assert slots.value == 0 and s == 1
    assert lib.fs_plan_pv_split(0, 5, 0, sms, None) == 0
