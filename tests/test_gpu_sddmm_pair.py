"""The dense tensor-core SDDMM computed by pairs of CTAs (clusters of two, tcgen05 cta_group::2) on transposed tiles
(lane = mask column) and sampled through a column view of the mask, against the fp64 oracle and against the
single-CTA kernel it replaces (VSPARSE_B200_SDDMM_PAIR=0 switches it off).  Tolerance: conftest.assert_close
(rel-L2 <= 5e-3, max-abs <= 2e-2)."""
import numpy as np
import pytest
import torch

from conftest import assert_close
from gpu_util import DEV, custom, dev, problem, sddmm_oracle, structure
from vectorsparse_b200 import VS_PATH_TENSOR, _lib, cvse, ops

pytestmark = pytest.mark.gpu


def run(a, k, lhs, rhs, out_dtype, pair, monkeypatch):
    monkeypatch.setenv("VSPARSE_B200_SDDMM", "dense")
    monkeypatch.setenv("VSPARSE_B200_SDDMM_PAIR", "1" if pair else "0")
    ri, ro, ci = structure(a)
    nnz = a.nnz_vec * a.V
    out = torch.full((nnz + 64,), float("nan"), dtype=out_dtype, device=DEV)
    ops.sddmm.wmmaSddmm(a.m_vec, k, a.n, a.nnz_vec, ri, ro, ci, dev(lhs), dev(rhs), out, a.V, None, 1)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    host = out.float().cpu().numpy()
    assert np.all(np.isnan(host[nnz:])), "wrote past the end of the output"
    assert not np.any(np.isnan(host[:nnz])), "an output slot was never written"
    return host[:nnz]


def operands(a, k, seed, sigma=0.25):
    lhs = cvse.fill_random((a.m, k), np.float16, cvse.DIST_NORMAL, seed, sigma)
    rhs = cvse.fill_random((a.n, k), np.float16, cvse.DIST_NORMAL, seed + 1, sigma)
    return lhs, rhs


@pytest.mark.parametrize("V", [2, 4, 8])
@pytest.mark.parametrize("shape", [(256, 512, 256), (2048, 512, 64), (264, 200, 128), (520, 1000, 192), (128, 64, 512), (40, 72, 64),
                                   (1024, 128, 128), (776, 130, 64)])
def test_pairs_agree_with_the_oracle_and_the_single_cta_kernel(V, shape, monkeypatch):
    """Row counts that are not multiples of 256 (the second CTA of the last pair has few or no rows), mask widths that
    are not multiples of 32, widths of at most 128 (128-column items) and just above."""
    M, n, k = shape
    for s in (0.5, 0.9):
        a = problem(cvse.GEN_BETA, 3 * M + n + V, M // V, n, V, s)
        lhs, rhs = operands(a, k, 5)
        want = sddmm_oracle(a, k, lhs, rhs)
        for out_t in (torch.float16, torch.float32):
            two = run(a, k, lhs, rhs, out_t, True, monkeypatch)
            one = run(a, k, lhs, rhs, out_t, False, monkeypatch)
            assert_close(two, want, f"pairs {shape} V={V} s={s}")
            assert_close(one, want, f"single {shape} V={V} s={s}")
            assert np.array_equal(two, one), "same products in the same order: the two kernels must agree exactly"


@pytest.mark.parametrize("resident", ["1", "0"])
def test_resident_and_streamed_rhs_agree(resident, monkeypatch):
    """The rhs of a batch entry either stays in shared memory (when it fits) or streams through it like lhs
    (VSPARSE_B200_SDDMM_RESIDENT=0 forces that); several batch entries, so that resident tiles are replaced."""
    monkeypatch.setenv("VSPARSE_B200_SDDMM", "dense")
    monkeypatch.setenv("VSPARSE_B200_SDDMM_PAIR", "1")
    monkeypatch.setenv("VSPARSE_B200_SDDMM_RESIDENT", resident)
    V, k, n, batch = 8, 128, 512, 37
    a = problem(cvse.GEN_BETA, 77, 768 // V, n, V, 0.9)
    lhs = cvse.fill_random((batch, a.m * k), np.float16, cvse.DIST_NORMAL, 1, 0.25)
    rhs = cvse.fill_random((batch, n * k), np.float16, cvse.DIST_NORMAL, 2, 0.25)
    ri, ro, ci = structure(a)
    d_l, d_r = dev(lhs), dev(rhs)
    out = torch.full((batch, a.nnz_vec * V), float("nan"), dtype=torch.float32, device=DEV)
    rc = _lib.lib().vs_sddmm_batched(VS_PATH_TENSOR, 0, 1, a.m_vec, k, n, a.nnz_vec, ri.data_ptr(), ro.data_ptr(), ci.data_ptr(),
                                     d_l.data_ptr(), d_r.data_ptr(), out.data_ptr(), V, batch, a.m * k, n * k, a.nnz_vec * V,
                                     torch.cuda.current_stream().cuda_stream, 1)
    assert rc == 0
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    host = out.cpu().numpy()
    for b in (0, 1, 2, 18, batch - 1):
        assert_close(host[b], sddmm_oracle(a, k, lhs[b].reshape(a.m, k), rhs[b].reshape(n, k)), f"entry {b}, resident={resident}")


def test_dense_rows_and_rows_in_any_order(monkeypatch):
    """Full and nearly full vector-rows, empty rows, and a structure whose columns are not sorted inside a row."""
    lens = [0, 1, 15, 16, 17, 200, 384, 0, 33, 384, 2, 97]
    a = custom(lens, 384, 8, seed=4)
    lhs, rhs = operands(a, 128, 7)
    assert_close(run(a, 128, lhs, rhs, torch.float32, True, monkeypatch), sddmm_oracle(a, 128, lhs, rhs), "dense rows")
    rng = np.random.default_rng(3)
    ci = a.col_indices.copy()
    for i in range(a.m_vec):
        seg = ci[a.row_offsets[i]:a.row_offsets[i + 1]]
        rng.shuffle(seg)
    shuffled = cvse.CVSE(a.m_vec, a.n, 8, a.row_offsets, ci, a.row_indices)
    assert_close(run(shuffled, 128, lhs, rhs, torch.float32, True, monkeypatch), sddmm_oracle(shuffled, 128, lhs, rhs), "unsorted rows")


def test_many_items_per_pair_and_batch_strides(monkeypatch):
    """More work items than pairs fit on the device (every pair walks several items and both accumulator buffers),
    batch entries at padded strides."""
    monkeypatch.setenv("VSPARSE_B200_SDDMM", "dense")
    monkeypatch.setenv("VSPARSE_B200_SDDMM_PAIR", "1")
    V, k, n, batch = 8, 64, 300, 48
    a = problem(cvse.GEN_BETA, 21, 1024 // V, n, V, 0.8)          # 4 row tiles x 2 column tiles x 48 entries = 384 items
    s_l, s_r, s_o = a.m * k + 16, n * k + 24, a.nnz_vec * V + 8
    lhs = cvse.fill_random((batch, s_l), np.float16, cvse.DIST_NORMAL, 1, 0.25)
    rhs = cvse.fill_random((batch, s_r), np.float16, cvse.DIST_NORMAL, 2, 0.25)
    ri, ro, ci = structure(a)
    d_l, d_r = dev(lhs), dev(rhs)
    out = torch.full((batch, s_o), float("nan"), dtype=torch.float16, device=DEV)
    rc = _lib.lib().vs_sddmm_batched(VS_PATH_TENSOR, 0, 0, a.m_vec, k, n, a.nnz_vec, ri.data_ptr(), ro.data_ptr(), ci.data_ptr(),
                                     d_l.data_ptr(), d_r.data_ptr(), out.data_ptr(), V, batch, s_l, s_r, s_o,
                                     torch.cuda.current_stream().cuda_stream, 1)
    assert rc == 0
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    host = out.float().cpu().numpy()
    assert np.all(np.isnan(host[:, a.nnz_vec * V:])), "padding between batch entries was written"
    for b in (0, 1, 17, batch - 1):
        want = sddmm_oracle(a, k, lhs[b, :a.m * k].reshape(a.m, k), rhs[b, :n * k].reshape(n, k))
        assert_close(host[b, :a.nnz_vec * V], want, f"entry {b}")


def test_non_finite_products_outside_the_mask_do_not_leak(monkeypatch):
    a = custom([3, 5, 17, 9], 128, 8, seed=2)
    lhs, rhs = operands(a, 64, 3, 1.0)
    unused = sorted(set(range(128)) - set(a.col_indices.tolist()))
    rhs[unused[0]] = np.inf
    rhs[unused[1]] = np.nan
    got = run(a, 64, lhs, rhs, torch.float32, True, monkeypatch)
    clean = rhs.copy(); clean[unused[0]] = 0; clean[unused[1]] = 0
    assert_close(got, sddmm_oracle(a, 64, lhs, clean), "unreferenced inf / nan")


@pytest.mark.parametrize("V", [2, 4, 8])
def test_a_column_named_twice_in_a_vector_row(V, monkeypatch):
    """Every entry gets its outputs, also when a vector-row names the same column two or three times (the column view
    of the mask holds one of them; the fix-up kernel copies its outputs to the others)."""
    a = custom([5, 0, 9, 40, 3, 17, 64, 8] * 9, 200, V, seed=6)
    ci = a.col_indices.copy()
    ro = a.row_offsets
    ci[ro[0] + 1] = ci[ro[0]]                      # twice
    ci[ro[3] + 7] = ci[ro[3] + 20] = ci[ro[3] + 2]  # three times
    ci[ro[70] + 1] = ci[ro[70]]                    # in a later block of vector-rows
    dup = cvse.CVSE(a.m_vec, a.n, V, a.row_offsets, ci, a.row_indices)
    lhs, rhs = operands(dup, 64, 11)
    want = sddmm_oracle(dup, 64, lhs, rhs)
    for out_t in (torch.float16, torch.float32):
        assert_close(run(dup, 64, lhs, rhs, out_t, True, monkeypatch), want, f"repeated columns V={V}")


def test_masks_wider_than_the_plan_holds_fall_back_to_the_single_cta_kernel(monkeypatch):
    """Mask widths above 8192 columns (the plan kernel keeps a block's cells in shared memory) run the single-CTA
    kernel: same results as with the pair kernel switched off."""
    a = problem(cvse.GEN_BETA, 9, 256 // 8, 8448, 8, 0.97)
    lhs, rhs = operands(a, 128, 4)
    wide = run(a, 128, lhs, rhs, torch.float16, True, monkeypatch)
    assert_close(wide, sddmm_oracle(a, 128, lhs, rhs), "mask of 8448 columns")
    assert np.array_equal(wide, run(a, 128, lhs, rhs, torch.float16, False, monkeypatch))
