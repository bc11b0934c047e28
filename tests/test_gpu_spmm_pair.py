"""The densifying tensor-core SpMM computed by pairs of CTAs (clusters of two, tcgen05 cta_group::2), which takes
dense widths that are multiples of 128, against the fp64 oracle and against the single-CTA kernel it replaces there
(VSPARSE_B200_SPMM_PAIR=0 switches it off).  Tolerance: conftest.assert_close (rel-L2 <= 5e-3, max-abs <= 2e-2)."""
import numpy as np
import pytest
import torch

from conftest import assert_close
from gpu_util import DEV, custom, dev, problem, spmm_inputs, spmm_oracle, structure
from vectorsparse_b200 import VS_PATH_TENSOR, _lib, cvse, ops

pytestmark = pytest.mark.gpu


def run(a, N, vals, B, out_dtype, pair, monkeypatch, mode="dense"):
    monkeypatch.setenv("VSPARSE_B200_SPMM", mode)
    monkeypatch.setenv("VSPARSE_B200_SPMM_PAIR", "1" if pair else "0")
    ri, ro, ci = structure(a)
    m = a.m_vec * a.V
    out = torch.full((m * N + 64,), float("nan"), dtype=out_dtype, device=DEV)
    ops.spmm.wmmaSpmm(a.m_vec, a.V, N, a.n, ri, ro, ci, dev(vals), dev(B), out)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    host = out.float().cpu().numpy()
    assert np.all(np.isnan(host[m * N:])), "wrote past the end of the output"
    return host[:m * N].reshape(m, N)


@pytest.mark.parametrize("V", [2, 4, 8])
@pytest.mark.parametrize("shape", [(256, 512, 256), (2048, 512, 256), (264, 200, 128), (520, 1000, 384), (128, 64, 512), (40, 72, 1024)])
def test_pairs_agree_with_the_oracle_and_the_single_cta_kernel(V, shape, monkeypatch):
    """Row counts that are not multiples of 256 (the second CTA of the last pair has few or no rows), contraction
    lengths that are not multiples of 64, widths that give 256-column items (256, 512, 1024) and 128-column items
    (128, 384)."""
    M, K, N = shape
    for s in (0.5, 0.9):
        a = problem(cvse.GEN_BETA, 3 * M + K + V, M // V, K, V, s)
        vals, B = spmm_inputs(a, N, np.float16, 5, sigma=0.5)
        want = spmm_oracle(a, N, vals, B)
        for out_t in (torch.float16, torch.float32):
            two = run(a, N, vals, B, out_t, True, monkeypatch)
            one = run(a, N, vals, B, out_t, False, monkeypatch)
            assert_close(two, want, f"pairs {shape} V={V} s={s}")
            assert_close(one, want, f"single {shape} V={V} s={s}")
            assert np.max(np.abs(two - one)) <= 1e-2


def test_many_items_per_pair_and_batch_strides(monkeypatch):
    """More work items than pairs fit on the device (every pair walks several items and both accumulator buffers),
    batch entries at padded strides, shared values."""
    monkeypatch.setenv("VSPARSE_B200_SPMM", "dense")
    monkeypatch.setenv("VSPARSE_B200_SPMM_PAIR", "1")
    V, N, K, batch = 8, 256, 192, 40
    a = problem(cvse.GEN_BETA, 21, 1024 // V, K, V, 0.8)          # 4 row tiles x 40 entries = 160 items
    row = (a.nnz_vec * V + 7) // 8 * 8 + 8
    vals = cvse.fill_random((batch, row), np.float16, cvse.DIST_NORMAL, 1, 0.5)
    B = cvse.fill_random((batch, K * N + 16), np.float16, cvse.DIST_NORMAL, 2, 1.0)
    ri, ro, ci = structure(a)
    d_vals, d_B = dev(vals), dev(B)
    out = torch.full((batch, a.m * N + 8), float("nan"), dtype=torch.float16, device=DEV)
    rc = _lib.lib().vs_spmm_batched(VS_PATH_TENSOR, 0, 0, a.m_vec, V, N, K, ri.data_ptr(), ro.data_ptr(), ci.data_ptr(),
                                    d_vals.data_ptr(), d_B.data_ptr(), out.data_ptr(), batch, row, B.shape[1], out.shape[1],
                                    torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    host = out.float().cpu().numpy()
    assert np.all(np.isnan(host[:, a.m * N:])), "padding between batch entries was written"
    for b in (0, 1, 17, batch - 1):
        want = spmm_oracle(a, N, vals[b, :a.nnz_vec * V], B[b, :K * N].reshape(K, N))
        assert_close(host[b, :a.m * N].reshape(a.m, N), want, f"entry {b}")


def test_edge_structures(monkeypatch):
    """Empty rows, an empty matrix, a single vector-row, rows of 1 / 15 / 16 / 17 / 33 vectors."""
    for lens in ([0, 1, 15, 16, 17, 31, 32, 33, 0, 0, 64, 96, 2, 0], [0, 0, 0], [40]):
        a = custom(lens, 96, 8, seed=4)
        vals, B = spmm_inputs(a, 128, np.float16, 7, sigma=1.0)
        if vals.size == 0:
            vals = np.zeros(8, np.float16)
        got = run(a, 128, vals, B, torch.float32, True, monkeypatch)
        assert_close(got, spmm_oracle(a, 128, vals[:a.nnz_vec * 8], B), f"rows {lens}")
        for i, l in enumerate(lens):
            if l == 0:
                assert np.all(got[i * 8:(i + 1) * 8] == 0.0)


def test_non_finite_sums_and_repeated_columns_still_go_to_the_gather_kernel(monkeypatch):
    a = custom([3, 5, 17, 9], 128, 8, seed=2)
    vals, B = spmm_inputs(a, 128, np.float16, 3, sigma=1.0)
    unused = sorted(set(range(128)) - set(a.col_indices.tolist()))
    B[unused[0]] = np.inf
    got = run(a, 128, vals, B, torch.float32, True, monkeypatch)
    Bz = B.copy(); Bz[unused[0]] = 0
    assert_close(got, spmm_oracle(a, 128, vals, Bz), "unreferenced inf")
    ci = a.col_indices.copy()
    ci[1] = ci[0]
    dup = cvse.CVSE(a.m_vec, a.n, 8, a.row_offsets, ci, a.row_indices)
    vals, B = spmm_inputs(dup, 128, np.float16, 12, sigma=1.0)
    assert_close(run(dup, 128, vals, B, torch.float32, True, monkeypatch), spmm_oracle(dup, 128, vals, B), "repeated column")


@pytest.mark.parametrize("V", [1, 2, 8])
def test_transposed_product_by_pairs(V, monkeypatch):
    """vs_spmm_t through the same kernel: out [K x N] = A^T . rhs."""
    import oracle
    monkeypatch.setenv("VSPARSE_B200_SPMM_T", "dense")
    N, K = 256, 328
    a = problem(cvse.GEN_BETA, 31 + V, 520 // V if V > 1 else 520, K, V, 0.8)
    vals = cvse.fill_random((a.nnz_vec * V,), np.float16, cvse.DIST_NORMAL, 1, 0.5)
    R = cvse.fill_random((a.m, N), np.float16, cvse.DIST_NORMAL, 2, 1.0)
    want = oracle.spmm_t(a.m_vec, V, N, K, a.row_offsets, a.col_indices, vals.astype(np.float32), R.astype(np.float32))
    t_off, t_rows, t_src = (dev(x) for x in cvse.transpose(a))
    outs = []
    for pair in ("1", "0"):
        monkeypatch.setenv("VSPARSE_B200_SPMM_PAIR", pair)
        out = torch.full((K, N), float("nan"), dtype=torch.float32, device=DEV)
        ops.spmm_t(a.m_vec, V, N, K, t_off, t_rows, t_src, dev(vals), dev(R), out)
        torch.cuda.synchronize()
        assert ops.device_status() == 0
        outs.append(out.cpu().numpy())
        assert_close(outs[-1], want, f"transposed, pairs={pair}, V={V}")


def test_kernel_timing_brackets_the_multiplying_kernel(monkeypatch):
    """vs_kernel_timing: one pair of events per multiplying kernel while it is on, none after it is switched off, and
    the results are the same either way."""
    a = problem(cvse.GEN_BETA, 8, 1024 // 8, 256, 8, 0.9)
    vals, B = spmm_inputs(a, 256, np.float16, 5, sigma=0.5)
    plain = run(a, 256, vals, B, torch.float16, True, monkeypatch)
    ops.kernel_timing(True)
    timed = [run(a, 256, vals, B, torch.float16, True, monkeypatch) for _ in range(3)]
    ms, n = ops.kernel_timing(False)
    assert n == 3 and 0.0 < ms < 50.0
    assert all(np.array_equal(t, plain) for t in timed)
    run(a, 256, vals, B, torch.float16, True, monkeypatch)
    assert ops.kernel_timing(False) == (0.0, 0)
