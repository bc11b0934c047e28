"""The two tensor-core SDDMM kernels behind `wmmaSddmm`: dense 256 x 128 tiles of lhs . rhs^T sampled at the mask,
and the row-gather kernel.  The library chooses on the host (it is given the number of mask entries);
VSPARSE_B200_SDDMM=dense|gather (read at every call) forces one.  Both must agree with the fp64 oracle within the
tolerance of conftest.assert_close, write every output exactly once and nothing else."""
import numpy as np
import pytest
import torch

from conftest import assert_close
from gpu_util import DEV, custom, dev, problem, sddmm_oracle, structure
from test_gpu_sddmm import operands, run_sddmm
from vectorsparse_b200 import VS_PATH_TENSOR, _lib, cvse, ops

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("V", [2, 4, 8])
@pytest.mark.parametrize("shape", [(256, 512, 256), (264, 200, 128), (40, 72, 64), (520, 1000, 192)])
def test_dense_and_gather_agree_on_ragged_shapes(V, shape, monkeypatch):
    """Rows not a multiple of 256, mask columns not a multiple of 128 or 32, one to four stages per tile."""
    M, n, k = shape
    for s in (0.5, 0.9):
        a = problem(cvse.GEN_BETA, 3 * M + n + V, M // V, n, V, s)
        lhs, rhs = operands(a, k, 7, 0.25)
        want = sddmm_oracle(a, k, lhs, rhs)
        for out_t in (torch.float16, torch.float32):
            for mode in ("dense", "gather"):
                monkeypatch.setenv("VSPARSE_B200_SDDMM", mode)
                assert_close(run_sddmm(VS_PATH_TENSOR, a, k, lhs, rhs, out_t), want, f"{mode} {shape} V={V} s={s}")


def test_unsorted_columns_empty_rows_and_dense_rows(monkeypatch):
    V, k = 8, 128
    a = custom([0, 300, 0, 5, 64, 1, 0, 33], 300, V, seed=6)
    rng = np.random.default_rng(1)
    ci = a.col_indices.copy()
    for r in range(a.m_vec):
        lo, hi = a.row_offsets[r], a.row_offsets[r + 1]
        ci[lo:hi] = ci[lo:hi][rng.permutation(hi - lo)]
    shuffled = cvse.CVSE(a.m_vec, a.n, V, a.row_offsets, ci, a.row_indices)
    lhs, rhs = operands(shuffled, k, 9, 0.25)
    want = sddmm_oracle(shuffled, k, lhs, rhs)
    for mode in ("dense", "gather"):
        monkeypatch.setenv("VSPARSE_B200_SDDMM", mode)
        assert_close(run_sddmm(VS_PATH_TENSOR, shuffled, k, lhs, rhs, torch.float32), want, f"unsorted, {mode}")


def test_non_finite_products_outside_the_mask_do_not_leak(monkeypatch):
    """The dense tile holds lhs-row x rhs-row products the mask never names; an Inf there must stay there."""
    V, k = 8, 64
    a = custom([3, 5, 17, 9], 128, V, seed=2)
    lhs, rhs = operands(a, k, 4, 0.25)
    unused = sorted(set(range(128)) - set(a.col_indices.tolist()))
    rhs[unused[0]] = np.inf
    rhs[unused[1]] = np.nan
    rz = rhs.copy(); rz[unused[:2]] = 0
    want = sddmm_oracle(a, k, lhs, rz)
    for mode in ("dense", "gather"):
        monkeypatch.setenv("VSPARSE_B200_SDDMM", mode)
        assert_close(run_sddmm(VS_PATH_TENSOR, a, k, lhs, rhs, torch.float32), want, f"inf outside the mask, {mode}")


def test_choice_follows_density_and_contraction_length(monkeypatch):
    """Left to itself the library takes the dense kernel at 90 % sparsity and k = 256, the gather kernel at 99.5 %
    and at k = 64; either way the result is the oracle's."""
    monkeypatch.delenv("VSPARSE_B200_SDDMM", raising=False)
    for s, k in ((0.9, 256), (0.995, 256), (0.9, 64)):
        a = problem(cvse.GEN_UNIFORM, 11, 128, 2048, 8, s)
        lhs, rhs = operands(a, k, 5, 0.25)
        assert_close(run_sddmm(VS_PATH_TENSOR, a, k, lhs, rhs, torch.float16), sddmm_oracle(a, k, lhs, rhs), f"auto s={s} k={k}")


def test_batched_with_strides(monkeypatch):
    monkeypatch.setenv("VSPARSE_B200_SDDMM", "dense")
    V, k, batch = 4, 128, 3
    a = problem(cvse.GEN_BETA, 21, 96, 320, V, 0.7)
    ri, ro, ci = structure(a)
    lhs = cvse.fill_random((batch, a.m * k + 8), np.float16, cvse.DIST_NORMAL, 1, 0.25)
    rhs = cvse.fill_random((batch, a.n * k + 16), np.float16, cvse.DIST_NORMAL, 2, 0.25)
    stride_out = (a.nnz_vec * V + 7) // 8 * 8 + 8
    out = torch.full((batch, stride_out), float("nan"), dtype=torch.float32, device=DEV)
    d_l, d_r = dev(lhs), dev(rhs)
    rc = _lib.lib().vs_sddmm_batched(VS_PATH_TENSOR, 0, 1, a.m_vec, k, a.n, a.nnz_vec, ri.data_ptr(), ro.data_ptr(),
                                     ci.data_ptr(), d_l.data_ptr(), d_r.data_ptr(), out.data_ptr(), V, batch,
                                     lhs.shape[1], rhs.shape[1], stride_out, torch.cuda.current_stream().cuda_stream, 1)
    assert rc == 0
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    host = out.cpu().numpy()
    nnz = a.nnz_vec * V
    assert np.all(np.isnan(host[:, nnz:])), "padding between batch entries was written"
    for b in range(batch):
        want = sddmm_oracle(a, k, lhs[b, :a.m * k].reshape(a.m, k), rhs[b, :a.n * k].reshape(a.n, k))
        assert_close(host[b, :nnz], want, f"batched entry {b}")
