"""vs_spmm_t: out = A^T . rhs for a CVSE matrix A, against the fp64 oracle within conftest.assert_close.  Every test
runs three times: with the tensor-core kernel forced (A^T as one-value vectors through the densifying SpMM kernel),
with the CUDA-core kernel forced, and with the library's own choice (VSPARSE_B200_SPMM_T, read at every call)."""
import numpy as np
import pytest
import torch

import oracle
from conftest import assert_close
from gpu_util import DEV, custom, dev, problem
from vectorsparse_b200 import _lib, cvse, ops

pytestmark = pytest.mark.gpu


@pytest.fixture(params=["dense", "gather", None], autouse=True)
def kernel_choice(request, monkeypatch):
    if request.param:
        monkeypatch.setenv("VSPARSE_B200_SPMM_T", request.param)
    else:
        monkeypatch.delenv("VSPARSE_B200_SPMM_T", raising=False)
    return request.param


def t_structure(a):
    t_off, t_rows, t_src = cvse.transpose(a)
    if t_rows.size == 0:   # keep valid pointers for an empty matrix
        t_rows = np.zeros(4, np.int32)
        t_src = np.zeros(4, np.int32)
    return dev(t_off), dev(t_rows), dev(t_src)


def inputs(a, N, seed, sigma=0.5):
    vals = cvse.fill_random((a.nnz_vec * a.V,), np.float16, cvse.DIST_NORMAL, seed, sigma)
    B = cvse.fill_random((a.m_vec * a.V, N), np.float16, cvse.DIST_NORMAL, seed + 1, 1.0)
    return vals, B


def want_of(a, N, vals, B):
    return oracle.spmm_t(a.m_vec, a.V, N, a.n, a.row_offsets, a.col_indices, vals.astype(np.float32), B.astype(np.float32))


def run(a, N, vals, B, out_dtype):
    t_off, t_rows, t_src = t_structure(a)
    out = torch.full((a.n * N + 64,), float("nan"), dtype=out_dtype, device=DEV)
    d_vals = dev(vals) if vals.size else torch.zeros(8, dtype=torch.float16, device=DEV)
    ops.spmm_t(a.m_vec, a.V, N, a.n, t_off, t_rows, t_src, d_vals, dev(B), out)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    host = out.float().cpu().numpy()
    assert np.all(np.isnan(host[a.n * N:])), "wrote past the end of the output"
    return host[:a.n * N].reshape(a.n, N)


@pytest.mark.parametrize("V", [1, 2, 4, 8])
@pytest.mark.parametrize("shape", [(256, 512, 256), (264, 200, 192), (40, 72, 8), (128, 67, 520)])
def test_against_oracle(V, shape):
    """Widths of one chunk, less than a chunk, eight columns, and more than two chunks with a ragged tail; column
    counts that are not a multiple of the rows a CTA takes."""
    M, K, N = shape
    for s in (0.5, 0.9):
        a = problem(cvse.GEN_BETA, 3 * M + K + V, M // V, K, V, s)
        vals, B = inputs(a, N, 9)
        want = want_of(a, N, vals, B)
        for out_t in (torch.float16, torch.float32):
            assert_close(run(a, N, vals, B, out_t), want, f"spmm_t {shape} V={V} s={s} {out_t}")


def test_columns_nobody_names_and_empty_matrix():
    for lens in ([0, 3, 0, 40, 1], [0, 0, 0]):
        a = custom(lens, 48, 8, seed=2)
        vals, B = inputs(a, 64, 4)
        got = run(a, 64, vals, B, torch.float32)
        assert_close(got, want_of(a, 64, vals, B), f"rows {lens}")
        named = np.zeros(48, bool)
        named[a.col_indices] = True
        assert np.all(got[~named] == 0.0), "a column without nonzero vectors must give a row of zeros"


def test_long_column_lists():
    """A column named by every vector-row: several 32-entry index batches and an odd tail."""
    a = custom([7] * 75, 7, 4, seed=0)
    vals, B = inputs(a, 128, 6)
    assert_close(run(a, 128, vals, B, torch.float16), want_of(a, 128, vals, B), "dense columns")


def test_batched_with_shared_and_strided_operands():
    V, N, batch = 8, 64, 5
    a = problem(cvse.GEN_BETA, 21, 32, 96, V, 0.8)
    t_off, t_rows, t_src = t_structure(a)
    vals = cvse.fill_random((batch, a.nnz_vec * V), np.float16, cvse.DIST_NORMAL, 1, 0.5)
    B = cvse.fill_random((batch, a.m_vec * V, N), np.float16, cvse.DIST_NORMAL, 2, 1.0)
    out = torch.empty((batch, a.n, N), dtype=torch.float32, device=DEV)
    ops.spmm_t(a.m_vec, V, N, a.n, t_off, t_rows, t_src, dev(vals), dev(B), out)
    shared = torch.empty((batch, a.n, N), dtype=torch.float32, device=DEV)
    ops.spmm_t(a.m_vec, V, N, a.n, t_off, t_rows, t_src, dev(vals[0]), dev(B), shared)
    torch.cuda.synchronize()
    for b in range(batch):
        assert_close(out[b].cpu().numpy(), want_of(a, N, vals[b], B[b]), f"batch entry {b}")
        assert_close(shared[b].cpu().numpy(), want_of(a, N, vals[0], B[b]), f"shared values, entry {b}")


def test_runs_are_bit_identical():
    a = problem(cvse.GEN_UNIFORM, 8, 64, 256, 4, 0.9)
    vals, B = inputs(a, 256, 3)
    first = run(a, 256, vals, B, torch.float32)
    assert np.array_equal(first, run(a, 256, vals, B, torch.float32))


def test_a_column_named_twice_by_one_vector_row_is_added_twice():
    """Two vectors of one vector-row in the same column are two entries of A^T at the same place: the tensor-core
    kernel's tile has room for one, so the plan kernel sends such a matrix to the CUDA-core kernel."""
    a = custom([6, 0, 9, 4], 96, 8, seed=3)
    ci = a.col_indices.copy()
    ci[1] = ci[0]
    ci[a.row_offsets[2] + 5] = ci[a.row_offsets[2] + 2]
    dup = cvse.CVSE(a.m_vec, a.n, 8, a.row_offsets, ci, a.row_indices)
    vals, B = inputs(dup, 64, 12, sigma=1.0)
    assert_close(run(dup, 64, vals, B, torch.float32), want_of(dup, 64, vals, B), "repeated column")


def test_non_finite_rows_nobody_reads_do_not_leak():
    """A row of rhs that belongs to a vector-row without nonzeros is never read by the sum; a dense tile would
    multiply it by zero.  An Inf there must not turn into NaNs in the output."""
    a = custom([5, 0, 7, 3], 40, 4, seed=6)
    vals, B = inputs(a, 64, 2)
    B = B.copy()
    B[4:8] = np.float16(np.inf)          # the rows of vector-row 1, which is empty
    want = want_of(a, 64, vals, np.where(np.isfinite(B), B, 0).astype(np.float16))
    got = run(a, 64, vals, B, torch.float32)
    assert np.all(np.isfinite(got))
    assert_close(got, want, "Inf in an unread row")


def test_argument_errors():
    L = _lib.lib()
    z = torch.zeros(64, dtype=torch.float16, device=DEV)
    i = torch.zeros(64, dtype=torch.int32, device=DEV)
    p = lambda t: t.data_ptr()
    assert L.vs_spmm_t(_lib.VS_F16, _lib.VS_F16, 2, 3, 8, 4, p(i), p(i), p(i), p(z), p(z), p(z), None) == -1   # vector length
    assert L.vs_spmm_t(_lib.VS_F32, _lib.VS_F32, 2, 4, 8, 4, p(i), p(i), p(i), p(z), p(z), p(z), None) == -2   # dtype
    assert L.vs_spmm_t(_lib.VS_F16, _lib.VS_F16, 2, 4, 12, 4, p(i), p(i), p(i), p(z), p(z), p(z), None) == -3  # width % 8
    assert L.vs_spmm_t(_lib.VS_F16, _lib.VS_F16, 2, 4, 8, 4, None, p(i), p(i), p(z), p(z), p(z), None) == -4   # null
    assert L.vs_spmm_t(_lib.VS_F16, _lib.VS_F16, 2, 4, 8, 4, p(i), p(i), p(i), p(z) + 2, p(z), p(z), None) == -5  # alignment
