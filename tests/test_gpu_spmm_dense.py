"""The two tensor-core SpMM kernels behind `wmmaSpmm`: the densifying kernel (zero-filled tiles of A times plain
tile loads of B) and the gather kernels (one row of B per nonzero vector).  The library chooses between them on
the device by density; VSPARSE_B200_SPMM=dense|gather (read at every call) forces one.  Both must agree with the
fp64 oracle within the tolerance of conftest.assert_close on every shape, including the ragged ones."""
import numpy as np
import pytest
import torch

from conftest import assert_close
from gpu_util import DEV, custom, dev, problem, spmm_inputs, spmm_oracle, structure
from vectorsparse_b200 import VS_PATH_TENSOR, _lib, cvse, ops

pytestmark = pytest.mark.gpu


def run(a, N, vals, B, out_dtype, mode, monkeypatch):
    if mode:
        monkeypatch.setenv("VSPARSE_B200_SPMM", mode)
    else:
        monkeypatch.delenv("VSPARSE_B200_SPMM", raising=False)
    ri, ro, ci = structure(a)
    m = a.m_vec * a.V
    out = torch.full((m * N + 64,), float("nan"), dtype=out_dtype, device=DEV)
    d_vals = dev(vals) if vals.size else torch.zeros(8, dtype=torch.float16, device=DEV)
    ops.spmm.wmmaSpmm(a.m_vec, a.V, N, a.n, ri, ro, ci, d_vals, dev(B), out)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    host = out.float().cpu().numpy()
    assert np.all(np.isnan(host[m * N:])), "wrote past the end of the output"
    return host[:m * N].reshape(m, N)


@pytest.mark.parametrize("V", [2, 4, 8])
@pytest.mark.parametrize("shape", [(256, 512, 256), (264, 200, 192), (40, 72, 64), (520, 1000, 320), (128, 64, 64)])
def test_dense_and_gather_agree_on_ragged_shapes(V, shape, monkeypatch):
    """Rows not a multiple of 256, columns of A not a multiple of 64, widths of B that leave a half tile (one box
    of B per stage instead of two)."""
    M, K, N = shape
    for s in (0.5, 0.9):
        a = problem(cvse.GEN_BETA, 7 * M + K + V, M // V, K, V, s)
        vals, B = spmm_inputs(a, N, np.float16, 5, sigma=0.5)
        want = spmm_oracle(a, N, vals, B)
        for out_t in (torch.float16, torch.float32):
            d = run(a, N, vals, B, out_t, "dense", monkeypatch)
            g = run(a, N, vals, B, out_t, "gather", monkeypatch)
            assert_close(d, want, f"dense {shape} V={V} s={s}")
            assert_close(g, want, f"gather {shape} V={V} s={s}")


def test_unsorted_columns(monkeypatch):
    """Nothing in CVSE says the columns of a vector-row are ascending: the plan buckets them whatever the order."""
    V, N = 8, 128
    a = problem(cvse.GEN_UNIFORM, 3, 64, 320, V, 0.8)
    vals, B = spmm_inputs(a, N, np.float16, 6, sigma=0.5)
    want = spmm_oracle(a, N, vals, B)
    rng = np.random.default_rng(0)
    ci = a.col_indices.copy()
    v2 = vals.reshape(-1, V).copy()
    for r in range(a.m_vec):
        lo, hi = a.row_offsets[r], a.row_offsets[r + 1]
        perm = rng.permutation(hi - lo)
        ci[lo:hi] = ci[lo:hi][perm]
        v2[lo:hi] = v2[lo:hi][perm]
    shuffled = cvse.CVSE(a.m_vec, a.n, V, a.row_offsets, ci, a.row_indices)
    for mode in ("dense", "gather"):
        assert_close(run(shuffled, N, v2.reshape(-1), B, torch.float32, mode, monkeypatch), want, f"unsorted, {mode}")


def test_empty_rows_and_empty_matrix(monkeypatch):
    for lens in ([0, 0, 5, 0, 64, 1, 0], [0, 0, 0, 0]):
        a = custom(lens, 64, 8, seed=4)
        vals, B = spmm_inputs(a, 64, np.float16, 8, sigma=1.0)
        want = spmm_oracle(a, 64, vals, B)
        for mode in ("dense", "gather", None):
            assert_close(run(a, 64, vals, B, torch.float16, mode, monkeypatch), want, f"rows {lens}, {mode}")


def test_choice_by_density(monkeypatch):
    """Left to itself the library multiplies dense tiles at 90 % sparsity and gathers rows at 99.5 %; either
    way the result is the oracle's."""
    for s in (0.9, 0.995):
        a = problem(cvse.GEN_UNIFORM, 11, 128, 2048, 8, s)
        vals, B = spmm_inputs(a, 256, np.float16, 9, sigma=0.5)
        assert_close(run(a, 256, vals, B, torch.float16, None, monkeypatch), spmm_oracle(a, 256, vals, B), f"auto, s={s}")


def test_non_finite_sums_are_redone_by_the_gather_kernel(monkeypatch):
    """0 x Inf inside a densified tile is a NaN the reference never computes: the dense kernel notices and the
    gather kernel behind it overwrites the output.  Inf in a row that IS referenced must still come through."""
    a = custom([3, 5, 17, 9], 128, 8, seed=2)
    vals, B = spmm_inputs(a, 64, np.float16, 3, sigma=1.0)
    used = sorted(set(a.col_indices.tolist()))
    unused = sorted(set(range(128)) - set(used))
    B[unused[0]] = np.inf
    got = run(a, 64, vals, B, torch.float32, "dense", monkeypatch)
    Bz = B.copy(); Bz[unused[0]] = 0
    assert_close(got, spmm_oracle(a, 64, vals, Bz), "unreferenced inf")
    B[used[0], 5] = np.inf
    got = run(a, 64, vals, B, torch.float32, "dense", monkeypatch)
    rows_hit = [r for r in range(a.m_vec) if used[0] in a.col_indices[a.row_offsets[r]:a.row_offsets[r + 1]]]
    assert rows_hit and all(not np.all(np.isfinite(got[r * 8:(r + 1) * 8, 5])) for r in rows_hit)


def test_batched_strides_streams_and_growing_scratch(monkeypatch):
    """Batch strides with padding, two streams (each keeps its own plan scratch), a larger matrix after a smaller
    one on the same stream (the scratch grows)."""
    monkeypatch.setenv("VSPARSE_B200_SPMM", "dense")
    V, N, batch = 4, 128, 3
    lib = _lib.lib()
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    results = []
    for it, (m_vec, K) in enumerate([(64, 256), (512, 1024), (32, 128)]):
        a = problem(cvse.GEN_BETA, 50 + it, m_vec, K, V, 0.7)
        vals = cvse.fill_random((batch, (a.nnz_vec * V + 7) // 8 * 8 + 8), np.float16, cvse.DIST_NORMAL, 1 + it, 0.5)
        B = cvse.fill_random((batch, K * N + 16), np.float16, cvse.DIST_NORMAL, 2 + it, 1.0)
        ri, ro, ci = structure(a)
        d_vals, d_B = dev(vals), dev(B)
        out = torch.full((batch, a.m * N + 8), float("nan"), dtype=torch.float32, device=DEV)
        st = streams[it % 2]
        st.wait_stream(torch.cuda.current_stream())
        rc = lib.vs_spmm_batched(VS_PATH_TENSOR, 0, 1, a.m_vec, V, N, K, ri.data_ptr(), ro.data_ptr(), ci.data_ptr(),
                                 d_vals.data_ptr(), d_B.data_ptr(), out.data_ptr(), batch, vals.shape[1], B.shape[1],
                                 out.shape[1], st.cuda_stream)
        assert rc == 0
        results.append((a, vals, B, out, (ri, ro, ci, d_vals, d_B)))
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    for a, vals, B, out, _ in results:
        host = out.cpu().numpy()
        assert np.all(np.isnan(host[:, a.m * N:])), "padding between batch entries was written"
        for b in range(batch):
            want = spmm_oracle(a, N, vals[b, :a.nnz_vec * V], B[b, :a.n * N].reshape(a.n, N))
            assert_close(host[b, :a.m * N].reshape(a.m, N), want, f"batched m_vec={a.m_vec} entry {b}")


def test_caller_owned_workspace(monkeypatch):
    """With a workspace set the plan goes into the caller's buffer and the library allocates nothing; a buffer that
    is too small sends the call to the gather kernels instead.  Same results either way."""
    monkeypatch.setenv("VSPARSE_B200_SPMM", "dense")
    V, N = 8, 128
    a = problem(cvse.GEN_BETA, 17, 64, 320, V, 0.8)
    vals, B = spmm_inputs(a, N, np.float16, 4, sigma=0.5)
    want = spmm_oracle(a, N, vals, B)
    need = _lib.lib().vs_spmm_workspace_bytes(a.m_vec, V, a.n, 1, 0)
    assert need > 0
    poison = 0xA5
    for size in (need, 64):
        ws = torch.full((size + 256,), poison, dtype=torch.uint8, device=DEV)
        ops.set_workspace(ws[:size])
        try:
            got = run(a, N, vals, B, torch.float32, "dense", monkeypatch)
        finally:
            ops.set_workspace(None)
        assert_close(got, want, f"caller workspace of {size} bytes")
        tail = ws[size:].cpu().numpy()
        assert np.all(tail == poison), "wrote past the end of the caller's workspace"
        used = bool((ws[:size].cpu().numpy() != poison).any())
        assert used == (size == need), "the plan must live in the caller's buffer exactly when it fits"


def test_duplicate_columns_in_a_vector_row_are_added(monkeypatch):
    """The reference's generator can pad a row with a column it already holds (include/bm_test_utils.h:70-127);
    its kernels add both values.  A dense tile has one place per (row, column), so the plan kernel reports such
    matrices and the gather kernel takes the call."""
    V, N = 8, 64
    a = custom([6, 0, 9, 4], 96, V, seed=3)
    ci = a.col_indices.copy()
    ci[1] = ci[0]                                  # vector-row 0 names its first column twice
    ci[a.row_offsets[2] + 5] = ci[a.row_offsets[2] + 2]
    dup = cvse.CVSE(a.m_vec, a.n, V, a.row_offsets, ci, a.row_indices)
    vals, B = spmm_inputs(dup, N, np.float16, 12, sigma=1.0)
    want = spmm_oracle(dup, N, vals, B)
    for mode in ("dense", "gather", None):
        assert_close(run(dup, N, vals, B, torch.float32, mode, monkeypatch), want, f"duplicate columns, {mode}")
