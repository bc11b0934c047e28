"""SDDMM, masked softmax and fixed-mask attention parity on the GPU, through the C ABI, against the fp64 oracle.

Values: rel-L2 <= 5e-3 and max-abs <= 2e-2 (fp16 inputs, fp32 accumulation).  Structure: the index arrays are
inputs and must come back byte-identical; exactly nnz_vec * V outputs are written, each once."""
import numpy as np
import pytest
import torch

import oracle
from conftest import assert_close
from gpu_util import DEV, custom, dev, problem, sddmm_oracle, structure
from vectorsparse_b200 import VS_PATH_CUDA_CORE, VS_PATH_TENSOR, VsError, cvse, ops

pytestmark = pytest.mark.gpu


def run_sddmm(path, a, k, lhs, rhs, out_dtype, algorithm=1):
    ri, ro, ci = structure(a)
    before = [t.clone() for t in (ri, ro, ci)]
    nnz = a.nnz_vec * a.V
    out = torch.full((nnz + 64,), float("nan"), dtype=out_dtype, device=DEV)
    if path == VS_PATH_TENSOR:
        ops.sddmm.wmmaSddmm(a.m_vec, k, a.n, a.nnz_vec, ri, ro, ci, dev(lhs), dev(rhs), out, a.V, None, algorithm)
    else:
        ops.sddmm.cudaSddmm(a.m_vec, k, a.n, a.nnz_vec, ri, ro, ci, dev(lhs), dev(rhs), out, a.V, None)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    for b, t in zip(before, (ri, ro, ci)):
        assert torch.equal(b, t), "structure arrays were modified"
    host = out.float().cpu().numpy()
    assert np.all(np.isnan(host[nnz:])), "wrote past the end of the output"
    assert not np.any(np.isnan(host[:nnz])), "an output slot was never written"
    return host[:nnz]


def operands(a, k, seed, sigma=1.0):
    lhs = cvse.fill_random((a.m, k), np.float16, cvse.DIST_NORMAL, seed, sigma)
    rhs = cvse.fill_random((a.n, k), np.float16, cvse.DIST_NORMAL, seed + 1, sigma)
    return lhs, rhs


@pytest.mark.parametrize("V", [1, 2, 4, 8])
@pytest.mark.parametrize("out_t", [torch.float16, torch.float32])
def test_cuda_core_all_vector_lengths(V, out_t):
    a = problem(cvse.GEN_BETA, 30 + V, 96, 200, V, 0.8)
    for k in (64, 72, 256):
        lhs, rhs = operands(a, k, 3, 0.25)
        got = run_sddmm(VS_PATH_CUDA_CORE, a, k, lhs, rhs, out_t)
        assert_close(got, sddmm_oracle(a, k, lhs, rhs), f"cuda-core V={V} k={k}")


@pytest.mark.parametrize("V", [2, 4, 8])
@pytest.mark.parametrize("out_t", [torch.float16, torch.float32])
@pytest.mark.parametrize("k", [64, 128, 256])
def test_tensor_path(V, out_t, k):
    a = problem(cvse.GEN_BETA, 40 + V, 64, 300, V, 0.5)  # rows of 0..300 entries: up to three tiles each
    lhs, rhs = operands(a, k, 5, 0.25)
    got = run_sddmm(VS_PATH_TENSOR, a, k, lhs, rhs, out_t)
    assert_close(got, sddmm_oracle(a, k, lhs, rhs), f"tensor V={V} k={k}")


def test_all_algorithm_values_give_the_same_correct_result():
    a = problem(cvse.GEN_BETA, 5, 32, 128, 8, 0.7)
    lhs, rhs = operands(a, 64, 9, 0.25)
    base = run_sddmm(VS_PATH_TENSOR, a, 64, lhs, rhs, torch.float32, 0)
    assert_close(base, sddmm_oracle(a, 64, lhs, rhs), "alg 0")
    for alg in (1, 2, 3):
        assert np.array_equal(base, run_sddmm(VS_PATH_TENSOR, a, 64, lhs, rhs, torch.float32, alg))
    ri, ro, ci = structure(a)
    with pytest.raises(VsError):
        ops.sddmm.wmmaSddmm(a.m_vec, 64, a.n, a.nnz_vec, ri, ro, ci, dev(lhs), dev(rhs),
                            torch.zeros(a.nnz_vec * 8, device=DEV), 8, None, 4)


@pytest.mark.parametrize("path", [VS_PATH_TENSOR, VS_PATH_CUDA_CORE])
def test_golden_fixtures(golden, path):
    for name, c in golden.items():
        V, k = c["V"], c["k"]
        if c["row_offsets"][-1] == 0 or (path == VS_PATH_TENSOR and (V == 1 or k % 64)):
            continue
        a = cvse.CVSE(c["m_vec"], c["K"], V, c["row_offsets"], c["col_indices"], cvse.row_swizzle(c["row_offsets"]))
        got = run_sddmm(path, a, k, c["lhs16"], c["rhs16"], torch.float32)
        assert_close(got, c["f64_sddmm_h16"], name)
        assert np.all(np.abs(got - c["ref_sddmm_h16"]) <= 0.5), name  # the reference's own criterion


@pytest.mark.parametrize("path", [VS_PATH_TENSOR, VS_PATH_CUDA_CORE])
def test_edge_rows(path):
    lens = [0, 1, 127, 128, 129, 0, 0, 255, 256, 257, 3, 0]
    a = custom(lens, 300, 8, seed=2)
    lhs, rhs = operands(a, 64, 4, 0.25)
    assert_close(run_sddmm(path, a, 64, lhs, rhs, torch.float16), sddmm_oracle(a, 64, lhs, rhs), "edge rows")
    # an empty mask launches nothing and succeeds
    e = custom([0, 0], 16, 8)
    ri, ro, ci = structure(e)
    z = torch.zeros(16 * 64, dtype=torch.float16, device=DEV)
    fn = ops.sddmm.wmmaSddmm if path == VS_PATH_TENSOR else ops.sddmm.cudaSddmm
    args = (2, 64, 16, 0, ri, ro, ci, z, z, z, 8, None) + ((1,) if path == VS_PATH_TENSOR else ())
    assert fn(*args) == 0


@pytest.mark.parametrize("MK", [(64, 64), (256, 576), (512, 2048), (1024, 256), (2048, 512)])
@pytest.mark.parametrize("V", [2, 4, 8])
def test_config3_shapes(MK, V):
    """Same masks as the SpMM sweep; lhs M x 256, rhs K x 256, N(0,1) fp16."""
    M, K = MK
    for s in (0.5, 0.7, 0.8, 0.9, 0.95, 0.98):
        a = problem(cvse.GEN_BETA, 1000 + M + int(s * 100), M // V, K, V, s)
        lhs, rhs = operands(a, 256, 21, 1.0)
        want = sddmm_oracle(a, 256, lhs, rhs)
        # N(0,1) operands with k = 256: outputs ~ N(0, 16); fp16 output rounding alone is ~1e-2 absolute, so the
        # absolute bound is checked on the fp32 output and the relative bound on both
        got32 = run_sddmm(VS_PATH_TENSOR, a, 256, lhs, rhs, torch.float32)
        assert_close(got32, want, f"cfg3 {MK} V={V} s={s}")
        got16 = run_sddmm(VS_PATH_TENSOR, a, 256, lhs, rhs, torch.float16)
        assert np.linalg.norm(got16 - want) <= 5e-3 * np.linalg.norm(want)
        assert np.array_equal(got16, got32.astype(np.float16).astype(np.float32))  # same sums, rounded once
        assert_close(run_sddmm(VS_PATH_CUDA_CORE, a, 256, lhs, rhs, torch.float32), want, f"cfg3 cc {MK} V={V}")


@pytest.mark.parametrize("path", [VS_PATH_TENSOR, VS_PATH_CUDA_CORE])
def test_row_order_and_batching_are_bit_exact(path):
    V, k, batch = 8, 64, 3
    a = problem(cvse.GEN_BETA, 8, 96, 400, V, 0.8, sort=True)
    ident = cvse.CVSE(a.m_vec, a.n, V, a.row_offsets, a.col_indices, cvse.row_swizzle(a.row_offsets, sort=False))
    lhs = cvse.fill_random((batch, a.m, k), np.float16, cvse.DIST_NORMAL, 1, 0.25)
    rhs = cvse.fill_random((batch, a.n, k), np.float16, cvse.DIST_NORMAL, 2, 0.25)
    single = [run_sddmm(path, a, k, lhs[b], rhs[b], torch.float16) for b in range(batch)]
    assert np.array_equal(single[0], run_sddmm(path, ident, k, lhs[0], rhs[0], torch.float16))
    ri, ro, ci = structure(a)
    out = torch.empty((batch, a.nnz_vec * V), dtype=torch.float16, device=DEV)
    ops.sddmm_batched(path, a.m_vec, k, a.n, a.nnz_vec, ri, ro, ci, dev(lhs), dev(rhs), out, V)
    torch.cuda.synchronize()
    for b in range(batch):
        assert np.array_equal(out[b].float().cpu().numpy(), single[b])


@pytest.mark.parametrize("V", [1, 2, 4, 8])
@pytest.mark.parametrize("dt", [torch.float16, torch.float32])
def test_softmax(V, dt):
    a = custom([0, 1, 5, 33, 64, 100, 0, 7], 128, V, seed=3)
    nnz = a.nnz_vec * V
    scores = cvse.fill_random((2, nnz), np.float32, cvse.DIST_NORMAL, 4, 3.0)
    if dt == torch.float16:
        scores = scores.astype(np.float16)
    ri, ro, ci = structure(a)
    d_s = dev(scores)
    d_p = torch.full_like(d_s, float("nan"))
    ops.softmax_cvse(a.m_vec, V, ri, ro, d_s, d_p, 0.125)
    torch.cuda.synchronize()
    for b in range(2):
        want = oracle.softmax(a.m_vec, V, a.row_offsets, scores[b].astype(np.float32), 0.125)
        assert_close(d_p[b].float().cpu().numpy(), want, "softmax")
    # in place
    ops.softmax_cvse(a.m_vec, V, ri, ro, d_s, d_s, 0.125)
    torch.cuda.synchronize()
    assert torch.equal(d_s, d_p)


@pytest.mark.parametrize("path", [VS_PATH_TENSOR, VS_PATH_CUDA_CORE])
def test_attention_small(path):
    """SDDMM -> softmax(1/sqrt(d)) -> SpMM on a band + strided mask, 3 heads sharing it."""
    V, d, n, heads = 8, 64, 512, 3
    a = problem(cvse.GEN_BAND, 6, n // V, n, V, 0.8, band=64)
    q = cvse.fill_random((heads, n, d), np.float16, cvse.DIST_NORMAL, 1, 1.0)
    k = cvse.fill_random((heads, n, d), np.float16, cvse.DIST_NORMAL, 2, 1.0)
    v = cvse.fill_random((heads, n, d), np.float16, cvse.DIST_NORMAL, 3, 1.0)
    ri, ro, ci = structure(a)
    out = torch.empty((heads, n, d), dtype=torch.float16, device=DEV)
    ws = torch.empty((heads, a.nnz_vec * V), dtype=torch.float16, device=DEV)
    ops.attention_cvse(path, a.m_vec, V, n, d, a.nnz_vec, ri, ro, ci, dev(q), dev(k), dev(v), out, ws, 0.125)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    for h in range(heads):
        want = oracle.attention(a.m_vec, V, d, d, a.row_offsets, a.col_indices, q[h].astype(np.float32),
                                k[h].astype(np.float32), v[h].astype(np.float32), 0.125)
        assert_close(out[h].float().cpu().numpy(), want, f"attention head {h}")


def test_software_gather_kernel_for_strides_tma_cannot_address():
    """Batch strides that are not multiples of k fall back to the cp.async tensor-core SDDMM."""
    V, k, batch = 8, 64, 2
    a = problem(cvse.GEN_BETA, 17, 40, 200, V, 0.5)
    lhs = cvse.fill_random((batch, a.m, k), np.float16, cvse.DIST_NORMAL, 1, 0.25)
    rhs = cvse.fill_random((batch, a.n, k), np.float16, cvse.DIST_NORMAL, 2, 0.25)
    pad = 8
    fl = torch.zeros((batch, a.m * k + pad), dtype=torch.float16, device=DEV)
    fr = torch.zeros((batch, a.n * k + pad), dtype=torch.float16, device=DEV)
    fl[:, :a.m * k] = dev(lhs).reshape(batch, -1)
    fr[:, :a.n * k] = dev(rhs).reshape(batch, -1)
    ri, ro, ci = structure(a)
    nnz = a.nnz_vec * V
    out = torch.empty((batch, nnz), dtype=torch.float32, device=DEV)
    from vectorsparse_b200 import _lib
    rc = _lib.lib().vs_sddmm_batched(VS_PATH_TENSOR, 0, 1, a.m_vec, k, a.n, a.nnz_vec, ri.data_ptr(), ro.data_ptr(),
                                     ci.data_ptr(), fl.data_ptr(), fr.data_ptr(), out.data_ptr(), V, batch,
                                     a.m * k + pad, a.n * k + pad, nnz, torch.cuda.current_stream().cuda_stream, 1)
    assert rc == 0
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    for b in range(batch):
        assert_close(out[b].cpu().numpy(), sddmm_oracle(a, k, lhs[b], rhs[b]), f"software gather, entry {b}")


@pytest.mark.parametrize("path", [VS_PATH_TENSOR])
def test_attention_config5_full_size(path):
    """The configured size of the fixed-mask attention workload: sequence 4096, head dimension 64, V = 8, a band of
    256 plus strided vectors at 90 % sparsity (410 entries per row), scale 1/8 — two heads sharing the mask, forward,
    against the fp64 oracle of the whole pipeline."""
    V, d, n, heads = 8, 64, 4096, 2
    a = problem(cvse.GEN_BAND, 2026, n // V, n, V, 0.9, band=256)
    assert abs(a.nnz_vec / a.m_vec - 410) <= 1
    q, k, v = (cvse.fill_random((heads, n, d), np.float16, cvse.DIST_NORMAL, 31 + i, 1.0) for i in range(3))
    ri, ro, ci = structure(a)
    out = torch.full((heads, n, d), float("nan"), dtype=torch.float16, device=DEV)
    ws = torch.empty((heads, a.nnz_vec * V), dtype=torch.float16, device=DEV)
    ops.attention_cvse(path, a.m_vec, V, n, d, a.nnz_vec, ri, ro, ci, dev(q), dev(k), dev(v), out, ws, 0.125)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    for h in range(heads):
        want = oracle.attention(a.m_vec, V, d, d, a.row_offsets, a.col_indices, q[h].astype(np.float32),
                                k[h].astype(np.float32), v[h].astype(np.float32), 0.125)
        assert_close(out[h].float().cpu().numpy(), want, f"config 5, head {h}")


def test_attention_with_an_empty_mask_writes_zeros():
    """No mask entries and no workspace: the output rows are zero (nothing to average), nothing else is touched."""
    V, d, n, heads = 8, 64, 128, 2
    a = custom([0] * (n // V), n, V)
    ri, ro, ci = structure(a)
    q = torch.ones((heads, n, d), dtype=torch.float16, device=DEV)
    out = torch.full((heads * n * d + 64,), float("nan"), dtype=torch.float16, device=DEV)
    from vectorsparse_b200 import _lib
    import ctypes as C
    rc = _lib.lib().vs_attention_cvse(VS_PATH_TENSOR, a.m_vec, V, n, d, 0, ri.data_ptr(), ro.data_ptr(), ci.data_ptr(), q.data_ptr(),
                                      q.data_ptr(), q.data_ptr(), out.data_ptr(), None, C.c_float(0.125), heads,
                                      torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    host = out.float().cpu().numpy()
    assert np.all(host[:heads * n * d] == 0.0) and np.all(np.isnan(host[heads * n * d:]))
