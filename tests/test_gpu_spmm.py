"""SpMM parity on the GPU, through the C ABI (ctypes -> libvsparse_b200.so), against the fp64 oracle.

Tolerance (floating point): rel-L2 <= 5e-3 and max-abs <= 2e-2 with fp16 inputs / fp32 accumulation, checked by
conftest.assert_close.  Structure-independent properties (row order, batching, column sharding) are bit-exact."""
import numpy as np
import pytest
import torch

from conftest import assert_close
from gpu_util import DEV, custom, dev, problem, spmm_inputs, spmm_oracle, structure
from vectorsparse_b200 import VS_PATH_CUDA_CORE, VS_PATH_TENSOR, VsError, cvse, ops

pytestmark = pytest.mark.gpu

FN = {VS_PATH_TENSOR: ops.spmm.wmmaSpmm, VS_PATH_CUDA_CORE: ops.spmm.cudaSpmm}


def run_spmm(path, a, N, vals, B, out_dtype):
    ri, ro, ci = structure(a)
    m = a.m_vec * a.V
    out = torch.full((m * N + 64,), float("nan"), dtype=out_dtype, device=DEV)
    d_vals = dev(vals) if vals.size else torch.zeros(8, dtype=dev(B).dtype, device=DEV)
    FN[path](a.m_vec, a.V, N, a.n, ri, ro, ci, d_vals, dev(B), out)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    host = out.float().cpu().numpy()
    assert np.all(np.isnan(host[m * N:])), "wrote past the end of the output"
    return host[:m * N].reshape(m, N)


def test_config1_fp32_cuda_core():
    """fp32, A 256x256 V=4, 90% of the vectors zero, values N(0,1), B 256x128 U(-1,1), seed 0."""
    for sort in (False, True):
        a = problem(cvse.GEN_FIXED, 0, 64, 256, 4, 0.9, sort=sort)
        vals = cvse.fill_random((a.nnz_vec * 4,), np.float32, cvse.DIST_NORMAL, 0, 1.0)
        B = cvse.fill_random((256, 128), np.float32, cvse.DIST_UNIFORM, 1)
        got = run_spmm(VS_PATH_CUDA_CORE, a, 128, vals, B, torch.float32)
        want = spmm_oracle(a, 128, vals, B)
        assert_close(got, want, "config 1")
        assert np.max(np.abs(got - want)) < 1e-4  # fp32 in and out: far inside the tolerance


@pytest.mark.parametrize("V", [1, 2, 4, 8])
@pytest.mark.parametrize("dt", ["f32", "f16f16", "f16f32"])
def test_cuda_core_all_vector_lengths(V, dt):
    in_np = np.float32 if dt == "f32" else np.float16
    out_t = torch.float16 if dt == "f16f16" else torch.float32
    a = problem(cvse.GEN_BETA, 10 + V, 96, 200, V, 0.8)
    N = 72 if dt != "f32" else 68  # not a multiple of 64: only 16-byte chunks are required on this path
    vals, B = spmm_inputs(a, N, in_np, 3, sigma=0.5)
    got = run_spmm(VS_PATH_CUDA_CORE, a, N, vals, B, out_t)
    assert_close(got, spmm_oracle(a, N, vals, B), f"cuda-core V={V} {dt}")


@pytest.mark.parametrize("V", [2, 4, 8])
@pytest.mark.parametrize("out_t", [torch.float16, torch.float32])
@pytest.mark.parametrize("N", [64, 128, 192, 256])
def test_tensor_path_vector_lengths_and_widths(V, out_t, N):
    a = problem(cvse.GEN_BETA, 20 + V, 64, 160, V, 0.7)
    vals, B = spmm_inputs(a, N, np.float16, 5, sigma=0.5)
    got = run_spmm(VS_PATH_TENSOR, a, N, vals, B, out_t)
    assert_close(got, spmm_oracle(a, N, vals, B), f"tensor V={V} N={N}")


@pytest.mark.parametrize("path", [VS_PATH_TENSOR, VS_PATH_CUDA_CORE])
def test_golden_fixtures(golden, path):
    """The committed reference-host vectors: same inputs through the GPU path."""
    for name, c in golden.items():
        V, N = c["V"], c["N"]
        if path == VS_PATH_TENSOR and (V == 1 or N % 64):
            continue
        a = cvse.CVSE(c["m_vec"], c["K"], V, c["row_offsets"], c["col_indices"], cvse.row_swizzle(c["row_offsets"]))
        got = run_spmm(path, a, N, c["values16"], c["B16"], torch.float32)
        assert_close(got, c["f64_spmm_h16"], name)
        # and the reference's own criterion: within 0.5 of its fp32 host loop (spmm_benchmark.cpp:214)
        assert np.all(np.abs(got - c["ref_spmm_h16"]) <= 0.5), name


@pytest.mark.parametrize("path", [VS_PATH_TENSOR, VS_PATH_CUDA_CORE])
def test_edge_rows(path):
    """Empty rows (their C rows must be zeros), single entries, 15/16/17/31/32/33 tails, a full row."""
    lens = [0, 1, 15, 16, 17, 31, 32, 33, 0, 0, 64, 96, 2, 0]
    a = custom(lens, 96, 8, seed=4)
    vals, B = spmm_inputs(a, 128, np.float16, 7, sigma=1.0)
    got = run_spmm(path, a, 128, vals, B, torch.float32)
    assert_close(got, spmm_oracle(a, 128, vals, B), "edge rows")
    for i, l in enumerate(lens):
        if l == 0:
            assert np.all(got[i * 8:(i + 1) * 8] == 0.0)
    # a matrix with no nonzeros at all
    e = custom([0, 0, 0], 32, 8)
    got = run_spmm(path, e, 64, np.zeros(0, np.float16), np.ones((32, 64), np.float16), torch.float16)
    assert np.all(got == 0.0)
    # one vector-row
    s = custom([40], 40, 8)
    vals, B = spmm_inputs(s, 64, np.float16, 9, sigma=1.0)
    assert_close(run_spmm(path, s, 64, vals, B, torch.float16), spmm_oracle(s, 64, vals, B), "single row")


def test_inf_in_unreferenced_row_does_not_leak():
    """A dense row that no nonzero references may hold Inf/NaN; zero padding must not turn it into NaNs."""
    a = custom([3, 5, 17], 64, 8, seed=1)
    vals, B = spmm_inputs(a, 64, np.float16, 2, sigma=1.0)
    unused = sorted(set(range(64)) - set(a.col_indices.tolist()))
    B[unused[0]] = np.inf
    B[unused[1]] = np.nan
    for path in (VS_PATH_TENSOR, VS_PATH_CUDA_CORE):
        got = run_spmm(path, a, 64, vals, B, torch.float32)
        Bz = B.copy(); Bz[unused[:2]] = 0
        assert_close(got, spmm_oracle(a, 64, vals, Bz), "unreferenced inf")


@pytest.mark.parametrize("MK", [(64, 64), (256, 576), (512, 2048), (1024, 256), (2048, 512)])
@pytest.mark.parametrize("V", [2, 4, 8])
def test_config2_shapes(MK, V):
    """ResNet-50-like layer shapes, Beta(2,2)-skewed rows, values N(0, 0.02), B N(0,1), N = 256."""
    M, K = MK
    for s in (0.5, 0.7, 0.8, 0.9, 0.95, 0.98):
        a = problem(cvse.GEN_BETA, 1000 + M + int(s * 100), M // V, K, V, s)
        vals, B = spmm_inputs(a, 256, np.float16, 11, sigma=0.02)
        want = spmm_oracle(a, 256, vals, B)
        for out_t in (torch.float16, torch.float32):
            assert_close(run_spmm(VS_PATH_TENSOR, a, 256, vals, B, out_t), want, f"cfg2 {MK} V={V} s={s}")
        assert_close(run_spmm(VS_PATH_CUDA_CORE, a, 256, vals, B, torch.float16), want, f"cfg2 cc {MK} V={V} s={s}")


@pytest.mark.parametrize("V", [1, 4])
def test_config4_full_size_fp32(V):
    """M = K = 4096, uniform random positions, values and B U(-1,1), N = 256, against the oracle."""
    a = problem(cvse.GEN_UNIFORM, 40 + V, 4096 // V, 4096, V, 0.9)
    vals, B = spmm_inputs(a, 256, np.float32, 13)
    got = run_spmm(VS_PATH_CUDA_CORE, a, 256, vals, B, torch.float32)
    assert_close(got, spmm_oracle(a, 256, vals, B), f"cfg4 V={V}")


@pytest.mark.parametrize("V", [1, 4])
@pytest.mark.parametrize("N", [1024, 8192])
@pytest.mark.parametrize("s", [0.8, 0.95])
def test_config4_wide_dense_operands(V, N, s):
    """M = K = 4096, fp32, N = 1024 and 8192 (B and C of 134 MB each at 8192: element offsets beyond 2^24 in every
    direction), sparsity 0.8 and 0.95, every output compared with the fp64 oracle.  At N = 8192 a size-independent
    property is checked as well: the product is linear in B, so C restricted to a column block must equal the
    product with that block of B alone, bit for bit (first, middle and last 256 columns)."""
    a = problem(cvse.GEN_UNIFORM, 400 + V + int(s * 100), 4096 // V, 4096, V, s)
    vals = cvse.fill_random((a.nnz_vec * V,), np.float32, cvse.DIST_UNIFORM, 13)
    B = cvse.fill_random((4096, N), np.float32, cvse.DIST_UNIFORM, 14, 1.0)
    got = run_spmm(VS_PATH_CUDA_CORE, a, N, vals, B, torch.float32)
    assert_close(got, spmm_oracle(a, N, vals, B, threads=16), f"cfg4 V={V} N={N} s={s}")
    if N == 8192:
        for c0 in (0, N // 2 - 128, N - 256):
            part = run_spmm(VS_PATH_CUDA_CORE, a, 256, vals, np.ascontiguousarray(B[:, c0:c0 + 256]), torch.float32)
            assert np.array_equal(part, got[:, c0:c0 + 256]), f"column block at {c0}"


@pytest.mark.parametrize("path,dt", [(VS_PATH_TENSOR, np.float16), (VS_PATH_CUDA_CORE, np.float16), (VS_PATH_CUDA_CORE, np.float32)])
def test_row_order_batching_and_column_shards_are_bit_exact(path, dt):
    """Properties that hold at any size: the row swizzle never changes a bit; a batched launch equals separate
    launches; computing a column slice of B alone equals the slice of the full product."""
    V, N, batch = 8, 256, 3
    a_sorted = problem(cvse.GEN_BETA, 77, 128, 512, V, 0.9, sort=True)
    a_ident = cvse.CVSE(a_sorted.m_vec, a_sorted.n, V, a_sorted.row_offsets, a_sorted.col_indices,
                        cvse.row_swizzle(a_sorted.row_offsets, sort=False))
    out_t = torch.float16 if dt == np.float16 else torch.float32
    vals = cvse.fill_random((batch, a_sorted.nnz_vec * V), dt, cvse.DIST_NORMAL, 1, 0.5)
    B = cvse.fill_random((batch, 512, N), dt, cvse.DIST_NORMAL, 2, 1.0)
    full = [run_spmm(path, a_sorted, N, vals[b], B[b], out_t) for b in range(batch)]
    assert np.array_equal(full[0], run_spmm(path, a_ident, N, vals[0], B[0], out_t))
    # batched
    ri, ro, ci = structure(a_sorted)
    out = torch.empty((batch, a_sorted.m, N), dtype=out_t, device=DEV)
    ops.spmm_batched(path, a_sorted.m_vec, V, N, 512, ri, ro, ci, dev(vals), dev(B), out)
    torch.cuda.synchronize()
    for b in range(batch):
        assert np.array_equal(out[b].float().cpu().numpy(), full[b])
    # shared values (stride 0) with per-batch B
    ops.spmm_batched(path, a_sorted.m_vec, V, N, 512, ri, ro, ci, dev(vals[0]), dev(B), out)
    torch.cuda.synchronize()
    assert np.array_equal(out[0].float().cpu().numpy(), full[0])
    # column shards: two halves of B, each computed alone
    for g in range(2):
        Bs = np.ascontiguousarray(B[0][:, g * 128:(g + 1) * 128])
        part = run_spmm(path, a_sorted, 128, vals[0], Bs, out_t)
        assert np.array_equal(part, full[0][:, g * 128:(g + 1) * 128])


def test_rejected_arguments_raise():
    a = custom([2, 2], 16, 8)
    ri, ro, ci = structure(a)
    v = torch.zeros(64, dtype=torch.float16, device=DEV)
    B = torch.zeros(16 * 64, dtype=torch.float16, device=DEV)
    out = torch.zeros(16 * 64, dtype=torch.float16, device=DEV)
    with pytest.raises(VsError) as e:
        ops.spmm.wmmaSpmm(2, 1, 64, 16, ri, ro, ci, v, B, out)  # V = 1 on the tensor path
    assert e.value.code == -1
    with pytest.raises(VsError) as e:
        ops.spmm.wmmaSpmm(2, 8, 32, 16, ri, ro, ci, v, B, out)  # width not a multiple of 64
    assert e.value.code == -3
    with pytest.raises(VsError) as e:
        ops.spmm.wmmaSpmm(2, 8, 64, 16, ri, ro, ci, v.float(), B.float(), out.float())  # float tensor path
    assert e.value.code == -2


@pytest.mark.parametrize("V", [2, 8])
def test_software_gather_kernel_for_strides_tma_cannot_address(V, monkeypatch):
    """A batch stride of B that is not a multiple of the dense width cannot be described by the row-gather tensor
    map: among the gather kernels the cp.async one takes over.  Same tolerance; the padding between entries must
    stay untouched.  (The densifying kernel, which would otherwise take this density, is switched off.)"""
    monkeypatch.setenv("VSPARSE_B200_SPMM", "gather")
    N, K, batch = 128, 160, 3
    a = problem(cvse.GEN_BETA, 91 + V, 48, K, V, 0.6)
    vals = cvse.fill_random((a.nnz_vec * V,), np.float16, cvse.DIST_NORMAL, 1, 0.5)
    B = cvse.fill_random((batch, K, N), np.float16, cvse.DIST_NORMAL, 2, 1.0)
    pad = 8   # 16 bytes: keeps alignment, breaks divisibility by N
    flat = torch.zeros((batch, K * N + pad), dtype=torch.float16, device=DEV)
    flat[:, :K * N] = dev(B).reshape(batch, K * N)
    ri, ro, ci = structure(a)
    out = torch.empty((batch, a.m, N), dtype=torch.float32, device=DEV)
    from vectorsparse_b200 import _lib
    rc = _lib.lib().vs_spmm_batched(VS_PATH_TENSOR, 0, 1, a.m_vec, V, N, K, ri.data_ptr(), ro.data_ptr(), ci.data_ptr(),
                                    dev(vals).data_ptr(), flat.data_ptr(), out.data_ptr(), batch, 0, K * N + pad,
                                    a.m * N, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    for b in range(batch):
        assert_close(out[b].cpu().numpy(), spmm_oracle(a, N, vals, B[b]), f"software gather, entry {b}")
