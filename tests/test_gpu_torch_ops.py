"""The optional PyTorch registration: torch.ops.vsparse.* give what the ops-module calls give, and FixedMaskAttention
back-propagates through the library's backward operators (gradients against the fp64 oracle, conftest tolerance)."""
import numpy as np
import pytest
import torch

import oracle
from conftest import assert_close
from gpu_util import DEV, dev, problem, spmm_oracle, structure
from vectorsparse_b200 import VS_PATH_CUDA_CORE, VS_PATH_TENSOR, cvse, torch_ops

pytestmark = pytest.mark.gpu


def test_registered_spmm_and_sddmm():
    V, N = 8, 128
    a = problem(cvse.GEN_BETA, 4, 32, 192, V, 0.8)
    ri, ro, ci = structure(a)
    vals = cvse.fill_random((a.nnz_vec * V,), np.float16, cvse.DIST_NORMAL, 1, 0.5)
    B = cvse.fill_random((a.n, N), np.float16, cvse.DIST_NORMAL, 2, 1.0)
    for path in (VS_PATH_TENSOR, VS_PATH_CUDA_CORE):
        C = torch.ops.vsparse.spmm(path, a.m_vec, V, ri, ro, ci, dev(vals), dev(B))
        assert C.shape == (a.m, N) and C.dtype == torch.float16
        assert_close(C.float().cpu().numpy(), spmm_oracle(a, N, vals, B), f"registered spmm, path {path}")
    lhs = cvse.fill_random((a.m, 64), np.float16, cvse.DIST_NORMAL, 3, 0.25)
    rhs = cvse.fill_random((a.n, 64), np.float16, cvse.DIST_NORMAL, 4, 0.25)
    S = torch.ops.vsparse.sddmm(VS_PATH_TENSOR, a.m_vec, V, a.nnz_vec, ri, ro, ci, dev(lhs), dev(rhs))
    want = oracle.sddmm(a.m_vec, 64, V, a.row_offsets, a.col_indices, lhs.astype(np.float32), rhs.astype(np.float32), acc="f64")
    assert_close(S.float().cpu().numpy(), want, "registered sddmm")
    P = torch.ops.vsparse.softmax(a.m_vec, V, ri, ro, S, 0.5)
    assert_close(P.float().cpu().numpy(), oracle.softmax(a.m_vec, V, a.row_offsets, S.float().cpu().numpy(), 0.5), "registered softmax")


def test_cpu_tensors_have_no_kernel():
    with pytest.raises((NotImplementedError, RuntimeError)):
        z = torch.zeros(8, dtype=torch.int32)
        torch.ops.vsparse.softmax(1, 8, z, z, torch.zeros(8, dtype=torch.float16), 1.0)


def test_autograd_through_fixed_mask_attention():
    V, d, n, heads = 8, 64, 512, 2
    a = problem(cvse.GEN_BAND, 6, n // V, n, V, 0.8, band=64)
    mask = torch_ops.AttentionMask(a, DEV)
    q, k, v, go = (cvse.fill_random((heads, n, d), np.float16, cvse.DIST_NORMAL, 10 + i, 1.0) for i in range(4))
    tq, tk, tv = (dev(x).requires_grad_(True) for x in (q, k, v))
    out = torch_ops.fixed_mask_attention(tq, tk, tv, mask, 0.125)
    out.backward(dev(go))
    torch.cuda.synchronize()
    for h in range(heads):
        want = oracle.attention(a.m_vec, V, d, d, a.row_offsets, a.col_indices, q[h].astype(np.float32), k[h].astype(np.float32),
                                v[h].astype(np.float32), 0.125)
        assert_close(out[h].detach().float().cpu().numpy(), want, f"forward, head {h}")
        wq, wk, wv = oracle.attention_backward(a.m_vec, V, d, a.row_offsets, a.col_indices, q[h].astype(np.float32),
                                               k[h].astype(np.float32), v[h].astype(np.float32), go[h].astype(np.float32), 0.125)
        assert_close(tq.grad[h].float().cpu().numpy(), wq, f"dQ, head {h}")
        assert_close(tk.grad[h].float().cpu().numpy(), wk, f"dK, head {h}")
        assert_close(tv.grad[h].float().cpu().numpy(), wv, f"dV, head {h}")


@pytest.mark.parametrize("batched", [False, True])
def test_autograd_through_the_sparse_dense_product(batched):
    """C = A @ B: the gradient of B is the product with the transposed matrix, the gradient of the values the sampled
    dense-dense product; both against the fp64 oracle (shared values with a batched B: summed over the batch)."""
    V, N, K = 8, 128, 192
    a = problem(cvse.GEN_BETA, 14, 256 // V, K, V, 0.8)
    mask = torch_ops.AttentionMask(a, DEV)
    vals = cvse.fill_random((a.nnz_vec * V,), np.float16, cvse.DIST_NORMAL, 1, 0.25)
    shape = (3, K, N) if batched else (K, N)
    B = cvse.fill_random(shape, np.float16, cvse.DIST_NORMAL, 2, 0.5)
    G = cvse.fill_random(shape[:-2] + (a.m, N), np.float16, cvse.DIST_NORMAL, 3, 0.25)
    tv, tb = dev(vals).requires_grad_(True), dev(B).requires_grad_(True)
    C = torch_ops.sparse_dense_product(tv, tb, mask)
    C.backward(dev(G))
    torch.cuda.synchronize()
    Bs, Gs = (B, G) if batched else (B[None], G[None])
    want_gv = np.zeros(a.nnz_vec * V, np.float64)
    for i in range(Bs.shape[0]):
        assert_close((C[i] if batched else C).detach().float().cpu().numpy(), spmm_oracle(a, N, vals, Bs[i]), f"forward {i}")
        want_gb = oracle.spmm_t(a.m_vec, V, N, K, a.row_offsets, a.col_indices, vals.astype(np.float32), Gs[i].astype(np.float32))
        assert_close((tb.grad[i] if batched else tb.grad).float().cpu().numpy(), want_gb, f"dB {i}")
        want_gv += oracle.sddmm(a.m_vec, N, V, a.row_offsets, a.col_indices, Gs[i].astype(np.float32), Bs[i].astype(np.float32), acc="f64")
    assert_close(tv.grad.float().cpu().numpy(), want_gv, "dvalues")
