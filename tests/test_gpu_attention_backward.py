"""Backward of the masked softmax and of fixed-mask attention on the GPU, through the C ABI, against the fp64
oracle (conftest.assert_close).  Neither has a counterpart in the reference."""
import numpy as np
import pytest
import torch

import oracle
from conftest import assert_close
from gpu_util import DEV, custom, dev, problem, structure
from vectorsparse_b200 import VS_PATH_CUDA_CORE, VS_PATH_TENSOR, cvse, ops

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("V", [1, 2, 4, 8])
@pytest.mark.parametrize("dtype", [np.float16, np.float32])
def test_softmax_backward(V, dtype):
    a = custom([0, 70, 3, 33, 0, 1, 200, 450], 512, V, seed=V)   # 450: longer than any register cache (two-pass path)
    ro = dev(a.row_offsets)
    s = cvse.fill_random((a.nnz_vec * V,), np.float32, cvse.DIST_NORMAL, 1, 2.0)
    p = oracle.softmax(a.m_vec, V, a.row_offsets, s, 0.5).astype(dtype)
    g = cvse.fill_random((a.nnz_vec * V,), dtype, cvse.DIST_NORMAL, 2, 1.0)
    want = oracle.softmax_backward(a.m_vec, V, a.row_offsets, p.astype(np.float64), g.astype(np.float64), 0.5)
    d_p, d_g = dev(p), dev(g)
    out = torch.full((a.nnz_vec * V + 16,), float("nan"), dtype=d_p.dtype, device=DEV)
    ops.softmax_cvse_backward(a.m_vec, V, ro, d_p, d_g, out, 0.5)
    torch.cuda.synchronize()
    host = out.float().cpu().numpy()
    assert np.all(np.isnan(host[a.nnz_vec * V:])), "wrote past the end"
    assert_close(host[:a.nnz_vec * V], want, f"softmax backward V={V}")
    # in place over the incoming gradient: same bits
    ops.softmax_cvse_backward(a.m_vec, V, ro, d_p, d_g, d_g, 0.5)
    torch.cuda.synchronize()
    assert torch.equal(d_g, out[:a.nnz_vec * V])


def test_softmax_backward_batched():
    V, batch = 8, 3
    a = problem(cvse.GEN_BETA, 2, 16, 128, V, 0.7)
    ro = dev(a.row_offsets)
    rng = np.random.default_rng(0)
    p = np.stack([oracle.softmax(a.m_vec, V, a.row_offsets, rng.standard_normal(a.nnz_vec * V).astype(np.float32), 1.0)
                  for _ in range(batch)]).astype(np.float16)
    g = cvse.fill_random((batch, a.nnz_vec * V), np.float16, cvse.DIST_NORMAL, 3, 1.0)
    out = torch.empty((batch, a.nnz_vec * V), dtype=torch.float16, device=DEV)
    ops.softmax_cvse_backward(a.m_vec, V, ro, dev(p), dev(g), out, 1.0)
    torch.cuda.synchronize()
    for b in range(batch):
        want = oracle.softmax_backward(a.m_vec, V, a.row_offsets, p[b].astype(np.float64), g[b].astype(np.float64), 1.0)
        assert_close(out[b].float().cpu().numpy(), want, f"batch entry {b}")


@pytest.mark.parametrize("path", [VS_PATH_TENSOR, VS_PATH_CUDA_CORE])
def test_attention_backward_small(path):
    """Seven operator calls (SDDMM, softmax, SpMM^T, SDDMM, softmax backward, SpMM, SpMM^T) on a band + strided mask,
    two heads sharing it; intermediates are fp16 on the GPU and double in the oracle."""
    V, d, n, heads = 8, 64, 512, 2
    a = problem(cvse.GEN_BAND, 6, n // V, n, V, 0.8, band=64)
    q, k, v, go = (cvse.fill_random((heads, n, d), np.float16, cvse.DIST_NORMAL, 10 + i, 1.0) for i in range(4))
    ri, ro, ci = structure(a)
    t_off, t_rows, t_src = (dev(x) for x in cvse.transpose(a))
    gq, gk, gv = (torch.empty((heads, n, d), dtype=torch.float16, device=DEV) for _ in range(3))
    ws_p, ws_g = (torch.empty((heads, a.nnz_vec * V), dtype=torch.float16, device=DEV) for _ in range(2))
    ops.attention_cvse_backward(path, a.m_vec, V, n, d, a.nnz_vec, ri, ro, ci, t_off, t_rows, t_src, dev(q), dev(k), dev(v),
                                dev(go), gq, gk, gv, ws_p, ws_g, 0.125)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    for h in range(heads):
        wq, wk, wv = oracle.attention_backward(a.m_vec, V, d, a.row_offsets, a.col_indices, q[h].astype(np.float32),
                                               k[h].astype(np.float32), v[h].astype(np.float32), go[h].astype(np.float32), 0.125)
        assert_close(gv[h].float().cpu().numpy(), wv, f"dV head {h}")
        assert_close(gq[h].float().cpu().numpy(), wq, f"dQ head {h}")
        assert_close(gk[h].float().cpu().numpy(), wk, f"dK head {h}")


def test_attention_backward_config5_full_size():
    """The configured size of the fixed-mask attention workload (sequence 4096, head dimension 64, V = 8, band 256 +
    strided vectors, 410 entries per row, scale 1/8), two heads: dQ, dK, dV against the fp64 oracle."""
    V, d, n, heads = 8, 64, 4096, 2
    a = problem(cvse.GEN_BAND, 2026, n // V, n, V, 0.9, band=256)
    q, k, v, go = (cvse.fill_random((heads, n, d), np.float16, cvse.DIST_NORMAL, 40 + i, 1.0) for i in range(4))
    ri, ro, ci = structure(a)
    t_off, t_rows, t_src = (dev(x) for x in cvse.transpose(a))
    gq, gk, gv = (torch.full((heads, n, d), float("nan"), dtype=torch.float16, device=DEV) for _ in range(3))
    ws_p, ws_g = (torch.empty((heads, a.nnz_vec * V), dtype=torch.float16, device=DEV) for _ in range(2))
    ops.attention_cvse_backward(VS_PATH_TENSOR, a.m_vec, V, n, d, a.nnz_vec, ri, ro, ci, t_off, t_rows, t_src, dev(q), dev(k),
                                dev(v), dev(go), gq, gk, gv, ws_p, ws_g, 0.125)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    for h in range(heads):
        wq, wk, wv = oracle.attention_backward(a.m_vec, V, d, a.row_offsets, a.col_indices, q[h].astype(np.float32),
                                               k[h].astype(np.float32), v[h].astype(np.float32), go[h].astype(np.float32), 0.125)
        assert_close(gv[h].float().cpu().numpy(), wv, f"config 5 dV head {h}")
        assert_close(gq[h].float().cpu().numpy(), wq, f"config 5 dQ head {h}")
        assert_close(gk[h].float().cpu().numpy(), wk, f"config 5 dK head {h}")
