"""The reference's own CUDA kernels, compiled unmodified for sm_100a into baseline/_ref/ (baseline/Makefile), on
small problems whose rows are padded to multiples of 32 vectors with zero values (see baseline/refk.py for why):
checked with the reference's own criterion, abs(device - host) <= 0.5 (spmm_benchmark.cpp:214,
sddmm_benchmark.cpp:288), against the oracle of the ORIGINAL matrix, and against this library's kernels on the same
inputs.  Context only: bench.py times these kernels next to the library's; nothing ships them.  Skipped where the
reference was not available to build from."""
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from baseline import refk  # noqa: E402
from gpu_util import DEV, dev, problem, sddmm_oracle, spmm_oracle  # noqa: E402
from vectorsparse_b200 import cvse, ops  # noqa: E402

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(refk.lib() is None, reason="baseline/_ref/libvsref_kernels.so not built")]


def padded(a):
    ro, ci, src = refk.pad_rows(a.row_offsets, a.col_indices, a.n)
    return cvse.CVSE(a.m_vec, a.n, a.V, ro, ci, cvse.row_swizzle(ro)), src


@pytest.mark.parametrize("V", [2, 4, 8])
def test_reference_wmma_spmm_agrees_with_its_host_criterion(V):
    N, K = 128, 256
    a = problem(cvse.GEN_BETA, 3 + V, 64 // V * 2, K, V, 0.8)
    vals = cvse.fill_random((a.nnz_vec * V,), np.float16, cvse.DIST_NORMAL, 1, 0.5)
    B = cvse.fill_random((K, N), np.float16, cvse.DIST_NORMAL, 2, 1.0)
    want = spmm_oracle(a, N, vals, B)
    p, src = padded(a)
    ri, ro, ci = p.to_device(DEV)
    d_vals, d_B = dev(refk.pad_values(vals, src, V)), dev(B)
    out = torch.zeros((a.m, N), dtype=torch.float32, device=DEV)
    rc = refk.lib().refk_wmma_spmm(p.m_vec, V, N, K, ri.data_ptr(), ro.data_ptr(), ci.data_ptr(), d_vals.data_ptr(), d_B.data_ptr(),
                                   out.data_ptr(), 1)
    assert rc == 0
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    assert np.all(np.abs(got - want) <= 0.5), "the reference's own pass criterion"
    ours = torch.empty_like(out)
    ops.spmm.wmmaSpmm(p.m_vec, V, N, K, ri, ro, ci, d_vals, d_B, ours)
    torch.cuda.synchronize()
    assert np.max(np.abs(ours.cpu().numpy() - got)) <= 2e-2


def test_reference_wmma_sddmm_agrees_with_its_host_criterion():
    """V = 8, algorithm 1 (the reference harness's default, mmaSddmmKernel8reg, src/wmma_sddmm.cu:250-504), half output,
    contraction length 256: the call bench.py times for context (bench.py checks a small problem the same way before
    it times any of these kernels)."""
    V, k, K = 8, 256, 512
    a = problem(cvse.GEN_BETA, 3, 128 // V, K, V, 0.8)
    lhs = cvse.fill_random((a.m, k), np.float16, cvse.DIST_NORMAL, 1, 0.25)
    rhs = cvse.fill_random((K, k), np.float16, cvse.DIST_NORMAL, 2, 0.25)
    want = sddmm_oracle(a, k, lhs, rhs)
    ri, ro, ci = a.to_device(DEV)
    out = torch.zeros(a.nnz_vec * V, dtype=torch.float16, device=DEV)
    d_lhs, d_rhs = dev(lhs), dev(rhs)
    rc = refk.lib().refk_wmma_sddmm(a.m_vec, k, K, a.nnz_vec, ri.data_ptr(), ro.data_ptr(), ci.data_ptr(), d_lhs.data_ptr(),
                                    d_rhs.data_ptr(), out.data_ptr(), V, 1, 0)
    assert rc == 0
    torch.cuda.synchronize()
    assert np.all(np.abs(out.float().cpu().numpy() - want) <= 0.5), "the reference's own pass criterion"
