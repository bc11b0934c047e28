"""Helpers shared by the GPU parity tests: seeded problems on the host, their copies on the device, and the
oracle results they are compared with."""
import numpy as np
import torch

import oracle
from vectorsparse_b200 import cvse

DEV = "cuda:0"


def problem(kind, seed, m_vec, n, V, sparsity, band=0, sort=True):
    return cvse.generate(kind, seed, m_vec, n, V, sparsity, band, sort)


def custom(lens, n, V, seed=0, sort=True):
    """CVSE with the given per-row vector counts (for edge cases)."""
    rng = np.random.default_rng(seed)
    ro = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    cols = [np.sort(rng.choice(n, int(l), replace=False)) for l in lens]
    ci = (np.concatenate(cols) if cols else np.zeros(0)).astype(np.int32)
    return cvse.CVSE(len(lens), n, V, ro, ci, cvse.row_swizzle(ro, sort))


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def structure(a):
    ri, ro, ci = a.to_device(DEV)
    if ci.numel() == 0:  # keep a valid pointer for empty matrices
        ci = torch.zeros(4, dtype=torch.int32, device=DEV)
    return ri, ro, ci


def spmm_inputs(a, N, dtype, seed, sigma=None):
    """values and B as numpy arrays of `dtype` (fp16 values are the rounded fp32 draws)."""
    if sigma is None:
        vals = cvse.fill_random((a.nnz_vec * a.V,), dtype, cvse.DIST_UNIFORM, seed)
    else:
        vals = cvse.fill_random((a.nnz_vec * a.V,), dtype, cvse.DIST_NORMAL, seed, sigma)
    B = cvse.fill_random((a.n, N), dtype, cvse.DIST_NORMAL if sigma is not None else cvse.DIST_UNIFORM, seed + 1, 1.0)
    return vals, B


def spmm_oracle(a, N, vals, B, threads=8):
    return oracle.spmm(a.m_vec, a.V, N, a.row_offsets, a.col_indices, vals.astype(np.float32),
                       B.astype(np.float32), acc="f64", threads=threads)


def sddmm_oracle(a, k, lhs, rhs, threads=8):
    return oracle.sddmm(a.m_vec, k, a.V, a.row_offsets, a.col_indices, lhs.astype(np.float32),
                        rhs.astype(np.float32), acc="f64", threads=threads)


def padded(t, extra=64, fill=float("nan")):
    """A buffer `extra` elements longer than needed, poison-filled, and the view the kernel writes: lets a test
    check that every output was written and nothing beyond it."""
    buf = torch.full((t + extra,), fill, dtype=torch.float32, device=DEV)
    return buf


def np_dtype(t):
    return np.float16 if t == torch.float16 else np.float32
