"""The reference's own CUDA kernels, compiled unmodified for sm_100a (baseline/Makefile), as a CONTEXT measurement.

Benchmark infrastructure only: bench.py and one GPU test load this module; the library never does.  The reference's
kernels are Volta-era code (mma.sync.m8n8k4 / WMMA, one warp per CTA, src/wmma_spmm.cu:13-116,
src/wmma_sddmm.cu:250-504); their residue path multiplies whatever the last register fragment holds
(src/spmm_utils/dense_tile.h:262-266, src/wmma_spmm.cu:93-110), which is only defined when every vector-row holds a
positive multiple of 32 vectors.  `pad_rows` therefore extends every row to such a length with columns the row does not
use and ZERO values, so that the padded product equals the original one and can be checked against it.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_ref", "libvsref_kernels.so")
_LIB = None


def lib():
    """The compiled reference kernels, or None where baseline/_ref/libvsref_kernels.so has not been built."""
    global _LIB
    if _LIB is None and os.path.exists(LIB_PATH):
        h = C.CDLL(LIB_PATH)
        vp, i = C.c_void_p, C.c_int
        h.refk_wmma_spmm.argtypes = [i, i, i, i, vp, vp, vp, vp, vp, vp, i]
        h.refk_cuda_spmm.argtypes = [i, i, i, i, vp, vp, vp, vp, vp, vp, i]
        h.refk_wmma_sddmm.argtypes = [i, i, i, i, vp, vp, vp, vp, vp, vp, i, i, i]
        h.refk_cuda_sddmm.argtypes = [i, i, i, i, vp, vp, vp, vp, vp, vp, i, i]
        for f in (h.refk_wmma_spmm, h.refk_cuda_spmm, h.refk_wmma_sddmm, h.refk_cuda_sddmm):
            f.restype = i
        _LIB = h
    return _LIB


def pad_rows(row_offsets: np.ndarray, col_indices: np.ndarray, n_cols: int, multiple: int = 32):
    """(row_offsets', col_indices', src): every row extended to a positive multiple of `multiple` entries with the
    lowest columns it does not hold yet; src[j'] is the index of entry j' in the original arrays, or -1 for padding."""
    m = len(row_offsets) - 1
    new_off = np.zeros(m + 1, np.int32)
    cols, src = [], []
    for i in range(m):
        lo, hi = int(row_offsets[i]), int(row_offsets[i + 1])
        have = col_indices[lo:hi]
        want = max(multiple, -(-(hi - lo) // multiple) * multiple)
        if want > n_cols:
            raise ValueError("a row cannot be padded beyond the number of columns")
        free = np.setdiff1d(np.arange(n_cols, dtype=np.int32), have, assume_unique=False)[:want - (hi - lo)]
        cols.append(np.concatenate([have, free]).astype(np.int32))
        src.append(np.concatenate([np.arange(lo, hi), -np.ones(len(free), np.int64)]))
        new_off[i + 1] = new_off[i] + want
    return new_off, np.concatenate(cols).astype(np.int32), np.concatenate(src).astype(np.int64)


def pad_values(values: np.ndarray, src: np.ndarray, V: int) -> np.ndarray:
    """Values of the padded structure: the original vectors where src >= 0, zeros for the padding."""
    v = values.reshape(-1, V)
    out = np.zeros((len(src), V), dtype=values.dtype)
    keep = src >= 0
    out[keep] = v[src[keep]]
    return out.reshape(-1)
