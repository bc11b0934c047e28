"""CVSE (column-vector sparse encoding) on the host: container, validator, builders, row swizzle, generators.

All heavy lifting is done by the C++ builder behind the C ABI (csrc/host_build.cpp), so a seed means the same
matrix here, in the C++ drivers and in the tests.  The reference keeps this logic inline in its drivers
(spmm_benchmark.cpp:21-60,89-97) and in include/bm_test_utils.h:70-142,196-215.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import _lib

GEN_FIXED, GEN_BETA, GEN_UNIFORM, GEN_BAND = 0, 1, 2, 3
DIST_UNIFORM, DIST_NORMAL = 0, 1


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


@dataclass
class CVSE:
    """Structure of a column-vector sparse matrix with m_vec * V rows and n columns (host arrays, int32)."""
    m_vec: int
    n: int
    V: int
    row_offsets: np.ndarray
    col_indices: np.ndarray
    row_indices: np.ndarray

    @property
    def nnz_vec(self) -> int:
        return int(self.row_offsets[self.m_vec])

    @property
    def m(self) -> int:
        return self.m_vec * self.V

    def validate(self) -> None:
        validate(self.m_vec, self.n, self.nnz_vec, self.row_offsets, self.col_indices)

    def to_device(self, device):
        """(row_indices, row_offsets, col_indices) as int32 torch tensors on `device`."""
        import torch
        return tuple(torch.from_numpy(np.ascontiguousarray(a)).to(device)
                     for a in (self.row_indices, self.row_offsets, self.col_indices))

    def to_dense(self, values: np.ndarray) -> np.ndarray:
        """Dense m x n matrix from the values array (values[j*V+v] -> row i*V+v, column col_indices[j])."""
        out = np.zeros((self.m, self.n), dtype=values.dtype)
        vals = values.reshape(-1, self.V)
        for i in range(self.m_vec):
            b, e = int(self.row_offsets[i]), int(self.row_offsets[i + 1])
            out[i * self.V:(i + 1) * self.V, self.col_indices[b:e]] = vals[b:e].T
        return out


def validate(m_vec, n, nnz_vec, row_offsets, col_indices) -> None:
    ro = np.ascontiguousarray(row_offsets, dtype=np.int32)
    ci = np.ascontiguousarray(col_indices, dtype=np.int32)
    if ro.size != m_vec + 1:
        raise _lib.VsError(-6, "vs_cvse_validate")
    _lib.check(_lib.lib().vs_cvse_validate(m_vec, n, nnz_vec, _ptr(ro), _ptr(ci)), "vs_cvse_validate")


def row_swizzle(row_offsets, sort: bool = True) -> np.ndarray:
    """Processing order of the vector-rows: identity, or longest first (ties by index)."""
    ro = np.ascontiguousarray(row_offsets, dtype=np.int32)
    m_vec = ro.size - 1
    out = np.empty(m_vec, dtype=np.int32)
    _lib.check(_lib.lib().vs_row_swizzle(1 if sort else 0, m_vec, _ptr(ro), _ptr(out)), "vs_row_swizzle")
    return out


def generate(kind: int, seed: int, m_vec: int, n: int, V: int, sparsity: float, band: int = 0,
             sort: bool = True) -> CVSE:
    """Seeded synthetic pattern; see vs_cvse_generate in include/vsparse_b200.h for the four kinds."""
    L = _lib.lib()
    ro = np.empty(m_vec + 1, dtype=np.int32)
    nnz = L.vs_cvse_generate(kind, seed, m_vec, n, V, float(sparsity), band, _ptr(ro), None)
    if nnz < 0:
        raise _lib.VsError(nnz, "vs_cvse_generate")
    ci = np.empty(max(nnz, 1), dtype=np.int32)
    rc = L.vs_cvse_generate(kind, seed, m_vec, n, V, float(sparsity), band, _ptr(ro), _ptr(ci))
    if rc < 0:
        raise _lib.VsError(rc, "vs_cvse_generate")
    ci = ci[:nnz]
    return CVSE(m_vec, n, V, ro, ci, row_swizzle(ro, sort))


def from_dense_mask(mask: np.ndarray, V: int, sort: bool = True) -> CVSE:
    """mask: [m_vec, n] array, nonzero where a column vector is present."""
    mk = np.ascontiguousarray(mask != 0, dtype=np.uint8)
    m_vec, n = mk.shape
    L = _lib.lib()
    ro = np.empty(m_vec + 1, dtype=np.int32)
    nnz = L.vs_cvse_from_dense_mask(m_vec, n, _ptr(mk), _ptr(ro), None)
    if nnz < 0:
        raise _lib.VsError(nnz, "vs_cvse_from_dense_mask")
    ci = np.empty(max(nnz, 1), dtype=np.int32)
    L.vs_cvse_from_dense_mask(m_vec, n, _ptr(mk), _ptr(ro), _ptr(ci))
    return CVSE(m_vec, n, V, ro, ci[:nnz], row_swizzle(ro, sort))


def transpose(a: CVSE):
    """Structure of A^T for ops.spmm_t: (t_offsets [n + 1], t_rows [nnz_vec], t_src [nnz_vec]) as int32 arrays — for each
    column of A its nonzero vectors as (vector-row, index of the vector in the CVSE arrays), ascending in the row."""
    t_off = np.empty(a.n + 1, dtype=np.int32)
    t_rows = np.empty(max(a.nnz_vec, 1), dtype=np.int32)
    t_src = np.empty(max(a.nnz_vec, 1), dtype=np.int32)
    ci = np.ascontiguousarray(a.col_indices, dtype=np.int32)
    _lib.check(_lib.lib().vs_cvse_transpose(a.m_vec, a.n, a.nnz_vec, _ptr(a.row_offsets), _ptr(ci), _ptr(t_off),
                                            _ptr(t_rows), _ptr(t_src)), "vs_cvse_transpose")
    return t_off, t_rows[:a.nnz_vec], t_src[:a.nnz_vec]


def prune_dense(weight: np.ndarray, V: int, sparsity: float, per_row: bool = False, sort: bool = True):
    """Vector-wise magnitude pruning of a dense [M, n] weight (M a multiple of V): keeps the V x 1 column vectors with
    the largest sums of absolute values, over the whole matrix or (per_row) the same number in every vector-row.
    Returns (CVSE, values) with values float32 in the CVSE layout values[j * V + v]."""
    w = np.ascontiguousarray(weight, dtype=np.float32)
    if w.ndim != 2 or w.shape[0] % V:
        raise ValueError("weight must be [M, n] with M a multiple of V")
    m_vec, n = w.shape[0] // V, w.shape[1]
    L = _lib.lib()
    ro = np.empty(m_vec + 1, dtype=np.int32)
    nnz = L.vs_cvse_prune_dense(m_vec, n, V, _ptr(w), float(sparsity), int(per_row), _ptr(ro), None, None)
    if nnz < 0:
        raise _lib.VsError(nnz, "vs_cvse_prune_dense")
    ci = np.empty(max(nnz, 1), dtype=np.int32)
    vals = np.empty(max(nnz, 1) * V, dtype=np.float32)
    L.vs_cvse_prune_dense(m_vec, n, V, _ptr(w), float(sparsity), int(per_row), _ptr(ro), _ptr(ci), _ptr(vals))
    return CVSE(m_vec, n, V, ro, ci[:nnz], row_swizzle(ro, sort)), vals[:nnz * V]


def from_smtx(path: str, V: int, sort: bool = True) -> CVSE:
    """Reads a DLMC .smtx pattern; its row count is the number of VECTOR rows (spmm_benchmark.cpp:26-33)."""
    L = _lib.lib()
    rows, cols, nnz = C.c_int(), C.c_int(), C.c_int()
    _lib.check(L.vs_smtx_read_header(path.encode(), C.byref(rows), C.byref(cols), C.byref(nnz)), "vs_smtx_read_header")
    ro = np.empty(rows.value + 1, dtype=np.int32)
    ci = np.empty(max(nnz.value, 1), dtype=np.int32)
    _lib.check(L.vs_smtx_read(path.encode(), rows.value, nnz.value, _ptr(ro), _ptr(ci)), "vs_smtx_read")
    return CVSE(rows.value, cols.value, V, ro, ci[:nnz.value], row_swizzle(ro, sort))


def to_smtx(path: str, a: CVSE) -> None:
    _lib.check(_lib.lib().vs_smtx_write(path.encode(), a.m_vec, a.n, a.nnz_vec, _ptr(a.row_offsets),
                                        _ptr(np.ascontiguousarray(a.col_indices))), "vs_smtx_write")


def fill_random(shape, dtype, dist: int, seed: int, sigma: float = 1.0) -> np.ndarray:
    """Seeded values: dist 0 = uniform(-1,1), dist 1 = normal(0, sigma); dtype float32 or float16."""
    dt = np.dtype(dtype)
    out = np.empty(shape, dtype=dt)
    code = _lib.VS_F16 if dt == np.float16 else _lib.VS_F32
    if dt not in (np.dtype(np.float16), np.dtype(np.float32)):
        raise _lib.VsError(-2, "vs_fill_random")
    _lib.check(_lib.lib().vs_fill_random(code, dist, seed, float(sigma), out.size, _ptr(out)), "vs_fill_random")
    return out
