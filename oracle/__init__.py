"""ctypes front end of the CPU oracle (TEST INFRASTRUCTURE ONLY).

Only the tests, the smoke entry and the benchmark's CPU-baseline legs import this module; the shipped
package never does.  `lib()` is the plain-C restatement (oracle/vs_oracle.c); `ref()` is the reference's
own host verification code compiled by `make -C oracle ref`, or None where that library is not present.

All arrays are numpy; fp16 data travel as float16 arrays (their 16-bit patterns are passed through).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None
_REF = None
_REF_TRIED = False

_I32P = C.POINTER(C.c_int)
_F32P = C.POINTER(C.c_float)
_F64P = C.POINTER(C.c_double)
_U16P = C.POINTER(C.c_uint16)


def build(ref: bool = False, reference: str | None = None) -> None:
    """Compile the oracle (and, with ref=True and a reference checkout present, the reference shim).  `reference`:
    where that checkout lies (default: the Makefile's, a directory named `reference` next to this repository)."""
    subprocess.run(["make", "-C", _HERE, "all"], check=True, capture_output=True)
    if ref:
        cmd = ["make", "-C", _HERE, "ref"] + ([f"REFERENCE={reference}"] if reference else [])
        subprocess.run(cmd, check=True, capture_output=True)


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "libvs_oracle.so")
        src = os.path.join(_HERE, "vs_oracle.c")
        if not os.path.exists(path) or os.path.getmtime(path) < os.path.getmtime(src):
            build()
        _LIB = C.CDLL(path)
    return _LIB


def ref():
    """The compiled reference host code, or None if oracle/_ref/libvsref.so has not been built."""
    global _REF, _REF_TRIED
    if not _REF_TRIED:
        _REF_TRIED = True
        path = os.path.join(_HERE, "_ref", "libvsref.so")
        if os.path.exists(path):
            _REF = C.CDLL(path)
    return _REF


def num_threads() -> int:
    return int(lib().vso_num_threads())


def _i32(a):
    a = np.ascontiguousarray(a, dtype=np.int32)
    return a, a.ctypes.data_as(_I32P)


def _f32(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(_F32P)


def _h16(a):
    a = np.ascontiguousarray(a, dtype=np.float16)
    return a, a.ctypes.data_as(_U16P)


def spmm(m_vec, V, N, row_offsets, col_indices, values, B, acc="f64", threads=1):
    """C = A(CVSE) @ B.  acc='f32' is the reference loop (spmm_benchmark.cpp:66-86); 'f64' the parity reference.

    float16 inputs with acc='f32' run the half-precision driver's loop (promotion per use)."""
    ro, rop = _i32(row_offsets)
    ci, cip = _i32(col_indices)
    M = m_vec * V
    if acc == "f64":
        v, vp = _f32(np.asarray(values, dtype=np.float32))
        b, bp = _f32(np.asarray(B, dtype=np.float32))
        out = np.empty((M, N), dtype=np.float64)
        lib().vso_spmm_f64(m_vec, V, N, rop, cip, vp, bp, out.ctypes.data_as(_F64P), threads)
        return out
    out = np.empty((M, N), dtype=np.float32)
    if np.asarray(values).dtype == np.float16:
        v, vp = _h16(values)
        b, bp = _h16(B)
        lib().vso_spmm_h16(m_vec, V, N, rop, cip, vp, bp, out.ctypes.data_as(_F32P), threads)
    else:
        v, vp = _f32(values)
        b, bp = _f32(B)
        lib().vso_spmm_f32(m_vec, V, N, rop, cip, vp, bp, out.ctypes.data_as(_F32P), threads)
    return out


def spmm_t(m_vec, V, N, K, row_offsets, col_indices, values, B):
    """C[K, N] = A(CVSE)^T @ B, B [m_vec * V, N]; fp64 accumulation.  No reference counterpart (see vs_oracle.c)."""
    ro, rop = _i32(row_offsets)
    ci, cip = _i32(col_indices)
    v, vp = _f32(np.asarray(values, dtype=np.float32))
    b, bp = _f32(np.asarray(B, dtype=np.float32))
    out = np.empty((K, N), dtype=np.float64)
    lib().vso_spmm_t_f64(m_vec, V, N, K, rop, cip, vp, bp, out.ctypes.data_as(_F64P))
    return out


def sddmm(m_vec, k, V, row_offsets, col_indices, lhs, rhs, acc="f64", threads=1):
    """out[j*V+v] = <lhs[i*V+v], rhs[col[j]]>.  acc='f32' is Host_sddmm (bm_test_utils.h:171-193)."""
    ro, rop = _i32(row_offsets)
    ci, cip = _i32(col_indices)
    nnz = int(ro[m_vec]) * V
    if acc == "f64":
        a, ap = _f32(np.asarray(lhs, dtype=np.float32))
        b, bp = _f32(np.asarray(rhs, dtype=np.float32))
        out = np.empty(nnz, dtype=np.float64)
        lib().vso_sddmm_f64(m_vec, k, V, rop, cip, ap, bp, out.ctypes.data_as(_F64P), threads)
        return out
    out = np.empty(nnz, dtype=np.float32)
    if np.asarray(lhs).dtype == np.float16:
        a, ap = _h16(lhs)
        b, bp = _h16(rhs)
        lib().vso_sddmm_h16(m_vec, k, V, rop, cip, ap, bp, out.ctypes.data_as(_F32P), threads)
    else:
        a, ap = _f32(lhs)
        b, bp = _f32(rhs)
        lib().vso_sddmm_f32(m_vec, k, V, rop, cip, ap, bp, out.ctypes.data_as(_F32P), threads)
    return out


def row_swizzle(mode, m_vec, row_offsets):
    """mode 0 identity, 1 sorted by row length descending (ties by index) — bm_test_utils.h:196-215."""
    ro, rop = _i32(row_offsets)
    out = np.empty(m_vec, dtype=np.int32)
    rc = lib().vso_row_swizzle(int(mode), m_vec, rop, out.ctypes.data_as(_I32P))
    if rc != 0:
        raise ValueError(f"vso_row_swizzle failed: {rc}")
    return out


def softmax(m_vec, V, row_offsets, scores, scale):
    ro, rop = _i32(row_offsets)
    s, sp = _f32(np.asarray(scores, dtype=np.float32))
    out = np.empty(s.shape, dtype=np.float64)
    lib().vso_softmax_f64(m_vec, V, rop, sp, C.c_double(scale), out.ctypes.data_as(_F64P))
    return out


def attention(m_vec, V, d, dv, row_offsets, col_indices, Q, K, Vm, scale):
    ro, rop = _i32(row_offsets)
    ci, cip = _i32(col_indices)
    q, qp = _f32(np.asarray(Q, dtype=np.float32))
    k, kp = _f32(np.asarray(K, dtype=np.float32))
    v, vp = _f32(np.asarray(Vm, dtype=np.float32))
    out = np.empty((m_vec * V, dv), dtype=np.float64)
    scratch = np.empty(2 * int(ro[m_vec]) * V, dtype=np.float64)
    lib().vso_attention_f64(m_vec, V, d, dv, rop, cip, qp, kp, vp, C.c_double(scale),
                            out.ctypes.data_as(_F64P), scratch.ctypes.data_as(_F64P))
    return out


def softmax_backward(m_vec, V, row_offsets, probs, grad_probs, scale):
    """Gradient of `softmax` with respect to its scores, fp64: scale * p * (g - sum_row(p * g)) per real row.  Numpy,
    one vector-row at a time.  No reference counterpart (the reference has no softmax): parity unpinned."""
    ro = np.asarray(row_offsets, dtype=np.int64)
    p = np.asarray(probs, dtype=np.float64).reshape(-1, V)
    g = np.asarray(grad_probs, dtype=np.float64).reshape(-1, V)
    out = np.zeros_like(p)
    for i in range(m_vec):
        b, e = ro[i], ro[i + 1]
        if e > b:
            dot = (p[b:e] * g[b:e]).sum(axis=0, keepdims=True)
            out[b:e] = scale * p[b:e] * (g[b:e] - dot)
    return out.reshape(-1)


def attention_backward(m_vec, V, d, row_offsets, col_indices, Q, K, Vm, dO, scale):
    """(dQ, dK, dV) of `attention` for one head, fp64 throughout (intermediates are not rounded): the composition
    P = softmax(scale * sddmm(Q, K)); dV = P^T dO; dP = sddmm(dO, Vm); dS = softmax_backward(P, dP); dQ = dS K;
    dK = dS^T Q over the oracle's own loops, each with a double accumulator.  Parity unpinned by the reference."""
    n = np.asarray(K).shape[0]
    lib_ = lib()
    ro, rop = _i32(row_offsets)
    ci, cip = _i32(col_indices)

    def sddmm64(lhs, rhs):
        l, lp = _f32(np.asarray(lhs, dtype=np.float32))
        r, rp = _f32(np.asarray(rhs, dtype=np.float32))
        out = np.empty(int(ro[m_vec]) * V, dtype=np.float64)
        lib_.vso_sddmm_f64(m_vec, d, V, rop, cip, lp, rp, out.ctypes.data_as(_F64P), 1)
        return out

    row_of = np.repeat(np.arange(m_vec, dtype=np.int64), np.diff(ro.astype(np.int64)))
    rows = (row_of[:, None] * V + np.arange(V, dtype=np.int64)[None, :]).reshape(-1)
    cols = np.repeat(ci[:int(ro[m_vec])].astype(np.int64), V)

    def matrix_of(vals):   # A [M, n] in double from CVSE values in double (repeated columns add up), kept sparse
        from scipy.sparse import coo_matrix
        return coo_matrix((vals, (rows, cols)), shape=(m_vec * V, n)).tocsr()

    s = sddmm64(Q, K)
    sv = s.reshape(-1, V) * scale   # softmax in double from the double scores, so nothing is rounded on the way
    Pm = np.zeros_like(sv)
    for i in range(m_vec):
        b, e = ro[i], ro[i + 1]
        if e > b:
            ex = np.exp(sv[b:e] - sv[b:e].max(axis=0, keepdims=True))
            Pm[b:e] = ex / ex.sum(axis=0, keepdims=True)
    P = Pm.reshape(-1)
    dO64 = np.asarray(dO, dtype=np.float64)
    dP = sddmm64(dO, Vm)
    dS = softmax_backward(m_vec, V, ro, P, dP, scale)
    Pd, dSd = matrix_of(P), matrix_of(dS)
    dV = np.asarray(Pd.T @ dO64)
    dQ = np.asarray(dSd @ np.asarray(K, dtype=np.float64))
    dK = np.asarray(dSd.T @ np.asarray(Q, dtype=np.float64))
    return dQ, dK, dV


def f32_to_h16(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    out = np.empty(a.shape, dtype=np.float16)
    lib().vso_f32_to_h16(a.ctypes.data_as(_F32P), out.ctypes.data_as(_U16P), C.c_int64(a.size))
    return out


def h16_to_f32(a):
    a = np.ascontiguousarray(a, dtype=np.float16)
    out = np.empty(a.shape, dtype=np.float32)
    lib().vso_h16_to_f32(a.ctypes.data_as(_U16P), out.ctypes.data_as(_F32P), C.c_int64(a.size))
    return out


# ---- the reference's own host code (present only where `make -C oracle ref` ran) ---------------------

def ref_spmm(m_vec, V, N, row_offsets, col_indices, values, B):
    r = ref()
    ro, rop = _i32(row_offsets)
    ci, cip = _i32(col_indices)
    out = np.empty((m_vec * V, N), dtype=np.float32)
    if np.asarray(values).dtype == np.float16:
        v, vp = _h16(values)
        b, bp = _h16(B)
        r.ref_spmm_host_h16(m_vec, V, N, rop, cip, vp, bp, out.ctypes.data_as(_F32P))
    else:
        v, vp = _f32(values)
        b, bp = _f32(B)
        r.ref_spmm_host_f32(m_vec, V, N, rop, cip, vp, bp, out.ctypes.data_as(_F32P))
    return out


def ref_sddmm(m_vec, k, V, row_offsets, col_indices, lhs, rhs, out16=False):
    r = ref()
    ro, rop = _i32(row_offsets)
    ci, cip = _i32(col_indices)
    nnz = int(ro[m_vec]) * V
    if np.asarray(lhs).dtype == np.float16:
        a, ap = _h16(lhs)
        b, bp = _h16(rhs)
        if out16:
            out = np.empty(nnz, dtype=np.float16)
            r.ref_sddmm_host_h16_out16(m_vec, k, V, rop, cip, ap, bp, out.ctypes.data_as(_U16P))
            return out
        out = np.empty(nnz, dtype=np.float32)
        r.ref_sddmm_host_h16(m_vec, k, V, rop, cip, ap, bp, out.ctypes.data_as(_F32P))
        return out
    a, ap = _f32(lhs)
    b, bp = _f32(rhs)
    out = np.empty(nnz, dtype=np.float32)
    r.ref_sddmm_host_f32(m_vec, k, V, rop, cip, ap, bp, out.ctypes.data_as(_F32P))
    return out


def ref_row_swizzle(sorted_, m_vec, row_offsets):
    ro, rop = _i32(row_offsets)
    out = np.empty(m_vec, dtype=np.int32)
    ref().ref_row_swizzle(int(bool(sorted_)), m_vec, rop, out.ctypes.data_as(_I32P))
    return out


def ref_make_dense(rows, cols, dtype=np.float32):
    out = np.empty((rows, cols), dtype=dtype)
    if dtype == np.float16:
        ref().ref_make_dense_h16(rows, cols, out.ctypes.data_as(_U16P))
    else:
        ref().ref_make_dense_f32(rows, cols, out.ctypes.data_as(_F32P))
    return out
