"""Operators on CUDA tensors, named and argued like the reference's C++ API.

    spmm.wmmaSpmm / spmm.cudaSpmm       include/wmma_spmm.cuh:7-29, include/cuda_spmm.cuh:7-29
    sddmm.wmmaSddmm / sddmm.cudaSddmm   include/wmma_sddmm.cuh:7-33, include/cuda_sddmm.cuh:7-32

Arguments keep the reference's order and meaning (m_vec, vec_length, k, n, row_indices, row_offsets,
column_indices, values, rhs_matrix, output_matrix); tensors replace raw device pointers and the element types
are taken from them, which is what overload resolution does in the reference.  Every call enqueues on the
current torch CUDA stream and returns 0; rejected arguments raise VsError (the reference prints and returns).
PyTorch is used for device memory and streams only: the arithmetic is in libvsparse_b200.so.
"""
from __future__ import annotations

import types

import torch

from . import _lib
from ._lib import VS_F16, VS_F32, VS_PATH_CUDA_CORE, VS_PATH_TENSOR

_DT = {torch.float16: VS_F16, torch.float32: VS_F32}


def _one_device(**tensors):
    """The CUDA device every given tensor lives on.  TypeError if one is not a CUDA tensor or if they are spread
    over several devices: the kernels, their tensor maps, the status word and the plan scratch all belong to ONE
    device, so pointers of another would be dereferenced on the wrong GPU.  None values (optional arguments) are
    skipped."""
    device = None
    for name, t in tensors.items():
        if t is None:
            continue
        if not getattr(t, "is_cuda", False):
            raise TypeError(f"{name} must be a CUDA tensor")
        if device is None:
            device, first = t.device, name
        elif t.device != device:
            raise TypeError(f"{name} is on {t.device} but {first} is on {device}: all operands must share one device")
    if device is None:
        raise TypeError("no CUDA tensor among the arguments")
    return device


def _dev(t: torch.Tensor, name: str, dtype=None):
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise TypeError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise TypeError(f"{name} must be {dtype}, got {t.dtype}")
    return t.data_ptr()


def _dtype_code(t: torch.Tensor, name: str) -> int:
    if t.dtype not in _DT:
        raise _lib.VsError(-2, name)
    return _DT[t.dtype]


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _need(t: torch.Tensor, numel: int, name: str):
    if t.numel() < numel:
        raise ValueError(f"{name} holds {t.numel()} elements, {numel} needed")


def _spmm(path, m_vec, vec_length, k, n, row_indices, row_offsets, column_indices, values, rhs_matrix,
          output_matrix, batch=1, nonzeros_vec=None):
    device = _one_device(row_indices=row_indices, row_offsets=row_offsets, column_indices=column_indices, values=values,
                         rhs_matrix=rhs_matrix, output_matrix=output_matrix)
    _need(row_indices, m_vec, "row_indices")
    _need(row_offsets, m_vec + 1, "row_offsets")
    _need(rhs_matrix, batch * n * k if rhs_matrix.dim() == 3 else n * k, "rhs_matrix")
    _need(output_matrix, batch * m_vec * vec_length * k, "output_matrix")
    if nonzeros_vec is not None:   # the reference signature carries no count: checked when the caller knows it
        _need(column_indices, nonzeros_vec, "column_indices")
        _need(values, (batch if values.dim() == 2 else 1) * nonzeros_vec * vec_length, "values")
    sv = values.stride(0) if values.dim() == 2 and batch > 1 else 0
    sr = rhs_matrix.stride(0) if rhs_matrix.dim() == 3 and batch > 1 else 0
    so = output_matrix.stride(0) if output_matrix.dim() == 3 and batch > 1 else 0
    with torch.cuda.device(device):
        rc = _lib.lib().vs_spmm_batched(
            path, _dtype_code(values, "values"), _dtype_code(output_matrix, "output_matrix"), m_vec, vec_length, k, n,
            _dev(row_indices, "row_indices", torch.int32), _dev(row_offsets, "row_offsets", torch.int32),
            _dev(column_indices, "column_indices", torch.int32), _dev(values, "values"),
            _dev(rhs_matrix, "rhs_matrix", values.dtype), _dev(output_matrix, "output_matrix"), batch, sv, sr, so,
            _stream())
    _lib.check(rc, "vs_spmm")
    return 0


def _sddmm(path, m_vec, k, n, nonzeros_vec, row_indices, row_offsets, col_indices, lhs_matrix, rhs_matrix,
           output_values, vec_length, algorithm, batch=1):
    _need(row_indices, m_vec, "row_indices")
    _need(row_offsets, m_vec + 1, "row_offsets")
    _need(col_indices, nonzeros_vec, "col_indices")
    _need(lhs_matrix, (batch if lhs_matrix.dim() == 3 else 1) * m_vec * vec_length * k, "lhs_matrix")
    _need(rhs_matrix, (batch if rhs_matrix.dim() == 3 else 1) * n * k, "rhs_matrix")
    _need(output_values, batch * nonzeros_vec * vec_length, "output_values")
    sl = lhs_matrix.stride(0) if lhs_matrix.dim() == 3 and batch > 1 else 0
    sr = rhs_matrix.stride(0) if rhs_matrix.dim() == 3 and batch > 1 else 0
    so = output_values.stride(0) if output_values.dim() == 2 and batch > 1 else 0
    device = _one_device(row_indices=row_indices, row_offsets=row_offsets, col_indices=col_indices, lhs_matrix=lhs_matrix,
                         rhs_matrix=rhs_matrix, output_values=output_values)
    with torch.cuda.device(device):
        rc = _lib.lib().vs_sddmm_batched(
            path, _dtype_code(lhs_matrix, "lhs_matrix"), _dtype_code(output_values, "output_values"), m_vec, k, n,
            nonzeros_vec, _dev(row_indices, "row_indices", torch.int32), _dev(row_offsets, "row_offsets", torch.int32),
            _dev(col_indices, "col_indices", torch.int32), _dev(lhs_matrix, "lhs_matrix"),
            _dev(rhs_matrix, "rhs_matrix", lhs_matrix.dtype), _dev(output_values, "output_values"), vec_length, batch,
            sl, sr, so, _stream(), algorithm)
    _lib.check(rc, "vs_sddmm")
    return 0


# ---- namespaces mirroring the reference -------------------------------------------------------------------

def _wmmaSpmm(m_vec, vec_length, k, n, row_indices, row_offsets, column_indices, values, rhs_matrix, output_matrix,
              nonzeros_vec=None):
    """Tensor-core SpMM, V in {2,4,8}; fp16 in, fp16 or fp32 out (src/wmma_spmm.cu:388-409).  nonzeros_vec (not in
    the reference signature, optional): row_offsets[m_vec] when the caller knows it, so that the sizes of
    column_indices and values can be checked on the host."""
    return _spmm(VS_PATH_TENSOR, m_vec, vec_length, k, n, row_indices, row_offsets, column_indices, values,
                 rhs_matrix, output_matrix, nonzeros_vec=nonzeros_vec)


def _cudaSpmm(m_vec, vec_length, k, n, row_indices, row_offsets, column_indices, values, rhs_matrix, output_matrix,
              nonzeros_vec=None):
    """CUDA-core SpMM, V in {1,2,4,8}; fp16 or fp32 (src/cuda_spmm.cu:304-338; fp32 is a stub there).  nonzeros_vec:
    as for wmmaSpmm."""
    return _spmm(VS_PATH_CUDA_CORE, m_vec, vec_length, k, n, row_indices, row_offsets, column_indices, values,
                 rhs_matrix, output_matrix, nonzeros_vec=nonzeros_vec)


def _wmmaSddmm(m_vec, k, n, nonzeros_vec, row_indices, row_offsets, col_indices, lhs_matrix, rhs_matrix,
               output_values, vec_length, stream=None, algorithm=1):
    """Tensor-core SDDMM (src/wmma_sddmm.cu:3175-3202).  `stream`: a torch.cuda.Stream or None (current)."""
    if stream is not None:
        with torch.cuda.stream(stream):
            return _sddmm(VS_PATH_TENSOR, m_vec, k, n, nonzeros_vec, row_indices, row_offsets, col_indices,
                          lhs_matrix, rhs_matrix, output_values, vec_length, algorithm)
    return _sddmm(VS_PATH_TENSOR, m_vec, k, n, nonzeros_vec, row_indices, row_offsets, col_indices, lhs_matrix,
                  rhs_matrix, output_values, vec_length, algorithm)


def _cudaSddmm(m_vec, k, n, nonzeros_vec, row_indices, row_offsets, col_indices, lhs_matrix, rhs_matrix,
               output_values, vec_length, stream=None):
    """CUDA-core SDDMM (src/cuda_sddmm.cu:1257-1331)."""
    if stream is not None:
        with torch.cuda.stream(stream):
            return _sddmm(VS_PATH_CUDA_CORE, m_vec, k, n, nonzeros_vec, row_indices, row_offsets, col_indices,
                          lhs_matrix, rhs_matrix, output_values, vec_length, 0)
    return _sddmm(VS_PATH_CUDA_CORE, m_vec, k, n, nonzeros_vec, row_indices, row_offsets, col_indices, lhs_matrix,
                  rhs_matrix, output_values, vec_length, 0)


spmm = types.SimpleNamespace(wmmaSpmm=_wmmaSpmm, cudaSpmm=_cudaSpmm)
sddmm = types.SimpleNamespace(wmmaSddmm=_wmmaSddmm, cudaSddmm=_cudaSddmm)


# ---- batched forms, softmax and attention (no counterpart in the reference) ---------------------------------

def spmm_batched(path, m_vec, vec_length, k, n, row_indices, row_offsets, column_indices, values, rhs_matrix,
                 output_matrix, nonzeros_vec=None):
    """values [B, nnz] (or [nnz], shared), rhs [B, n, k] (or [n, k]), out [B, m, k]: one launch for B products."""
    batch = output_matrix.shape[0]
    return _spmm(path, m_vec, vec_length, k, n, row_indices, row_offsets, column_indices, values, rhs_matrix,
                 output_matrix, batch, nonzeros_vec=nonzeros_vec)


def spmm_t(m_vec, vec_length, k, n, t_offsets, t_rows, t_src, values, rhs_matrix, output_matrix, nonzeros_vec=None):
    """output [n, k] (or [B, n, k]) = A^T @ rhs, rhs [m_vec * V, k] (or [B, ...]), values [nnz] (or [B, nnz]): the
    product with the transposed CVSE matrix; t_offsets / t_rows / t_src come from cvse.transpose (on the device)."""
    batch = output_matrix.shape[0] if output_matrix.dim() == 3 else 1
    _need(t_offsets, n + 1, "t_offsets")
    _need(rhs_matrix, (batch if rhs_matrix.dim() == 3 else 1) * m_vec * vec_length * k, "rhs_matrix")
    _need(output_matrix, batch * n * k, "output_matrix")
    sv = values.stride(0) if values.dim() == 2 and batch > 1 else 0
    sr = rhs_matrix.stride(0) if rhs_matrix.dim() == 3 and batch > 1 else 0
    so = output_matrix.stride(0) if output_matrix.dim() == 3 and batch > 1 else 0
    if t_rows.numel() != t_src.numel():
        raise ValueError(f"t_rows holds {t_rows.numel()} entries, t_src {t_src.numel()}: both list the nonzero vectors")
    if nonzeros_vec is not None:   # checked when the caller knows the count (t_offsets lives on the device)
        _need(t_rows, nonzeros_vec, "t_rows")
        _need(values, (batch if values.dim() == 2 else 1) * nonzeros_vec * vec_length, "values")
    device = _one_device(t_offsets=t_offsets, t_rows=t_rows, t_src=t_src, values=values, rhs_matrix=rhs_matrix,
                         output_matrix=output_matrix)
    with torch.cuda.device(device):
        rc = _lib.lib().vs_spmm_t_batched(
            _dtype_code(values, "values"), _dtype_code(output_matrix, "output_matrix"), m_vec, vec_length, k, n,
            _dev(t_offsets, "t_offsets", torch.int32), _dev(t_rows, "t_rows", torch.int32), _dev(t_src, "t_src", torch.int32),
            _dev(values, "values"), _dev(rhs_matrix, "rhs_matrix", values.dtype), _dev(output_matrix, "output_matrix"),
            batch, sv, sr, so, _stream())
    _lib.check(rc, "vs_spmm_t")
    return 0


def sddmm_batched(path, m_vec, k, n, nonzeros_vec, row_indices, row_offsets, col_indices, lhs_matrix, rhs_matrix,
                  output_values, vec_length, algorithm=1):
    """lhs [B, m, k], rhs [B, n, k], out [B, nnz]."""
    batch = output_values.shape[0]
    return _sddmm(path, m_vec, k, n, nonzeros_vec, row_indices, row_offsets, col_indices, lhs_matrix, rhs_matrix,
                  output_values, vec_length, algorithm, batch)


def softmax_cvse(m_vec, vec_length, row_indices, row_offsets, scores, probs, scale=1.0):
    """Row softmax over the CVSE values; scores/probs [nnz] or [B, nnz]; probs may be scores."""
    batch = scores.shape[0] if scores.dim() == 2 else 1
    stride = scores.stride(0) if scores.dim() == 2 and batch > 1 else 0
    device = _one_device(row_indices=row_indices, row_offsets=row_offsets, scores=scores, probs=probs)
    with torch.cuda.device(device):
        rc = _lib.lib().vs_softmax_cvse(_dtype_code(scores, "scores"), m_vec, vec_length,
                                        _dev(row_indices, "row_indices", torch.int32),
                                        _dev(row_offsets, "row_offsets", torch.int32), _dev(scores, "scores"),
                                        _dev(probs, "probs", scores.dtype), float(scale), batch, stride, _stream())
    _lib.check(rc, "vs_softmax_cvse")
    return 0


def attention_cvse(path, m_vec, vec_length, n, d, nonzeros_vec, row_indices, row_offsets, col_indices, q, kmat,
                   vmat, out, workspace, scale):
    """softmax(scale * SDDMM(q, k)) @ v for [B, ., d] fp16 tensors sharing one mask; workspace [B, nnz] fp16."""
    batch = q.shape[0] if q.dim() == 3 else 1
    _need(workspace, batch * nonzeros_vec * vec_length, "workspace")
    _need(col_indices, nonzeros_vec, "col_indices")
    device = _one_device(row_indices=row_indices, row_offsets=row_offsets, col_indices=col_indices, q=q, kmat=kmat, vmat=vmat,
                         out=out, workspace=workspace)
    with torch.cuda.device(device):
        rc = _lib.lib().vs_attention_cvse(path, m_vec, vec_length, n, d, nonzeros_vec,
                                          _dev(row_indices, "row_indices", torch.int32),
                                          _dev(row_offsets, "row_offsets", torch.int32),
                                          _dev(col_indices, "col_indices", torch.int32),
                                          _dev(q, "q", torch.float16), _dev(kmat, "kmat", torch.float16),
                                          _dev(vmat, "vmat", torch.float16), _dev(out, "out", torch.float16),
                                          _dev(workspace, "workspace", torch.float16), float(scale), batch, _stream())
    _lib.check(rc, "vs_attention_cvse")
    return 0


def softmax_cvse_backward(m_vec, vec_length, row_offsets, probs, grad_probs, grad_scores, scale=1.0):
    """Gradient of softmax_cvse with respect to its scores; all three [nnz] or [B, nnz]; grad_scores may be grad_probs."""
    batch = probs.shape[0] if probs.dim() == 2 else 1
    stride = probs.stride(0) if probs.dim() == 2 and batch > 1 else 0
    device = _one_device(row_offsets=row_offsets, probs=probs, grad_probs=grad_probs, grad_scores=grad_scores)
    with torch.cuda.device(device):
        rc = _lib.lib().vs_softmax_cvse_backward(_dtype_code(probs, "probs"), m_vec, vec_length,
                                                 _dev(row_offsets, "row_offsets", torch.int32), _dev(probs, "probs"),
                                                 _dev(grad_probs, "grad_probs", probs.dtype),
                                                 _dev(grad_scores, "grad_scores", probs.dtype), float(scale), batch, stride,
                                                 _stream())
    _lib.check(rc, "vs_softmax_cvse_backward")
    return 0


def attention_cvse_backward(path, m_vec, vec_length, n, d, nonzeros_vec, row_indices, row_offsets, col_indices, t_offsets,
                            t_rows, t_src, q, kmat, vmat, grad_out, grad_q, grad_k, grad_v, probs_workspace, grad_workspace,
                            scale):
    """Gradients of attention_cvse for [B, ., d] fp16 tensors sharing one mask; both workspaces [B, nnz] fp16."""
    batch = q.shape[0] if q.dim() == 3 else 1
    for w, name in ((probs_workspace, "probs_workspace"), (grad_workspace, "grad_workspace")):
        _need(w, batch * nonzeros_vec * vec_length, name)
    f16 = torch.float16
    for tsr, name in ((col_indices, "col_indices"), (t_rows, "t_rows"), (t_src, "t_src")):
        _need(tsr, nonzeros_vec, name)
    device = _one_device(row_indices=row_indices, row_offsets=row_offsets, col_indices=col_indices, t_offsets=t_offsets,
                         t_rows=t_rows, t_src=t_src, q=q, kmat=kmat, vmat=vmat, grad_out=grad_out, grad_q=grad_q, grad_k=grad_k,
                         grad_v=grad_v, probs_workspace=probs_workspace, grad_workspace=grad_workspace)
    with torch.cuda.device(device):
        rc = _lib.lib().vs_attention_cvse_backward(
            path, m_vec, vec_length, n, d, nonzeros_vec, _dev(row_indices, "row_indices", torch.int32),
            _dev(row_offsets, "row_offsets", torch.int32), _dev(col_indices, "col_indices", torch.int32),
            _dev(t_offsets, "t_offsets", torch.int32), _dev(t_rows, "t_rows", torch.int32), _dev(t_src, "t_src", torch.int32),
            _dev(q, "q", f16), _dev(kmat, "kmat", f16), _dev(vmat, "vmat", f16), _dev(grad_out, "grad_out", f16),
            _dev(grad_q, "grad_q", f16), _dev(grad_k, "grad_k", f16), _dev(grad_v, "grad_v", f16),
            _dev(probs_workspace, "probs_workspace", f16), _dev(grad_workspace, "grad_workspace", f16), float(scale), batch,
            _stream())
    _lib.check(rc, "vs_attention_cvse_backward")
    return 0


def set_workspace(buffer=None) -> None:
    """Hands the tensor-path kernels a caller-owned plan scratch (a CUDA uint8 tensor) for the calls of this host
    thread, or returns to the library's own per-stream buffers (None).  See include/vsparse_b200.h."""
    if buffer is None:
        _lib.check(_lib.lib().vs_set_workspace(None, 0), "vs_set_workspace")
    else:
        _lib.check(_lib.lib().vs_set_workspace(buffer.data_ptr(), buffer.numel() * buffer.element_size()), "vs_set_workspace")


def device_status(clear: bool = True) -> int:
    """Status word of the current device: 0 unless a kernel gave up on a bounded wait."""
    import ctypes as C
    v = C.c_uint32(0)
    _lib.check(_lib.lib().vs_device_status(1 if clear else 0, C.byref(v)), "vs_device_status")
    return int(v.value)


def kernel_timing(enable: bool):
    """Switches the event bracketing of the dense tensor-core multiplying kernels on or off and returns
    (total milliseconds, launches) of the kernels bracketed since the last call (synchronous)."""
    import ctypes as C
    ms, n = C.c_double(0.0), C.c_int(0)
    _lib.check(_lib.lib().vs_kernel_timing(1 if enable else 0, C.byref(ms), C.byref(n)), "vs_kernel_timing")
    return float(ms.value), int(n.value)


def measure_fp32_fma() -> float:
    """fp32 FMA throughput of the current device in TFLOP/s (a register-only probe kernel; synchronous)."""
    import ctypes as C
    v = C.c_double(0.0)
    _lib.check(_lib.lib().vs_measure_fp32_fma(C.byref(v)), "vs_measure_fp32_fma")
    return float(v.value)
