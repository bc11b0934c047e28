"""Optional PyTorch registration of the operators (the reference has none; its tooling around the C++ API is Python).

    torch.ops.vsparse.spmm(path, m_vec, V, row_indices, row_offsets, col_indices, values, rhs) -> C
    torch.ops.vsparse.sddmm(path, m_vec, V, nonzeros_vec, row_indices, row_offsets, col_indices, lhs, rhs) -> values
    torch.ops.vsparse.softmax(m_vec, V, row_indices, row_offsets, scores, scale) -> probabilities
    torch.ops.vsparse.attention(path, m_vec, V, nonzeros_vec, row_indices, row_offsets, col_indices, q, k, v, scale) -> out

thin functional wrappers (they allocate the result) over vectorsparse_b200.ops, registered for the CUDA dispatch key
only: there is no CPU implementation to fall back to.  `FixedMaskAttention` ties the forward and backward operators
of fixed-mask sparse attention into torch.autograd, so that the pair can sit inside a training step:

    mask = AttentionMask(cvse_matrix, device)
    out = fixed_mask_attention(q, k, v, mask, scale)          # [B, n, d] fp16, differentiable in q, k, v

`SparseDenseProduct` does the same for the product itself (a layer with a column-vector-sparse weight):

    c = sparse_dense_product(values, b, mask)                 # [m, N] = A(values) @ b, differentiable in values and b
    # backward: d b = A^T @ d c (vs_spmm_t), d values = (d c @ b^T) sampled at the structure (vs_sddmm)
"""
from __future__ import annotations

import torch

from . import cvse as _cvse
from . import ops
from ._lib import VS_PATH_TENSOR

_LIB = torch.library.Library("vsparse", "DEF")
_LIB.define("spmm(int path, int m_vec, int V, Tensor row_indices, Tensor row_offsets, Tensor col_indices, Tensor values, "
            "Tensor rhs) -> Tensor")
_LIB.define("sddmm(int path, int m_vec, int V, int nonzeros_vec, Tensor row_indices, Tensor row_offsets, Tensor col_indices, "
            "Tensor lhs, Tensor rhs) -> Tensor")
_LIB.define("softmax(int m_vec, int V, Tensor row_indices, Tensor row_offsets, Tensor scores, float scale) -> Tensor")
_LIB.define("attention(int path, int m_vec, int V, int nonzeros_vec, Tensor row_indices, Tensor row_offsets, Tensor col_indices, "
            "Tensor q, Tensor k, Tensor v, float scale) -> Tensor")


def _spmm(path, m_vec, V, row_indices, row_offsets, col_indices, values, rhs):
    batched = rhs.dim() == 3
    n, k = rhs.shape[-2], rhs.shape[-1]
    shape = (rhs.shape[0], m_vec * V, k) if batched else (m_vec * V, k)
    out = torch.empty(shape, dtype=values.dtype, device=values.device)
    if batched:
        ops.spmm_batched(path, m_vec, V, k, n, row_indices, row_offsets, col_indices, values, rhs, out)
    else:
        ops._spmm(path, m_vec, V, k, n, row_indices, row_offsets, col_indices, values, rhs, out)
    return out


def _sddmm(path, m_vec, V, nonzeros_vec, row_indices, row_offsets, col_indices, lhs, rhs):
    batched = lhs.dim() == 3
    n, k = rhs.shape[-2], rhs.shape[-1]
    shape = (lhs.shape[0], nonzeros_vec * V) if batched else (nonzeros_vec * V,)
    out = torch.empty(shape, dtype=lhs.dtype, device=lhs.device)
    if batched:
        ops.sddmm_batched(path, m_vec, k, n, nonzeros_vec, row_indices, row_offsets, col_indices, lhs, rhs, out, V)
    else:
        ops._sddmm(path, m_vec, k, n, nonzeros_vec, row_indices, row_offsets, col_indices, lhs, rhs, out, V, 1)
    return out


def _softmax(m_vec, V, row_indices, row_offsets, scores, scale):
    probs = torch.empty_like(scores)
    ops.softmax_cvse(m_vec, V, row_indices, row_offsets, scores, probs, scale)
    return probs


def _attention(path, m_vec, V, nonzeros_vec, row_indices, row_offsets, col_indices, q, k, v, scale):
    batch = q.shape[0] if q.dim() == 3 else 1
    n, d = k.shape[-2], k.shape[-1]
    out = torch.empty_like(q)
    ws = torch.empty((batch, nonzeros_vec * V), dtype=torch.float16, device=q.device)
    ops.attention_cvse(path, m_vec, V, n, d, nonzeros_vec, row_indices, row_offsets, col_indices, q, k, v, out, ws, scale)
    return out


_LIB.impl("spmm", _spmm, "CUDA")
_LIB.impl("sddmm", _sddmm, "CUDA")
_LIB.impl("softmax", _softmax, "CUDA")
_LIB.impl("attention", _attention, "CUDA")


class AttentionMask:
    """A fixed CVSE mask on one device: the structure the forward operators read and its transpose for the backward
    products (built once, on the host, by cvse.transpose)."""

    def __init__(self, a: _cvse.CVSE, device):
        self.m_vec, self.n, self.V, self.nnz_vec = a.m_vec, a.n, a.V, a.nnz_vec
        self.row_indices, self.row_offsets, self.col_indices = a.to_device(device)
        self.t_offsets, self.t_rows, self.t_src = (torch.from_numpy(x).to(device) for x in _cvse.transpose(a))


class FixedMaskAttention(torch.autograd.Function):
    """softmax(scale * Q K^T at the mask) V with the library's forward and backward operators (the probabilities are
    recomputed in the backward pass, not kept)."""

    @staticmethod
    def forward(ctx, q, k, v, mask: AttentionMask, scale: float, path: int = VS_PATH_TENSOR):
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        out = torch.ops.vsparse.attention(path, mask.m_vec, mask.V, mask.nnz_vec, mask.row_indices, mask.row_offsets,
                                          mask.col_indices, q, k, v, float(scale))
        ctx.save_for_backward(q, k, v)
        ctx.mask, ctx.scale, ctx.path = mask, float(scale), path
        return out

    @staticmethod
    def backward(ctx, grad_out):
        q, k, v = ctx.saved_tensors
        m = ctx.mask
        batch = q.shape[0] if q.dim() == 3 else 1
        gq, gk, gv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        ws_p, ws_g = (torch.empty((batch, m.nnz_vec * m.V), dtype=torch.float16, device=q.device) for _ in range(2))
        ops.attention_cvse_backward(ctx.path, m.m_vec, m.V, m.n, k.shape[-1], m.nnz_vec, m.row_indices, m.row_offsets, m.col_indices,
                                    m.t_offsets, m.t_rows, m.t_src, q, k, v, grad_out.contiguous(), gq, gk, gv, ws_p, ws_g, ctx.scale)
        return gq, gk, gv, None, None, None


def fixed_mask_attention(q, k, v, mask: AttentionMask, scale: float, path: int = VS_PATH_TENSOR):
    return FixedMaskAttention.apply(q, k, v, mask, scale, path)


class SparseDenseProduct(torch.autograd.Function):
    """C = A @ B with A a CVSE matrix (structure in `mask`, values a tensor), fp16, single or batched (values [nnz] or
    [batch, nnz], B [K, N] or [batch, K, N]).  The backward pass is two of the library's operators: the product with
    the transposed matrix for B, the sampled dense-dense product for the values; with batched B and shared values the
    gradients of the values are summed over the batch."""

    @staticmethod
    def forward(ctx, values, b, mask: AttentionMask, path: int = VS_PATH_TENSOR):
        values, b = values.contiguous(), b.contiguous()
        c = torch.ops.vsparse.spmm(path, mask.m_vec, mask.V, mask.row_indices, mask.row_offsets, mask.col_indices, values, b)
        ctx.save_for_backward(values, b)
        ctx.mask, ctx.path = mask, path
        return c

    @staticmethod
    def backward(ctx, grad_c):
        values, b = ctx.saved_tensors
        m = ctx.mask
        grad_c = grad_c.contiguous()
        grad_values = grad_b = None
        if ctx.needs_input_grad[1]:
            grad_b = torch.empty_like(b)
            ops.spmm_t(m.m_vec, m.V, b.shape[-1], m.n, m.t_offsets, m.t_rows, m.t_src, values, grad_c, grad_b, m.nnz_vec)
        if ctx.needs_input_grad[0]:
            g = torch.ops.vsparse.sddmm(ctx.path, m.m_vec, m.V, m.nnz_vec, m.row_indices, m.row_offsets, m.col_indices, grad_c, b)
            grad_values = g.sum(0) if (g.dim() == 2 and values.dim() == 1) else g
        return grad_values, grad_b, None, None


def sparse_dense_product(values, b, mask: AttentionMask, path: int = VS_PATH_TENSOR):
    return SparseDenseProduct.apply(values, b, mask, path)
