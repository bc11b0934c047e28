"""Sharding of the CVSE operators over the GPUs of one box — one process per GPU (torch.distributed).

Neither sharding needs a collective on the data path:
  * SpMM is split by COLUMNS of the dense operand: column j of C depends only on column j of B, so rank g holds
    B[:, c0:c0+w] contiguously (pitch w), computes the same columns of C, and the sparse matrix is replicated.
  * Batched SDDMM / softmax / attention are split by batch x head: contiguous ranges of independent problems that
    share one mask.
The only communication offered is an optional all-gather for callers that want one gathered result.
PyTorch is plumbing here (process group, device memory); the arithmetic is in libvsparse_b200.so.
"""
from __future__ import annotations

from typing import Callable, List, Tuple

import torch
import torch.distributed as dist


def column_shards(n_cols: int, world: int, multiple: int = 64) -> List[Tuple[int, int]]:
    """(first column, width) per rank.  Widths are multiples of `multiple` (64 for the tensor path, 8 / 4 for the
    fp16 / fp32 CUDA-core path) and differ by at most one block; trailing ranks get width 0 when there are fewer
    blocks than ranks (N = 256 over 8 GPUs: four ranks of 64 columns, four idle)."""
    if n_cols % multiple:
        raise ValueError(f"{n_cols} columns cannot be split in blocks of {multiple}")
    blocks = n_cols // multiple
    base, extra = divmod(blocks, world)
    out, start = [], 0
    for r in range(world):
        w = (base + (1 if r < extra else 0)) * multiple
        out.append((start, w))
        start += w
    return out


def batch_shards(batch: int, world: int) -> List[Tuple[int, int]]:
    """(first problem, count) per rank: contiguous ranges of the batch x head index, sizes differing by at most 1."""
    base, extra = divmod(batch, world)
    out, start = [], 0
    for r in range(world):
        c = base + (1 if r < extra else 0)
        out.append((start, c))
        start += c
    return out


def take_columns(dense: torch.Tensor, rank: int, world: int, multiple: int = 64) -> torch.Tensor:
    """This rank's contiguous column block of a [K, N] (or [B, K, N]) dense operand."""
    c0, w = column_shards(dense.shape[-1], world, multiple)[rank]
    return dense[..., c0:c0 + w].contiguous()


def spmm_column_sharded(spmm_fn: Callable, m_vec: int, vec_length: int, n_cols: int, k_sparse: int, structure,
                        values: torch.Tensor, rhs_local: torch.Tensor, out_local: torch.Tensor) -> None:
    """Runs this rank's share: spmm_fn is ops.spmm.wmmaSpmm / ops.spmm.cudaSpmm (or any callable with that
    signature); rhs_local / out_local are the rank's [K, w] / [M, w] blocks.  A rank whose width is 0 does nothing."""
    w = rhs_local.shape[-1]
    if w == 0:
        return
    ri, ro, ci = structure
    spmm_fn(m_vec, vec_length, w, k_sparse, ri, ro, ci, values, rhs_local, out_local)


def gather_columns(out_local: torch.Tensor, n_cols: int, multiple: int = 64, group=None) -> torch.Tensor:
    """All-gathers the per-rank [M, w_r] blocks into one row-major [M, N] matrix on every rank.  Ranks may hold
    different widths (including 0); blocks travel padded to the widest one."""
    world = dist.get_world_size(group)
    shards = column_shards(n_cols, world, multiple)
    w_max = max(w for _, w in shards)
    m = out_local.shape[0]
    padded = out_local.new_zeros((m, w_max))
    padded[:, :out_local.shape[1]] = out_local
    pieces = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(pieces, padded, group=group)
    full = out_local.new_empty((m, n_cols))
    for (c0, w), piece in zip(shards, pieces):
        if w:
            full[:, c0:c0 + w] = piece[:, :w]
    return full


def gather_batch(out_local: torch.Tensor, batch: int, group=None) -> torch.Tensor:
    """All-gathers per-rank [count_r, ...] results of a batch x head sharded operator into [batch, ...]."""
    world = dist.get_world_size(group)
    shards = batch_shards(batch, world)
    c_max = max(c for _, c in shards)
    padded = out_local.new_zeros((c_max,) + tuple(out_local.shape[1:]))
    padded[:out_local.shape[0]] = out_local
    pieces = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(pieces, padded, group=group)
    return torch.cat([piece[:c] for (_, c), piece in zip(shards, pieces)], dim=0)
