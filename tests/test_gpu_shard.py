"""The two partitions of the operators over the GPUs of one box (columns of the dense operand for SpMM, batch x head for
fixed-mask attention), run on ONE GPU: the G shards of a problem are computed one after another through
vectorsparse_b200.shard on the real kernels and reassembled; since neither partition changes the order of any sum,
the result must equal the unsharded one bit for bit, for G = 2, 4 and 8.  (The same helpers run one shard per rank
under torch.distributed; tests/test_shard_gloo.py covers the collectives on CPU.)"""
import numpy as np
import pytest
import torch

from gpu_util import DEV, dev, problem, structure
from vectorsparse_b200 import VS_PATH_TENSOR, cvse, ops, shard

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("G", [2, 4, 8])
@pytest.mark.parametrize("V", [1, 4])
def test_column_shards_of_the_fp32_spmm(G, V):
    """M = K = 4096 fp32 at 90 % sparsity, N = 1024: G column blocks of B, each multiplied alone (cudaSpmm)."""
    N, K = 1024, 4096
    a = problem(cvse.GEN_UNIFORM, 60 + V, 4096 // V, K, V, 0.9)
    st = structure(a)
    vals = dev(cvse.fill_random((a.nnz_vec * V,), np.float32, cvse.DIST_UNIFORM, 1))
    B = torch.from_numpy(cvse.fill_random((K, N), np.float32, cvse.DIST_UNIFORM, 2, 1.0)).to(DEV)
    full = torch.empty((a.m, N), dtype=torch.float32, device=DEV)
    ops.spmm.cudaSpmm(a.m_vec, V, N, K, *st, vals, B, full)
    parts = []
    for rank in range(G):
        B_local = shard.take_columns(B, rank, G)
        out_local = torch.full((a.m, B_local.shape[1]), float("nan"), dtype=torch.float32, device=DEV)
        shard.spmm_column_sharded(ops.spmm.cudaSpmm, a.m_vec, V, N, K, st, vals, B_local, out_local)
        parts.append(out_local)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert [p.shape[1] for p in parts] == [w for _, w in shard.column_shards(N, G)]
    assert torch.equal(torch.cat(parts, dim=1), full)


@pytest.mark.parametrize("G", [2, 4, 8])
def test_column_shards_of_the_tensor_core_spmm(G):
    """fp16 tensor-core SpMM, N = 1024: shards of 512, 256 and 128 columns go through the pair kernel, the unsharded
    product too; same bits."""
    V, N, K = 8, 1024, 512
    a = problem(cvse.GEN_BETA, 70, 1024 // V, K, V, 0.9)
    st = structure(a)
    vals = dev(cvse.fill_random((a.nnz_vec * V,), np.float16, cvse.DIST_NORMAL, 1, 0.5))
    B = torch.from_numpy(cvse.fill_random((K, N), np.float16, cvse.DIST_NORMAL, 2, 1.0)).to(DEV)
    full = torch.empty((a.m, N), dtype=torch.float16, device=DEV)
    ops.spmm.wmmaSpmm(a.m_vec, V, N, K, *st, vals, B, full)
    parts = []
    for rank in range(G):
        B_local = shard.take_columns(B, rank, G)
        out_local = torch.full((a.m, B_local.shape[1]), float("nan"), dtype=torch.float16, device=DEV)
        shard.spmm_column_sharded(ops.spmm.wmmaSpmm, a.m_vec, V, N, K, st, vals, B_local, out_local)
        parts.append(out_local)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert torch.equal(torch.cat(parts, dim=1), full)


@pytest.mark.parametrize("G", [2, 4, 8])
def test_batch_shards_of_fixed_mask_attention(G):
    """16 heads sharing one band + strided mask (sequence 1024, head dimension 64), split into G contiguous ranges."""
    V, d, n, heads = 8, 64, 1024, 16
    a = problem(cvse.GEN_BAND, 8, n // V, n, V, 0.9, band=128)
    ri, ro, ci = structure(a)
    q, k, v = (torch.from_numpy(cvse.fill_random((heads, n, d), np.float16, cvse.DIST_NORMAL, 20 + i, 1.0)).to(DEV) for i in range(3))
    full = torch.empty((heads, n, d), dtype=torch.float16, device=DEV)
    ws = torch.empty((heads, a.nnz_vec * V), dtype=torch.float16, device=DEV)
    ops.attention_cvse(VS_PATH_TENSOR, a.m_vec, V, n, d, a.nnz_vec, ri, ro, ci, q, k, v, full, ws, 0.125)
    parts = []
    for h0, cnt in shard.batch_shards(heads, G):
        o = torch.full((cnt, n, d), float("nan"), dtype=torch.float16, device=DEV)
        w = torch.empty((cnt, a.nnz_vec * V), dtype=torch.float16, device=DEV)
        ops.attention_cvse(VS_PATH_TENSOR, a.m_vec, V, n, d, a.nnz_vec, ri, ro, ci, q[h0:h0 + cnt].contiguous(),
                           k[h0:h0 + cnt].contiguous(), v[h0:h0 + cnt].contiguous(), o, w, 0.125)
        parts.append(o)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert torch.equal(torch.cat(parts, dim=0), full)
