"""Multi-process sharding logic on CPU (gloo, world size 2): column shards of SpMM and batch x head shards reassemble
to exactly the unsharded result.  The per-rank arithmetic is done by the CPU oracle here (this is a test); on GPUs
the same helpers wrap the CUDA operators."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from vectorsparse_b200 import cvse, shard


def test_shard_plans():
    assert shard.column_shards(8192, 8) == [(i * 1024, 1024) for i in range(8)]
    assert shard.column_shards(256, 8) == [(0, 64), (64, 64), (128, 64), (192, 64)] + [(256, 0)] * 4
    assert shard.column_shards(192, 2) == [(0, 128), (128, 64)]
    assert shard.column_shards(24, 2, multiple=4) == [(0, 12), (12, 12)]
    with pytest.raises(ValueError):
        shard.column_shards(100, 2)
    assert shard.batch_shards(128, 8) == [(i * 16, 16) for i in range(8)]
    assert shard.batch_shards(5, 2) == [(0, 3), (3, 2)]
    assert sum(c for _, c in shard.batch_shards(7, 4)) == 7
    x = torch.arange(6 * 192).reshape(6, 192)
    assert torch.equal(shard.take_columns(x, 1, 2), x[:, 128:192])


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, n_cols):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        V, K = 4, 96
        a = cvse.generate(cvse.GEN_BETA, 5, 24, K, V, 0.7)
        vals = cvse.fill_random((a.nnz_vec * V,), np.float32, cvse.DIST_NORMAL, 1, 1.0)
        B = cvse.fill_random((K, n_cols), np.float32, cvse.DIST_UNIFORM, 2)
        full = oracle.spmm(a.m_vec, V, n_cols, a.row_offsets, a.col_indices, vals, B, acc="f32")

        def cpu_spmm(m_vec, vec_length, k, n, ri, ro, ci, values, rhs, out):  # signature of ops.spmm.cudaSpmm
            out.copy_(torch.from_numpy(oracle.spmm(m_vec, vec_length, k, ro.numpy(), ci.numpy(), values.numpy(),
                                                    rhs.numpy(), acc="f32")))

        structure = tuple(torch.from_numpy(x) for x in (a.row_indices, a.row_offsets, a.col_indices))
        rhs_local = shard.take_columns(torch.from_numpy(B), rank, world)
        out_local = torch.empty((a.m, rhs_local.shape[1]), dtype=torch.float32)
        shard.spmm_column_sharded(cpu_spmm, a.m_vec, V, n_cols, K, structure, torch.from_numpy(vals), rhs_local, out_local)
        gathered = shard.gather_columns(out_local, n_cols)
        # sharding by columns changes no reduction order: the reassembled matrix is bit-identical
        assert np.array_equal(gathered.numpy().view(np.uint32), full.view(np.uint32))

        # batch x head sharding of SDDMM: 5 heads over 2 ranks
        heads, k = 5, 16
        lhs = cvse.fill_random((heads, a.m, k), np.float32, cvse.DIST_NORMAL, 3, 1.0)
        rhs = cvse.fill_random((heads, K, k), np.float32, cvse.DIST_NORMAL, 4, 1.0)
        want = np.stack([oracle.sddmm(a.m_vec, k, V, a.row_offsets, a.col_indices, lhs[h], rhs[h], acc="f32") for h in range(heads)])
        h0, cnt = shard.batch_shards(heads, world)[rank]
        mine = np.stack([oracle.sddmm(a.m_vec, k, V, a.row_offsets, a.col_indices, lhs[h], rhs[h], acc="f32")
                         for h in range(h0, h0 + cnt)])
        got = shard.gather_batch(torch.from_numpy(mine), heads)
        assert np.array_equal(got.numpy().view(np.uint32), want.view(np.uint32))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n_cols", [128, 192, 64])
def test_column_and_batch_shards_world2(n_cols):
    mp.spawn(_worker, args=(2, _free_port(), n_cols), nprocs=2, join=True)
