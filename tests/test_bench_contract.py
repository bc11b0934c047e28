"""bench.py's bookkeeping, checked on the CPU: the algorithmic flops and bytes every workload reports follow the
formulas of the operators' definitions, and every workload names the kernels a step launches."""
import importlib.util
import os

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
spec = importlib.util.spec_from_file_location("vs_bench", os.path.join(ROOT, "bench.py"))
bench = importlib.util.module_from_spec(spec)
spec.loader.exec_module(bench)


def test_default_workload_bytes_and_flops():
    w = bench.WORKLOADS["spmm_v8_s90"]
    a = bench.build_problem(w)
    flops, nbytes = bench.algorithmic(w, a)
    assert a.nnz_vec == 12685 and a.m_vec == 256
    assert flops == 2.0 * a.nnz_vec * 8 * 256 * 256
    # per instance: values + touched rows of B + C; once: column indices, row offsets and row order
    k_touched = int(np.unique(a.col_indices).size)
    per = a.nnz_vec * 8 * 2 + k_touched * 256 * 2 + 2048 * 256 * 2
    assert nbytes == per * 256 + a.nnz_vec * 4 + (2 * a.m_vec + 1) * 4 == 387554872


@pytest.mark.parametrize("name", sorted(bench.WORKLOADS))
def test_every_workload_is_described(name):
    w = bench.WORKLOADS[name]
    if w["M"] * w["K"] > 2048 * 2048:
        pytest.skip("large pattern: generated on the benchmark box only")
    a = bench.build_problem(w)
    flops, nbytes = bench.algorithmic(w, a)
    assert flops > 0 and nbytes > 0
    assert flops / nbytes < 400, "arithmetic intensity of a sparse product stays far below the dense ridge"
    assert bench.metric_name(w).endswith(")")


def test_transposed_and_attention_formulas():
    w = bench.WORKLOADS["spmm_t_v8_s90"]
    a = bench.build_problem(w)
    flops, nbytes = bench.algorithmic(w, a)
    assert flops == 2.0 * a.nnz_vec * 8 * 256 * 256
    rows_touched = int(np.count_nonzero(np.diff(a.row_offsets))) * 8
    per = a.nnz_vec * 8 * 2 + rows_touched * 256 * 2 + 512 * 256 * 2
    assert nbytes == per * 256 + a.nnz_vec * 8 + (512 + 1) * 4
    for name, products, passes, dense in (("attention_cfg5", 2, 4, 4), ("attention_bwd_cfg5", 5, 10, 7)):
        w = dict(bench.WORKLOADS[name], M=512, K=512, inst=2)       # the same recipe on a small mask
        a = bench.build_problem(w)
        flops, nbytes = bench.algorithmic(w, a)
        nnz = a.nnz_vec * 8
        assert flops == products * 2.0 * nnz * 64 * 2
        assert nbytes == (dense * 512 * 64 * 2 + passes * nnz * 2) * 2 + a.nnz_vec * 4 + (2 * a.m_vec + 1) * 4
