"""Host side of the transposed product: the structure of A^T (vs_cvse_transpose) and the oracle's restatement.
The reference has no transposed operator, so the oracle function is pinned here by the one thing it must equal:
the forward oracle (a restatement of spmm_benchmark.cpp:66-86, itself pinned to the reference's host loop) run on
A^T written out as a V = 1 CVSE matrix."""
import numpy as np
import pytest

import oracle
from vectorsparse_b200 import cvse
from vectorsparse_b200._lib import VsError


def _transposed_as_v1(a, vals):
    """A^T as a V = 1 CVSE matrix with values: row c holds (column i*V+v, value) for every vector (i, c) of A."""
    t_off, t_rows, t_src = cvse.transpose(a)
    V = a.V
    ro = (t_off.astype(np.int64) * V).astype(np.int32)
    ci = (t_rows[:, None].astype(np.int64) * V + np.arange(V)[None, :]).reshape(-1).astype(np.int32)
    v = vals.reshape(-1, V)[t_src].reshape(-1)
    return ro, ci, v


@pytest.mark.parametrize("V", [1, 2, 4, 8])
def test_transpose_lists_every_vector_once_in_row_order(V):
    a = cvse.generate(cvse.GEN_BETA, 11 + V, 24, 50, V, 0.7)
    t_off, t_rows, t_src = cvse.transpose(a)
    assert t_off[0] == 0 and t_off[-1] == a.nnz_vec and np.all(np.diff(t_off) >= 0)
    assert sorted(t_src.tolist()) == list(range(a.nnz_vec))
    row_of = np.repeat(np.arange(a.m_vec), np.diff(a.row_offsets))
    assert np.array_equal(t_rows, row_of[t_src])
    for c in range(a.n):
        seg = slice(t_off[c], t_off[c + 1])
        assert np.all(a.col_indices[t_src[seg]] == c)
        assert np.all(np.diff(t_rows[seg]) > 0)


def test_transpose_edges():
    empty = cvse.CVSE(3, 5, 4, np.zeros(4, np.int32), np.zeros(0, np.int32), np.arange(3, dtype=np.int32))
    t_off, t_rows, t_src = cvse.transpose(empty)
    assert np.all(t_off == 0) and t_rows.size == 0 and t_src.size == 0
    bad = cvse.CVSE(1, 4, 2, np.array([0, 2], np.int32), np.array([1, 9], np.int32), np.zeros(1, np.int32))
    with pytest.raises(VsError) as e:
        cvse.transpose(bad)
    assert e.value.code == -6


@pytest.mark.parametrize("V", [1, 2, 4, 8])
def test_oracle_spmm_t_equals_forward_oracle_on_the_transposed_matrix(V):
    a = cvse.generate(cvse.GEN_UNIFORM, 5 + V, 16, 40, V, 0.8)
    rng = np.random.default_rng(V)
    vals = rng.standard_normal(a.nnz_vec * V).astype(np.float32)
    B = rng.standard_normal((a.m_vec * V, 24)).astype(np.float32)
    got = oracle.spmm_t(a.m_vec, V, 24, a.n, a.row_offsets, a.col_indices, vals, B)
    ro, ci, v = _transposed_as_v1(a, vals)
    want = oracle.spmm(a.n, 1, 24, ro, ci, v, B, acc="f64")
    np.testing.assert_allclose(got, want, rtol=1e-12, atol=1e-12)
    dense = a.to_dense(vals).astype(np.float64)
    np.testing.assert_allclose(got, dense.T @ B.astype(np.float64), rtol=1e-10, atol=1e-10)
