"""Oracle of the attention backward pass (no reference counterpart: parity unpinned).  What can be checked on the
host: the softmax gradient against finite differences of the oracle's own forward softmax, and the composed
backward pass against finite differences of the oracle's forward attention."""
import numpy as np

import oracle
from vectorsparse_b200 import cvse


def test_softmax_backward_matches_finite_differences():
    V, scale = 4, 0.3
    a = cvse.generate(cvse.GEN_BETA, 4, 6, 20, V, 0.6)
    rng = np.random.default_rng(0)
    s = rng.standard_normal(a.nnz_vec * V).astype(np.float32)
    g = rng.standard_normal(a.nnz_vec * V)
    p = oracle.softmax(a.m_vec, V, a.row_offsets, s, scale)
    got = oracle.softmax_backward(a.m_vec, V, a.row_offsets, p, g, scale)
    eps = 1e-3
    for idx in rng.choice(s.size, 12, replace=False):
        sp, sm = s.copy(), s.copy()
        sp[idx] += eps
        sm[idx] -= eps
        lp = (oracle.softmax(a.m_vec, V, a.row_offsets, sp, scale) * g).sum()
        lm = (oracle.softmax(a.m_vec, V, a.row_offsets, sm, scale) * g).sum()
        fd = (lp - lm) / (float(sp[idx]) - float(sm[idx]))
        assert abs(fd - got[idx]) <= 1e-4 * max(1.0, abs(fd)), (idx, fd, got[idx])


def test_attention_backward_matches_finite_differences():
    V, d, n, scale = 2, 8, 12, 0.35
    a = cvse.generate(cvse.GEN_FIXED, 9, n // V, n, V, 0.5)
    rng = np.random.default_rng(1)
    Q, K, Vm, dO = (rng.standard_normal((n, d)).astype(np.float32) for _ in range(4))
    dQ, dK, dV = oracle.attention_backward(a.m_vec, V, d, a.row_offsets, a.col_indices, Q, K, Vm, dO, scale)

    def loss(q, k, v):
        return float((oracle.attention(a.m_vec, V, d, d, a.row_offsets, a.col_indices, q, k, v, scale) * dO).sum())

    eps = 1e-2   # inputs are float32: a wide step keeps the difference quotient clear of their rounding
    for which, grad in ((0, dQ), (1, dK), (2, dV)):
        for _ in range(6):
            r, c = int(rng.integers(n)), int(rng.integers(d))
            args_p, args_m = [Q.copy(), K.copy(), Vm.copy()], [Q.copy(), K.copy(), Vm.copy()]
            args_p[which][r, c] += eps
            args_m[which][r, c] -= eps
            h = float(args_p[which][r, c]) - float(args_m[which][r, c])
            fd = (loss(*args_p) - loss(*args_m)) / h
            assert abs(fd - grad[r, c]) <= 2e-3 * max(1.0, abs(fd)), (which, r, c, fd, grad[r, c])
