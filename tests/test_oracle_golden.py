"""The CPU oracle against the golden vectors produced by the reference's own host code (bit-exact), and — where
the compiled reference shim is present — against that code directly on fresh random problems."""
import numpy as np
import pytest

import oracle


def test_oracle_spmm_f32_matches_reference_loop(golden):
    for name, c in golden.items():
        got = oracle.spmm(c["m_vec"], c["V"], c["N"], c["row_offsets"], c["col_indices"], c["values32"], c["B32"], acc="f32")
        assert np.array_equal(got.view(np.uint32), c["ref_spmm_f32"].view(np.uint32)), name


def test_oracle_spmm_h16_matches_reference_loop(golden):
    for name, c in golden.items():
        got = oracle.spmm(c["m_vec"], c["V"], c["N"], c["row_offsets"], c["col_indices"], c["values16"], c["B16"], acc="f32")
        assert np.array_equal(got.view(np.uint32), c["ref_spmm_h16"].view(np.uint32)), name


def test_oracle_sddmm_matches_host_sddmm(golden):
    for name, c in golden.items():
        a = (c["m_vec"], c["k"], c["V"], c["row_offsets"], c["col_indices"])
        got32 = oracle.sddmm(*a, c["lhs32"], c["rhs32"], acc="f32")
        got16 = oracle.sddmm(*a, c["lhs16"], c["rhs16"], acc="f32")
        assert np.array_equal(got32.view(np.uint32), c["ref_sddmm_f32"].view(np.uint32)), name
        assert np.array_equal(got16.view(np.uint32), c["ref_sddmm_h16"].view(np.uint32)), name
        # OutType = half: Host_sddmm rounds the fp32 accumulator once
        assert np.array_equal(oracle.f32_to_h16(got16).view(np.uint16), c["ref_sddmm_h16_out16"].view(np.uint16)), name


def test_oracle_swizzle_matches_reference(golden):
    for name, c in golden.items():
        ro = c["row_offsets"]
        ident = oracle.row_swizzle(0, c["m_vec"], ro)
        assert np.array_equal(ident, c["ref_identity"]), name
        srt = oracle.row_swizzle(1, c["m_vec"], ro)
        assert sorted(srt.tolist()) == list(range(c["m_vec"])), name
        lens = np.diff(ro)[srt]
        # the reference's std::sort leaves the order of equal-length rows unspecified: compare lengths
        assert np.array_equal(lens, c["ref_sorted_lengths"]), name
        assert np.all(np.diff(lens) <= 0), name


def test_f64_oracle_agrees_with_f32_loops(golden):
    for name, c in golden.items():
        a = (c["m_vec"], c["V"], c["N"], c["row_offsets"], c["col_indices"])
        f64 = oracle.spmm(*a, c["values32"], c["B32"])
        assert np.array_equal(f64, c["f64_spmm_f32"]), name
        if f64.size:
            assert np.max(np.abs(f64 - c["ref_spmm_f32"])) < 1e-4, name
        s64 = oracle.sddmm(c["m_vec"], c["k"], c["V"], c["row_offsets"], c["col_indices"],
                           c["lhs16"].astype(np.float32), c["rhs16"].astype(np.float32))
        assert np.array_equal(s64, c["f64_sddmm_h16"]), name
        if s64.size:
            assert np.max(np.abs(s64 - c["ref_sddmm_h16"])) < 1e-3, name


def test_f64_against_dense_numpy(golden):
    """Independent restatement: densify A and use a plain matrix product."""
    for name, c in golden.items():
        m_vec, V, K = c["m_vec"], c["V"], c["K"]
        ro, ci = c["row_offsets"], c["col_indices"]
        A = np.zeros((m_vec * V, K))
        vals = c["values32"].astype(np.float64).reshape(-1, V)
        for i in range(m_vec):
            A[i * V:(i + 1) * V, ci[ro[i]:ro[i + 1]]] = vals[ro[i]:ro[i + 1]].T
        want = A @ c["B32"].astype(np.float64)
        assert np.allclose(c["f64_spmm_f32"], want, rtol=1e-12, atol=1e-12), name
        full = c["lhs16"].astype(np.float64) @ c["rhs16"].astype(np.float64).T
        want_s = np.concatenate([full[i * V:(i + 1) * V, ci[ro[i]:ro[i + 1]]].T.ravel() for i in range(m_vec)] + [np.zeros(0)])
        assert np.allclose(c["f64_sddmm_h16"], want_s, rtol=1e-12, atol=1e-12), name


def test_softmax_oracle(golden):
    for name, c in golden.items():
        m_vec, V, ro = c["m_vec"], c["V"], c["row_offsets"]
        sc = c["f64_sddmm_h16"].astype(np.float32)
        p = oracle.softmax(m_vec, V, ro, sc, 0.125)
        assert np.array_equal(p, c["f64_softmax"]), name
        p2 = p.reshape(-1, V)
        for i in range(m_vec):
            if ro[i + 1] > ro[i]:
                assert np.allclose(p2[ro[i]:ro[i + 1]].sum(axis=0), 1.0, atol=1e-12)


def test_attention_oracle_is_composition():
    rng = np.random.default_rng(3)
    m_vec, V, n, d = 6, 4, 24, 16
    lens = [3, 0, 24, 1, 7, 5]
    ro = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    ci = np.concatenate([np.sort(rng.choice(n, l, replace=False)) for l in lens]).astype(np.int32)
    Q, K, Vm = (rng.standard_normal(s).astype(np.float32) for s in ((m_vec * V, d), (n, d), (n, d)))
    O = oracle.attention(m_vec, V, d, d, ro, ci, Q, K, Vm, 0.25)
    s = oracle.sddmm(m_vec, d, V, ro, ci, Q, K)
    # softmax oracle takes float32 scores; redo in numpy with the double scores
    P = np.zeros((m_vec * V, n))
    s2 = s.reshape(-1, V)
    for i in range(m_vec):
        if lens[i] == 0:
            continue
        x = 0.25 * s2[ro[i]:ro[i + 1]]
        e = np.exp(x - x.max(axis=0))
        P[i * V:(i + 1) * V, ci[ro[i]:ro[i + 1]]] = (e / e.sum(axis=0)).T
    assert np.allclose(O, P @ Vm.astype(np.float64), rtol=1e-10, atol=1e-12)


@pytest.mark.skipif(oracle.ref() is None, reason="reference shim not built (needs the reference checkout)")
def test_oracle_vs_compiled_reference_random():
    rng = np.random.default_rng(11)
    for V in (1, 2, 4, 8):
        m_vec, K, N, k = 37, 53, 24, 40
        lens = rng.integers(0, K + 1, m_vec)
        ro = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
        ci = np.concatenate([np.sort(rng.choice(K, l, replace=False)) for l in lens]).astype(np.int32)
        vals = rng.standard_normal(int(ro[-1]) * V).astype(np.float32)
        B = rng.uniform(-1, 1, (K, N)).astype(np.float32)
        lhs = rng.standard_normal((m_vec * V, k)).astype(np.float32)
        rhs = rng.standard_normal((K, k)).astype(np.float32)
        for cast in (np.float32, np.float16):
            a = oracle.spmm(m_vec, V, N, ro, ci, vals.astype(cast), B.astype(cast), acc="f32")
            b = oracle.ref_spmm(m_vec, V, N, ro, ci, vals.astype(cast), B.astype(cast))
            assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
            a = oracle.sddmm(m_vec, k, V, ro, ci, lhs.astype(cast), rhs.astype(cast), acc="f32")
            b = oracle.ref_sddmm(m_vec, k, V, ro, ci, lhs.astype(cast), rhs.astype(cast))
            assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
        # threads do not change any bit (rows are independent)
        a1 = oracle.spmm(m_vec, V, N, ro, ci, vals, B, acc="f32", threads=1)
        a4 = oracle.spmm(m_vec, V, N, ro, ci, vals, B, acc="f32", threads=4)
        assert np.array_equal(a1.view(np.uint32), a4.view(np.uint32))
