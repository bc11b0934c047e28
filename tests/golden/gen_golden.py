"""Generates tests/golden/reference_host.npz: small CVSE problems with the outputs of the vectorSparse
reference's OWN host verification code (compiled by `make -C oracle ref` from the reference checkout) and of
the fp64 oracle.

Run where the reference checkout exists:   python tests/golden/gen_golden.py
The .npz is committed; the tests only read it.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle  # noqa: E402


def pattern(rng, m_vec, K, lens):
    ro = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    ci = np.concatenate([np.sort(rng.choice(K, int(l), replace=False)) for l in lens] + [np.zeros(0, np.int64)])
    return ro, ci.astype(np.int32)


def main():
    oracle.build(ref=True)
    if oracle.ref() is None:
        raise SystemExit("oracle/_ref/libvsref.so missing: the reference checkout is needed")
    rng = np.random.default_rng(20211114)
    out = {}
    names = []
    # (name, m_vec, K, V, N, k, row lengths)
    cases = [
        ("v2_small", 8, 16, 2, 8, 16, [3, 0, 1, 16, 5, 0, 2, 7]),
        ("v4_small", 8, 16, 4, 8, 16, [1, 2, 3, 4, 0, 6, 7, 8]),
        ("v8_small", 8, 16, 8, 8, 16, [0, 0, 5, 16, 1, 9, 2, 0]),
        ("v8_tail15_17", 6, 64, 8, 64, 64, [15, 17, 16, 31, 33, 32]),
        ("v4_tail", 5, 160, 4, 64, 64, [127, 128, 129, 1, 0]),
        ("v1_fine", 16, 32, 1, 16, 32, [0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 32]),
        ("v8_single_row", 1, 40, 8, 64, 64, [40]),
        ("v2_all_empty", 4, 8, 2, 8, 8, [0, 0, 0, 0]),
    ]
    for name, m_vec, K, V, N, k, lens in cases:
        ro, ci = pattern(rng, m_vec, K, lens)
        nnz = int(ro[-1])
        vals32 = rng.standard_normal(nnz * V).astype(np.float32)
        B32 = rng.uniform(-1, 1, (K, N)).astype(np.float32)
        lhs32 = rng.standard_normal((m_vec * V, k)).astype(np.float32)
        rhs32 = rng.standard_normal((K, k)).astype(np.float32)
        vals16, B16, lhs16, rhs16 = (x.astype(np.float16) for x in (vals32, B32, lhs32, rhs32))
        d = dict(m_vec=m_vec, K=K, V=V, N=N, k=k, row_offsets=ro, col_indices=ci, values32=vals32, B32=B32,
                 lhs32=lhs32, rhs32=rhs32, values16=vals16, B16=B16, lhs16=lhs16, rhs16=rhs16)
        # the reference's own host code
        d["ref_spmm_f32"] = oracle.ref_spmm(m_vec, V, N, ro, ci, vals32, B32)
        d["ref_spmm_h16"] = oracle.ref_spmm(m_vec, V, N, ro, ci, vals16, B16)
        d["ref_sddmm_f32"] = oracle.ref_sddmm(m_vec, k, V, ro, ci, lhs32, rhs32)
        d["ref_sddmm_h16"] = oracle.ref_sddmm(m_vec, k, V, ro, ci, lhs16, rhs16)
        d["ref_sddmm_h16_out16"] = oracle.ref_sddmm(m_vec, k, V, ro, ci, lhs16, rhs16, out16=True)
        sw = oracle.ref_row_swizzle(True, m_vec, ro)
        d["ref_sorted_lengths"] = np.diff(ro)[sw].astype(np.int32)
        d["ref_identity"] = oracle.ref_row_swizzle(False, m_vec, ro)
        # the fp64 parity reference (fp16 inputs promoted exactly)
        d["f64_spmm_h16"] = oracle.spmm(m_vec, V, N, ro, ci, vals16.astype(np.float32), B16.astype(np.float32))
        d["f64_sddmm_h16"] = oracle.sddmm(m_vec, k, V, ro, ci, lhs16.astype(np.float32), rhs16.astype(np.float32))
        d["f64_spmm_f32"] = oracle.spmm(m_vec, V, N, ro, ci, vals32, B32)
        sc = d["f64_sddmm_h16"].astype(np.float32)
        d["f64_softmax"] = oracle.softmax(m_vec, V, ro, sc, 0.125)
        for key, val in d.items():
            out[f"{name}/{key}"] = np.asarray(val)
        names.append(name)
    out["names"] = np.array(names)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_host.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
