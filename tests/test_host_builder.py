"""CVSE builder, row swizzle, .smtx I/O and the seeded generators (host only)."""
import hashlib
import os

import numpy as np
import pytest

import oracle
from vectorsparse_b200 import VsError, cvse


def digest(*arrays):
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()[:16]


def test_validate_accepts_and_rejects():
    ro = np.array([0, 2, 2, 5], np.int32)
    ci = np.array([0, 3, 1, 2, 3], np.int32)
    cvse.validate(3, 4, 5, ro, ci)
    for bad_ro, bad_ci, n in (
        (np.array([1, 2, 2, 5], np.int32), ci, 4),       # does not start at 0
        (np.array([0, 3, 2, 5], np.int32), ci, 4),       # not monotone
        (np.array([0, 2, 2, 4], np.int32), ci, 4),       # last offset != nnz
        (ro, np.array([0, 3, 1, 2, 4], np.int32), 4),    # column out of range
        (ro, np.array([0, -1, 1, 2, 3], np.int32), 4),   # negative column
    ):
        with pytest.raises(VsError) as e:
            cvse.validate(3, n, 5, bad_ro, bad_ci)
        assert e.value.code == -6


def test_row_swizzle_matches_oracle_and_is_stable():
    rng = np.random.default_rng(0)
    lens = rng.integers(0, 6, 200)
    ro = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    assert np.array_equal(cvse.row_swizzle(ro, sort=False), np.arange(200, dtype=np.int32))
    got = cvse.row_swizzle(ro, sort=True)
    assert np.array_equal(got, oracle.row_swizzle(1, 200, ro))
    # descending length, ties in ascending index order
    want = np.array(sorted(range(200), key=lambda i: (-lens[i], i)), np.int32)
    assert np.array_equal(got, want)
    assert cvse.row_swizzle(np.array([0], np.int32)).size == 0


def test_generators_shapes_and_laws():
    a = cvse.generate(cvse.GEN_FIXED, 0, 64, 256, 4, 0.9)
    a.validate()
    assert a.nnz_vec == 64 * 26 and np.all(np.diff(a.row_offsets) == 26)
    for i in range(a.m_vec):
        row = a.col_indices[a.row_offsets[i]:a.row_offsets[i + 1]]
        assert np.all(np.diff(row) > 0)

    b = cvse.generate(cvse.GEN_BETA, 7, 256, 512, 8, 0.9)
    b.validate()
    lens = np.diff(b.row_offsets)
    assert 0.08 < lens.mean() / 512 < 0.12 and lens.max() > 1.5 * lens.mean() and lens.min() < 0.5 * lens.mean()
    assert np.all(np.diff(lens[b.row_indices]) <= 0)  # sorted swizzle: longest first

    c = cvse.generate(cvse.GEN_UNIFORM, 2, 128, 128, 1, 0.8)
    c.validate()
    assert c.nnz_vec == round(128 * 128 * 0.2)

    e = cvse.generate(cvse.GEN_BAND, 3, 64, 512, 8, 0.9, band=64)
    e.validate()
    assert np.all(np.diff(e.row_offsets) == 64)  # round(0.1*512)=51 < band: the band wins
    e = cvse.generate(cvse.GEN_BAND, 3, 64, 512, 8, 0.85, band=64)
    assert np.all(np.diff(e.row_offsets) == 77)
    for i in (0, 17, 63):
        row = set(e.col_indices[e.row_offsets[i]:e.row_offsets[i + 1]].tolist())
        centre = i * 8 + 4
        lo = min(max(centre - 32, 0), 512 - 64)
        assert set(range(lo, lo + 64)) <= row
        extra = sorted(row - set(range(lo, lo + 64)))
        assert len({x % 16 for x in extra}) == 1  # strided part sits on one phase of the stride-16 lattice


def test_generators_are_deterministic():
    """A seed names one matrix: the digests pin the generator across platforms and refactors."""
    a = cvse.generate(cvse.GEN_FIXED, 0, 64, 256, 4, 0.9)
    b = cvse.generate(cvse.GEN_FIXED, 0, 64, 256, 4, 0.9)
    assert digest(a.row_offsets, a.col_indices) == digest(b.row_offsets, b.col_indices)
    c = cvse.generate(cvse.GEN_FIXED, 1, 64, 256, 4, 0.9)
    assert digest(a.col_indices) != digest(c.col_indices)
    x = cvse.fill_random((1000,), np.float32, cvse.DIST_NORMAL, 5, 0.02)
    y = cvse.fill_random((1000,), np.float32, cvse.DIST_NORMAL, 5, 0.02)
    assert np.array_equal(x, y)
    # prefix property: a longer draw starts with the shorter one (counter-based)
    z = cvse.fill_random((2000,), np.float32, cvse.DIST_NORMAL, 5, 0.02)
    assert np.array_equal(z[:1000], x)
    h = cvse.fill_random((1000,), np.float16, cvse.DIST_NORMAL, 5, 0.02)
    assert np.array_equal(h, oracle.f32_to_h16(x))  # fp16 = the fp32 draw rounded once
    u = cvse.fill_random((100000,), np.float32, cvse.DIST_UNIFORM, 9)
    assert -1.0 <= u.min() and u.max() < 1.0 and abs(u.mean()) < 0.01
    n = cvse.fill_random((200000,), np.float32, cvse.DIST_NORMAL, 9, 1.0)
    assert abs(n.mean()) < 0.01 and abs(n.std() - 1.0) < 0.01


def test_smtx_round_trip(tmp_path):
    a = cvse.generate(cvse.GEN_BETA, 4, 32, 96, 2, 0.7)
    p = str(tmp_path / "a.smtx")
    cvse.to_smtx(p, a)
    text = open(p).read().split("\n")
    assert text[0] == f"{a.m_vec}, {a.n}, {a.nnz_vec}"  # header as the reference parses it: "rows, cols, nnz"
    b = cvse.from_smtx(p, 2)
    assert (b.m_vec, b.n, b.V) == (a.m_vec, a.n, 2)
    assert np.array_equal(a.row_offsets, b.row_offsets) and np.array_equal(a.col_indices, b.col_indices)
    assert np.array_equal(a.row_indices, b.row_indices)
    with pytest.raises(VsError) as e:
        cvse.from_smtx(str(tmp_path / "missing.smtx"), 2)
    assert e.value.code == -7
    bad = tmp_path / "bad.smtx"
    bad.write_text("2, 4, 3\n0 1 3\n0 1 9\n")  # column 9 >= 4
    with pytest.raises(VsError) as e:
        cvse.from_smtx(str(bad), 2)
    assert e.value.code == -6
    trunc = tmp_path / "trunc.smtx"
    trunc.write_text("2, 4, 3\n0 1 3\n0 1\n")
    with pytest.raises(VsError) as e:
        cvse.from_smtx(str(trunc), 2)
    assert e.value.code == -7


def test_dense_mask_round_trip():
    rng = np.random.default_rng(1)
    mask = rng.random((17, 33)) < 0.2
    mask[5] = False
    a = cvse.from_dense_mask(mask, 4)
    a.validate()
    assert a.nnz_vec == int(mask.sum())
    vals = np.arange(1, a.nnz_vec * 4 + 1, dtype=np.float32)
    dense = a.to_dense(vals)
    assert dense.shape == (68, 33)
    assert np.array_equal((dense.reshape(17, 4, 33) != 0).all(axis=1), mask)


@pytest.mark.parametrize("V", [1, 2, 4, 8])
@pytest.mark.parametrize("per_row", [False, True])
def test_prune_dense_keeps_the_heaviest_vectors(V, per_row):
    rng = np.random.default_rng(10 + V)
    m_vec, n, s = 12, 40, 0.8
    w = rng.standard_normal((m_vec * V, n)).astype(np.float32)
    a, vals = cvse.prune_dense(w, V, s, per_row=per_row)
    a.validate()
    score = np.abs(w.astype(np.float64)).reshape(m_vec, V, n).sum(axis=1)
    if per_row:
        keep = int(round((1 - s) * n))
        assert np.all(np.diff(a.row_offsets) == keep)
        for i in range(m_vec):
            cols = a.col_indices[a.row_offsets[i]:a.row_offsets[i + 1]]
            assert np.all(np.diff(cols) > 0)
            assert set(cols) == set(np.argsort(-score[i], kind="stable")[:keep])
    else:
        keep = int(round((1 - s) * m_vec * n))
        assert a.nnz_vec == keep
        best = set(np.argsort(-score.ravel(), kind="stable")[:keep])
        got = {i * n + int(c) for i in range(m_vec) for c in a.col_indices[a.row_offsets[i]:a.row_offsets[i + 1]]}
        assert got == best
    # the values are the kept weights in the CVSE layout, so the dense expansion is the masked weight
    dense = a.to_dense(vals)
    mask = np.repeat((a.to_dense(np.ones(a.nnz_vec * V, np.float32)) != 0), 1, axis=0)
    assert np.array_equal(dense, np.where(mask, w, 0).astype(np.float32))


def test_prune_dense_edges():
    w = np.ones((8, 5), np.float32)
    a, vals = cvse.prune_dense(w, 4, 1.0)          # everything pruned
    assert a.nnz_vec == 0 and vals.size == 0 and np.all(a.row_offsets == 0)
    a, vals = cvse.prune_dense(w, 4, 0.0)          # nothing pruned
    assert a.nnz_vec == 10 and np.array_equal(a.to_dense(vals), w)
    a, _ = cvse.prune_dense(w, 4, 0.5)             # all scores tie: the lower (vector-row, column) wins
    assert a.nnz_vec == 5 and list(np.diff(a.row_offsets)) == [5, 0]
    with pytest.raises(VsError):
        cvse.prune_dense(w, 4, 1.5)
    with pytest.raises(ValueError):
        cvse.prune_dense(np.ones((6, 5), np.float32), 4, 0.5)
