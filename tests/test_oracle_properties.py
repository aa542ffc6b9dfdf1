"""The oracle against independent NumPy/list references, in the manner of the
reference's property tests (Test/NoFib/Prelude/{Fold,Scan,Permute,Stencil}.hs:
random shapes and arrays, result compared with a sequential list reference)."""
import numpy as np
from hypothesis import given, settings, strategies as st

import accelerate_b200 as A
from oracle import oracle

add = lambda a, b: a + b  # noqa: E731
shapes2 = st.tuples(st.integers(0, 12), st.integers(0, 24))


def ints(shape, seed):
    return np.random.default_rng(seed).integers(-100, 100, size=shape).astype(np.int64)


@settings(max_examples=40, deadline=None)
@given(shapes2, st.integers(0, 1 << 30))
def test_fold_and_scans_match_numpy(shape, seed):
    m = ints(shape, seed)
    assert np.array_equal(oracle.run(A.fold(add, 7, m)), m.sum(axis=1) + 7)                     # foldRef, Fold.hs:235
    want = np.concatenate([np.full((shape[0], 1), 3), 3 + np.cumsum(m, axis=1)], axis=1)
    assert np.array_equal(oracle.run(A.scanl(add, 3, m)), want)                                # scanlRef, Scan.hs:777
    rs = np.cumsum(m[:, ::-1], axis=1)[:, ::-1]
    want_r = np.concatenate([3 + rs, np.full((shape[0], 1), 3)], axis=1)
    assert np.array_equal(oracle.run(A.scanr(add, 3, m)), want_r)                              # scanrRef
    p, s = oracle.run(list(A.scanr_prime(add, 0, m)))
    assert np.array_equal(s, m.sum(axis=1))
    assert np.array_equal(p, np.concatenate([rs[:, 1:], np.zeros((shape[0], 1), np.int64)], axis=1) if shape[1] else p)
    if shape[1] > 0:
        assert np.array_equal(oracle.run(A.fold1(A.max_, m)), m.max(axis=1))
        assert np.array_equal(oracle.run(A.scanl1(add, m)), np.cumsum(m, axis=1))
        assert np.array_equal(oracle.run(A.scanr1(A.min_, m)), np.minimum.accumulate(m[:, ::-1], axis=1)[:, ::-1])


@settings(max_examples=30, deadline=None)
@given(st.lists(st.integers(0, 9), min_size=1, max_size=12), st.integers(0, 1 << 30))
def test_foldseg_matches_list_reference(lens, seed):
    lens = np.array(lens, np.int32)
    x = ints(int(lens.sum()), seed)
    off = np.concatenate([[0], np.cumsum(lens)])
    want = np.array([x[off[i]:off[i + 1]].sum() for i in range(len(lens))], np.int64)          # foldSegRef, Fold.hs:254
    assert np.array_equal(oracle.run(A.foldSeg(add, 0, x, lens)), want)


@settings(max_examples=30, deadline=None)
@given(st.integers(0, 200), st.integers(1, 17), st.integers(0, 1 << 30))
def test_permute_accumulate_matches_sequential_reference(n, bins, seed):
    g = np.random.default_rng(seed)
    keys = g.integers(-1, bins, size=n).astype(np.int64)           # -1 = Nothing
    vals = g.integers(-50, 50, size=n).astype(np.int64)
    want = np.zeros(bins, np.int64)
    for k, v in zip(keys, vals):                                   # permuteRef, Permute.hs:149-179
        if k >= 0:
            want[k] = v + want[k]
    ku = A.use(keys)
    got = oracle.run(A.permute(add, A.fill(bins, A.constant(0)), lambda ix: A.cond(ku[ix] < 0, A.Nothing_(1), A.Just_(A.index(ku[ix]))), vals))
    assert np.array_equal(got, want)


@settings(max_examples=25, deadline=None)
@given(st.tuples(st.integers(2, 9), st.integers(2, 11)), st.sampled_from(["clamp", "mirror", "wrap"]), st.integers(0, 1 << 30))
def test_stencil_3x3_matches_padded_reference(shape, bnd, seed):
    m = ints(shape, seed)
    mode = {"clamp": "edge", "mirror": "reflect", "wrap": "wrap"}[bnd]     # bound, Stencil.hs:637-669
    p = np.pad(m, 1, mode=mode)
    want = sum(p[i:i + shape[0], j:j + shape[1]] * (3 * i + j + 1) for i in range(3) for j in range(3))
    b = {"clamp": A.clamp, "mirror": A.mirror, "wrap": A.wrap}[bnd]
    got = oracle.run(A.stencil(lambda s: sum((s[i][j] * (3 * i + j + 1) for i in range(3) for j in range(3)), A.constant(0)), b, m))
    assert np.array_equal(got, want)
