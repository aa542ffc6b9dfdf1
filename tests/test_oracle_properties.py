"""The oracle against independent NumPy/list references, in the manner of the
reference's property tests (Test/NoFib/Prelude/{Fold,Scan,Permute,Stencil}.hs:
random shapes and arrays, result compared with a sequential list reference)."""
import numpy as np
import pytest
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


# ---- stencils against the reference suite's own list-based references ------------------------
# Every shape Test/NoFib/Prelude/Stencil.hs:48-97 lists, at its sizes (:112, :130, :148, :166,
# :186-188 ...), with a random tap pattern and a random boundary out of clamp / mirror / wrap /
# constant, the latter written as `function (\_ -> constant x)` as the reference's tests do (:118).
from tests import stencil_ref as SR  # noqa: E402

STENCIL_SHAPES = [((3,), 2, 256), ((5,), 3, 256), ((7,), 4, 256), ((9,), 5, 256),
                  ((3, 3), 2, 96), ((5, 5), 3, 96), ((7, 7), 4, 96), ((9, 9), 5, 96), ((3, 3, 3), 2, 32)]


def _boundary(kind, value, as_function=True):
    if kind == "constant":
        return ("constant", value), (A.function(lambda _ix: A.constant(value)) if as_function else A.constant_boundary(value))
    return kind, {"clamp": A.clamp, "mirror": A.mirror, "wrap": A.wrap}[kind]


def _examples(extent):
    return 12 if len(extent) == 1 else (5 if max(extent) <= 5 else 3)


@pytest.mark.parametrize("extent,lo,hi", STENCIL_SHAPES, ids=["x".join(map(str, e)) for e, _, _ in STENCIL_SHAPES])
@pytest.mark.parametrize("dtype", [np.int32, np.float64])
def test_stencil_matches_list_reference(extent, lo, hi, dtype):
    import random
    rnd = random.Random(hash((extent, str(dtype))) & 0xffff)
    for _ in range(_examples(extent)):
        sh = tuple(rnd.randint(lo, min(hi, 96 if len(extent) == 2 else (24 if len(extent) == 3 else hi))) for _ in extent)
        g = np.random.default_rng(rnd.randrange(1 << 30))
        xs = g.integers(-100, 100, size=sh).astype(dtype) if dtype == np.int32 else g.uniform(-1, 1, size=sh)
        cval = dtype(g.integers(-9, 9))
        kind = rnd.choice(["clamp", "mirror", "wrap", "constant"])
        ref_b, acc_b = _boundary(kind, cval.item(), as_function=rnd.random() < 0.7)
        pat = SR.random_pattern(rnd, extent)
        zero = dtype(0)
        want = np.array(SR.stencil_ref(lambda nb: SR.apply_pattern(pat, nb, zero, len(extent)), ref_b, xs.tolist(), sh, extent), dtype=dtype).reshape(sh)
        got = oracle.run(A.stencil(lambda s: SR.apply_pattern(pat, s, A.constant(zero), len(extent)), acc_b, xs, extent=extent))
        if dtype == np.int32:
            assert np.array_equal(got, want), (extent, sh, kind, pat)
        else:
            assert np.allclose(got, want, rtol=1e-12, atol=1e-12), (extent, sh, kind, pat)


@pytest.mark.parametrize("ext1,ext2", [((3,), (5,)), ((3, 3), (3, 3)), ((5, 3), (3, 7)), ((3, 3, 3), (3, 3, 3))])
def test_stencil2_matches_two_list_references(ext1, ext2):
    # stencil2 has no results test in the reference; its definition (Interpreter.hs:652-668) is two
    # stencil accesses with their own boundaries over the intersection of the shapes, which is what
    # two list-based references side by side compute
    import random
    rnd = random.Random(len(ext1) * 131 + sum(ext2))
    for _ in range(5):
        cap = {1: 60, 2: 24, 3: 10}[len(ext1)]
        sh1 = tuple(rnd.randint(max(e // 2 + 1, 2), cap) for e in ext1)
        sh2 = tuple(rnd.randint(max(e // 2 + 1, 2), cap) for e in ext2)
        g = np.random.default_rng(rnd.randrange(1 << 30))
        a, b = g.integers(-50, 50, size=sh1).astype(np.int64), g.integers(-50, 50, size=sh2).astype(np.int64)
        k1, k2 = rnd.choice(["clamp", "mirror", "wrap", "constant"]), rnd.choice(["clamp", "mirror", "wrap", "constant"])
        (r1, b1), (r2, b2) = _boundary(k1, 7), _boundary(k2, -3)
        p1, p2 = SR.random_pattern(rnd, ext1), SR.random_pattern(rnd, ext2)
        d = len(ext1)
        f_ref = lambda s, t: SR.apply_pattern(p1, s, 0, d) * 3 - SR.apply_pattern(p2, t, 0, d)  # noqa: E731
        f_acc = lambda s, t: SR.apply_pattern(p1, s, A.constant(0), d) * 3 - SR.apply_pattern(p2, t, A.constant(0), d)  # noqa: E731
        want = np.array(SR.stencil2_ref(f_ref, r1, a.tolist(), sh1, ext1, r2, b.tolist(), sh2, ext2), dtype=np.int64)
        got = oracle.run(A.stencil2(f_acc, b1, a, b2, b, extent1=ext1, extent2=ext2))
        assert got.shape == tuple(min(x, y) for x, y in zip(sh1, sh2))
        assert np.array_equal(got, want.reshape(got.shape)), (ext1, ext2, sh1, sh2, k1, k2)


# ---- segmented scans against list references (Test/NoFib/Prelude/Scan.hs:263-468, 850-946) --------
def _segments(rnd, total_cap):
    seg = []
    while sum(seg) < total_cap and len(seg) < 12:
        seg.append(rnd.choice([0, 0, 1, 2, 3, 5, 9]))
    return seg


@pytest.mark.parametrize("seed", range(12))
def test_segmented_scans_match_list_references(seed):
    import random
    rnd = random.Random(seed)
    seg = _segments(rnd, rnd.randint(0, 40)) if seed else []
    n = sum(seg)
    rows = rnd.randint(1, 3)
    m = np.random.default_rng(seed).integers(-20, 20, size=(rows, n)).astype(np.int64)
    sg = np.array(seg, np.int64)
    f = lambda a, b: a * 2 + b                                     # noqa: E731  (not commutative: order of operands shows)
    pf = lambda a, b: 2 * a + b                                    # noqa: E731
    z = 3
    parts = lambda row: np.split(row, np.cumsum(seg)[:-1]) if seg else []   # noqa: E731

    def lscan(xs, seeded):
        out, acc = [], (z if seeded else None)
        if seeded:
            out.append(acc)
        for x in xs:
            acc = int(x) if acc is None else pf(acc, int(x))
            out.append(acc)
        return out

    def rscan(xs, seeded):
        out, acc = [], (z if seeded else None)
        if seeded:
            out.append(acc)
        for x in reversed(xs):
            acc = int(x) if acc is None else pf(int(x), acc)
            out.append(acc)
        return out[::-1]

    def rows_of(fn):
        return np.array([sum((fn(list(p)) for p in parts(r)), []) for r in m], np.int64).reshape(rows, -1)
    if n > 0:
        assert np.array_equal(oracle.run(A.scanl1Seg(f, m, sg)), rows_of(lambda p: lscan(p, False)))
        if seg[0] == 0:
            # mkTailFlags (Prelude.hs:1379-1390) puts the flag of a leading empty segment at index -1:
            # the reference's own permute raises its bounds error there, and so does the restatement
            with pytest.raises(oracle.OracleError, match="out of bounds"):
                oracle.run(A.scanr1Seg(f, m, sg))
        else:
            assert np.array_equal(oracle.run(A.scanr1Seg(f, m, sg)), rows_of(lambda p: rscan(p, False)))
    assert np.array_equal(oracle.run(A.scanlSeg(f, z, m, sg)), rows_of(lambda p: lscan(p, True)))
    assert np.array_equal(oracle.run(A.scanrSeg(f, z, m, sg)), rows_of(lambda p: rscan(p, True)))
    body, sums = oracle.run(list(A.scanl_primeSeg(f, z, m, sg)))
    assert np.array_equal(body, rows_of(lambda p: lscan(p, True)[:-1]))
    assert np.array_equal(sums, rows_of(lambda p: lscan(p, True)[-1:]))
    body, sums = oracle.run(list(A.scanr_primeSeg(f, z, m, sg)))
    assert np.array_equal(body, rows_of(lambda p: rscan(p, True)[1:]))
    assert np.array_equal(sums, rows_of(lambda p: rscan(p, True)[:1]))


@settings(max_examples=25, deadline=None)
@given(st.integers(0, 40), st.integers(0, 1 << 30))
def test_issue264_negations(n, seed):
    # Test/NoFib/Issues/Issue264.hs: not.not, not (&&), not (||), their double negations, neg.neg
    g = np.random.default_rng(seed)
    x, y = g.integers(0, 2, n).astype(np.uint8), g.integers(0, 2, n).astype(np.uint8)
    bx, by = x.astype(bool), y.astype(bool)
    nn = lambda f: (lambda u, v: A.lnot(f(u, v)))  # noqa: E731
    assert np.array_equal(oracle.run(A.map(A.lnot, A.map(A.lnot, x))), x)
    assert np.array_equal(oracle.run(A.zipWith(nn(A.and_), x, y)), (~(bx & by)).astype(np.uint8))
    assert np.array_equal(oracle.run(A.zipWith(nn(A.or_), x, y)), (~(bx | by)).astype(np.uint8))
    assert np.array_equal(oracle.run(A.zipWith(lambda u, v: A.lnot(nn(A.and_)(u, v)), x, y)), (bx & by).astype(np.uint8))
    assert np.array_equal(oracle.run(A.zipWith(lambda u, v: A.lnot(nn(A.or_)(u, v)), x, y)), (bx | by).astype(np.uint8))
    for dt in (np.int8, np.int32, np.uint16, np.uint64, np.float32, np.float64):
        v = (g.normal(size=n) * 100).astype(dt)
        assert np.array_equal(oracle.run(A.map(lambda e: -(-e), v)), v)


@settings(max_examples=25, deadline=None)
@given(st.tuples(st.integers(0, 30), st.sampled_from([8, 64, 3, 17])), st.integers(0, 1 << 30))
def test_issue427_indices_of_truth(shape, seed):
    # Test/NoFib/Issues/Issue427.hs:52-83: filter over (row, column, flag) triples, the flag dropped afterwards
    xs = np.random.default_rng(seed).integers(0, 2, size=shape).astype(np.uint8)
    with_inds = A.imap(lambda ix, b: A.tup(ix[0], ix[1], b), xs)
    kept = A.filter_(lambda t: t[2].ne(0), with_inds)[0]
    got = oracle.run(A.map(lambda t: A.tup(t[0], t[1]), kept))
    want = np.argwhere(xs != 0)
    assert np.array_equal(got[0], want[:, 0]) and np.array_equal(got[1], want[:, 1])


def _black_scholes(lib, price, strike, years, one, c):
    """Call and put prices the way Test/NoFib/Spectral/BlackScholes.hs:72-100 writes them; `lib` supplies
    sqrt/log/exp/abs and the choice `where_(cond, a, b)`, `c` turns a Python number into the element type."""
    r, v = c(0.02), c(0.30)
    v_sqrt_t = v * lib.sqrt(years)
    d1 = (lib.log(price / strike) + (r + c(0.5) * v * v) * years) / v_sqrt_t
    d2 = d1 - v_sqrt_t

    def cnd(d):
        k = one / (one + c(0.2316419) * lib.abs(d))
        coeff = [0.31938153, -0.356563782, 1.781477937, -1.821255978, 1.330274429]
        acc = c(coeff[-1])
        for a in coeff[-2::-1]:                      # horner: x * foldr1 (\a b -> a + x*b) coeff
            acc = c(a) + k * acc
        p = c(0.39894228040143267793994605993438) * lib.exp(c(-0.5) * d * d) * (k * acc)
        return lib.where_(d > 0, one - p, p)
    n1, n2 = cnd(d1), cnd(d2)
    x_exp_rt = strike * lib.exp(-r * years)
    return price * n1 - x_exp_rt * n2, x_exp_rt * (one - n2) - price * (one - n1)


class _NumpyLib:
    sqrt, log, exp, abs = np.sqrt, np.log, np.exp, np.abs
    where_ = staticmethod(np.where)


class _AccLib:
    sqrt, log, exp = A.sqrt, A.log, A.exp
    abs = staticmethod(abs)
    where_ = staticmethod(A.cond)


@settings(max_examples=10, deadline=None)
@given(st.integers(0, 300), st.sampled_from(["f32", "f64"]), st.integers(0, 1 << 30))
def test_black_scholes_matches_numpy(n, ty, seed):
    dt = A.NP_OF[ty]
    g = np.random.default_rng(seed)
    price, strike, years = (g.uniform(5, 30, n).astype(dt), g.uniform(1, 100, n).astype(dt), g.uniform(0.25, 10, n).astype(dt))
    psy = A.use((price, strike, years))
    got = oracle.run(A.map(lambda t: A.tup(*_black_scholes(_AccLib, t[0], t[1], t[2], A.constant(dt(1)), lambda x: A.constant(dt(x)))), psy))
    want = _black_scholes(_NumpyLib, price, strike, years, dt(1), dt)
    for gv, wv in zip(got, want):                    # Test/Similar.hs:90-93: Float 5e-5 / 5e-3, Double 5e-9 / 5e-7
        tol = (5e-5, 5e-3) if ty == "f32" else (5e-9, 5e-7)
        assert np.all((np.abs(gv - wv) <= tol[0]) | (np.abs(gv - wv) <= tol[1] * np.maximum(np.abs(gv), np.abs(wv))))


@settings(max_examples=15, deadline=None)
@given(st.integers(0, 400), st.integers(0, 1 << 30))
def test_saxpy_and_sasum_match_numpy(n, seed):
    # Test/NoFib/Imaginary/SAXPY.hs:77-81 (zipWith (\x y -> alpha * x + y)) and SASUM.hs:74-78 (fold (+) 0 . map abs)
    g = np.random.default_rng(seed)
    x, y = g.normal(size=n).astype(np.float32), g.normal(size=n).astype(np.float32)
    alpha = np.float32(g.normal())
    assert np.array_equal(oracle.run(A.zipWith(lambda u, v: A.constant(alpha) * u + v, x, y)), alpha * x + y)
    acc = np.float32(0)
    for v in np.abs(x):
        acc = np.float32(acc + v)
    assert oracle.run(A.fold(add, np.float32(0), A.map(abs, x))) == acc
    xi = g.integers(-1000, 1000, n).astype(np.int32)
    assert oracle.run(A.fold(add, np.int32(0), A.map(abs, xi))) == np.abs(xi).sum(dtype=np.int32)


@settings(max_examples=30, deadline=None)
@given(st.integers(1, 3), st.sampled_from(["i8", "i32", "u16", "u64", "f16", "f32", "f64"]), st.integers(0, 1 << 30))
def test_filter_matches_list_reference(rank, ty, seed):
    # Test/NoFib/Prelude/Filter.hs:96-124: `filter even` on integral and `filter (> 0)` on floating elements,
    # ranks 1 to 3: the kept elements in row-major order, and how many every innermost row kept
    g = np.random.default_rng(seed)
    shape = tuple(int(d) for d in g.integers(0, 9, size=rank))
    dt = A.NP_OF[ty]
    if np.issubdtype(dt, np.integer):
        xs = g.integers(0, 100, size=shape).astype(dt)
        keep, pred = xs % 2 == 0, (lambda v: (v % 2).eq(0))
    else:
        xs = g.normal(size=shape).astype(dt)
        keep, pred = xs > 0, (lambda v: v > 0)
    vals, counts = oracle.run(list(A.filter_(pred, xs)))
    assert np.array_equal(vals, xs[keep]) and vals.dtype == dt
    assert np.array_equal(counts, keep.sum(axis=-1)) and counts.shape == shape[:-1]


def _shape(g, rank, lo):
    return tuple(int(d) for d in g.integers(lo, 6, size=rank))


@settings(max_examples=40, deadline=None)
@given(st.integers(1, 3), st.integers(1, 3), st.integers(0, 1 << 30))
def test_gather_scatter_accumulate_between_ranks(rank, rank2, seed):
    # Test/NoFib/Prelude/Backpermute.hs:131-153 (gather->DIMn) and Permute.hs:96-160 (scatter->DIMn with
    # unique or absent targets, accumulate->DIMn with Maybe targets): arrays of indices of another rank
    g = np.random.default_rng(seed)
    sh, sh2 = _shape(g, rank, 1), _shape(g, rank2, 0)
    xs = g.integers(-50, 50, size=sh).astype(np.int64)
    # gather: an array of shape sh2 of indices into xs
    lin = g.integers(0, xs.size, size=sh2)
    ixs = tuple(np.ascontiguousarray(c).astype(np.int64) for c in np.unravel_index(lin, sh))
    iu = A.use(ixs)
    got = oracle.run(A.backpermute(iu.shape, lambda j: iu[j], xs))
    assert np.array_equal(got, xs.reshape(-1)[lin])
    # scatter / accumulate: an array of shape sh of Maybe indices into a target of shape sh3 (not empty)
    sh3 = _shape(g, rank2, 1)
    n3 = int(np.prod(sh3))
    tgt = g.integers(0, n3, size=sh)
    absent = g.random(sh) < 0.4
    comps = tuple(np.ascontiguousarray(c).astype(np.int64) for c in np.unravel_index(tgt, sh3))
    mu = A.use((np.where(absent, 0, 1).astype(np.uint8),) + comps)
    dest = lambda j: A.let_(mu[j], lambda m: A.tup(m[0], A.index(*[m[1 + d] for d in range(rank2)])))  # noqa: E731
    want = np.zeros(n3, np.int64)
    np.add.at(want, tgt[~absent], xs[~absent])
    got = oracle.run(A.permute(add, A.fill(A.index(*sh3), A.constant(0)), dest, xs))
    assert np.array_equal(got, want.reshape(sh3))
    # `permute const` where no two sources share a target (the reference draws them that way)
    first = np.zeros(tgt.shape, bool)
    seen = set()
    for pos in np.ndindex(*sh):
        if not absent[pos] and int(tgt[pos]) not in seen:
            seen.add(int(tgt[pos]))
            first[pos] = True
    mu2 = A.use((first.astype(np.uint8),) + comps)
    dest2 = lambda j: A.let_(mu2[j], lambda m: A.tup(m[0], A.index(*[m[1 + d] for d in range(rank2)])))  # noqa: E731
    defaults = g.integers(-9, 9, size=sh3).astype(np.int64)
    want2 = defaults.reshape(-1).copy()
    want2[tgt[first]] = xs[first]
    got = oracle.run(A.permute(lambda new, old: new, defaults, dest2, xs))
    assert np.array_equal(got, want2.reshape(sh3))
