"""GPU parity: every skeleton against the CPU oracle on the same seeded inputs.

Sizes, element types and the monoids follow the reference's nofib suite
(Test/NoFib/Prelude/{Fold,Scan,Permute,Stencil}.hs); edge sizes cover tile and
warp boundaries of the kernels.  Integers must match bit for bit; floating-point
reductions use the reference's own tolerance (Test/Similar.hs:90-91,
absRelTol 0.00005 0.005 for Float) or the tighter one stated in the test."""
import numpy as np
import pytest

import accelerate_b200 as A
from accelerate_b200.backend import run as backend_run
from tests.util import check

pytestmark = pytest.mark.gpu
add = lambda a, b: a + b  # noqa: E731
SIZES_1D = [0, 1, 2, 31, 32, 33, 127, 128, 129, 255, 256, 257, 1023, 1024, 1025, 4095, 4096, 4097, 8193, 50001]
rng = np.random.default_rng(42)
F32_TOL = dict(rtol=5e-3, atol=5e-5)   # Test/Similar.hs:90-91


def ints(n, dtype=np.int32, lo=-1000, hi=1000):
    return rng.integers(lo, hi, size=n).astype(dtype)


def floats(n, dtype=np.float32):
    return rng.uniform(-1, 1, size=n).astype(dtype)


# ---- elementwise ----------------------------------------------------------------
@pytest.mark.parametrize("n", [0, 1, 3, 4, 5, 1000, 4099])
def test_map_zipwith(n):
    x, y = floats(n), floats(n)
    check(A.zipWith(lambda a, b: a * b + 1.5, x, y))
    check(A.map(lambda a: A.cond(a > 0.0, A.sqrt(a), -a), x), rtol=1e-6)
    check(A.zipWith(lambda a, b: A.tup(a + b, a.ne(b)), ints(n), ints(n)))


def test_zipwith_intersect_2d():
    a, b = ints((7, 12)), ints((5, 16))
    check(A.zipWith(add, a, b))
    check(A.zipWith(add, ints((8, 16)), ints((8, 16))))


def test_backpermute_transpose():
    m = ints((13, 21))
    mu = A.use(m)
    check(A.backpermute(A.index(21, 13), lambda ix: A.index(ix[1], ix[0]), mu))


def test_generate_index_math():
    check(A.generate(A.index(5, 7), lambda ix: ix[0] * 100 + ix[1]))
    check(A.generate(A.index(3, 4, 6), lambda ix: A.to_index(A.index(3, 4, 6), ix) % 5))


@pytest.mark.parametrize("ty", ["i8", "i16", "i32", "i64", "u8", "u16", "u32", "u64"])
def test_integer_primitives(ty):
    dt = A.NP_OF[ty]
    info = np.iinfo(dt)
    x = rng.integers(info.min, info.max, size=257, dtype=dt, endpoint=True)
    y = rng.integers(info.min, info.max, size=257, dtype=dt, endpoint=True)
    y[y == 0] = 3
    sh = rng.integers(0, 70, size=257).astype(np.int64)
    xs, ys, ss = A.use(x), A.use(y), A.use(sh)

    def f(ix):
        a, b, s = xs[ix], ys[ix], ss[ix]
        return A.tup(a + b, a - b, a * b, -a, abs(a), A.signum(a), A.quot(a, b), A.rem(a, b), a // b, a % b,
                     a & b, a | b, a ^ b, ~a, a << s, a >> s, A.rotate_l(a, s), A.rotate_r(a, s),
                     A.pop_count(a), A.count_leading_zeros(a), A.count_trailing_zeros(a),
                     A.max_(a, b), A.min_(a, b), a < b, a >= b, a.eq(b),
                     A.from_integral(a, "i64"), A.from_integral(a, "u8"), A.from_integral(a, "f32"), A.from_integral(a, "f64"))
    check(A.generate(A.index(257), f))


@pytest.mark.parametrize("ty", ["f32", "f64"])
def test_float_primitives_exact(ty):
    dt = A.NP_OF[ty]
    x = (rng.normal(size=300) * 50).astype(dt)
    y = (rng.normal(size=300) * 3).astype(dt)
    x[:6] = [0.5, 1.5, 2.5, -0.5, -1.5, -2.5]
    xs, ys = A.use(x), A.use(y)

    def f(ix):
        a, b = xs[ix], ys[ix]
        return A.tup(a + b, a - b, a * b, a / b, -a, abs(a), A.signum(a), A.recip(b), A.sqrt(abs(a)),
                     A.truncate(a), A.round_(a), A.floor(a), A.ceiling(a), A.round_(a, "i32"),
                     A.max_(a, b), A.min_(a, b), a < b, a.eq(b), A.is_nan(a / a),
                     A.to_floating(a, "f64"), A.to_floating(a, "f32"), A.bitcast(a, "u32" if ty == "f32" else "u64"))
    check(A.generate(A.index(300), f))


def test_float_transcendentals():
    x = rng.uniform(0.1, 3.0, size=500).astype(np.float32)
    xs = A.use(x)
    check(A.generate(A.index(500), lambda ix: A.tup(A.sin(xs[ix]), A.cos(xs[ix]), A.exp(xs[ix]), A.log(xs[ix]), A.tanh(xs[ix]),
                                                     xs[ix] ** 1.5, A.atan2(xs[ix], 2.0), A.log_base(2.0, xs[ix]))), rtol=4e-7 * 8)


def test_while_loop():
    # collatz step count
    x = rng.integers(1, 1000, size=200).astype(np.int64)
    xs = A.use(x)

    def f(ix):
        st = A.while_(lambda s: s[0] > 1, lambda s: A.tup(A.cond((s[0] % 2).eq(0), s[0] // 2, 3 * s[0] + 1), s[1] + 1),
                      A.tup(xs[ix], A.constant(0)))
        return st[1]
    check(A.generate(A.index(200), f))


# ---- fold -------------------------------------------------------------------------
@pytest.mark.parametrize("n", SIZES_1D)
def test_fold_sum_int(n):
    check(A.fold(add, 0, ints(n)))
    check(A.fold(add, 42, ints(n, np.int64)))          # non-neutral seed (Fold.hs:55-60)


@pytest.mark.parametrize("n", SIZES_1D[1:])
def test_fold1_minmax(n):
    check(A.fold1(A.max_, ints(n)))
    check(A.fold1(A.min_, floats(n)))


@pytest.mark.parametrize("n", [1, 100, 4096, 100003, 1 << 20])
def test_dotp(n):
    # Test/NoFib/Imaginary/DotP.hs:75-82
    x, y = floats(n), floats(n)
    check(A.fold(add, 0.0, A.zipWith(lambda a, b: a * b, x, y)), rtol=1e-4, atol=1e-4)


def test_dotp_config0():
    g = np.random.default_rng(42)
    x = g.uniform(-1, 1, 1 << 20).astype(np.float32)
    y = g.uniform(-1, 1, 1 << 20).astype(np.float32)
    got = check(A.fold(add, 0.0, A.zipWith(lambda a, b: a * b, x, y)), rtol=1e-4, atol=1e-4)
    assert abs(float(got) - float(np.dot(x.astype(np.float64), y.astype(np.float64)))) < 1e-4 * 600


@pytest.mark.parametrize("shape", [(1, 1), (3, 5), (16, 64), (7, 129), (50, 1000), (5, 4096), (2, 3, 33), (4, 0), (0, 7), (300, 4), (3, 70000)])
def test_fold_rows(shape):
    m = ints(shape)
    check(A.fold(add, 7, m))
    if shape[-1] > 0:
        check(A.fold1(A.max_, floats(shape)))


def _mss(a, b):
    # maximum segment sum monoid: non-commutative (Test/NoFib/Prelude/Fold.hs:287-309)
    return A.tup(A.max_(a[0], A.max_(b[0], a[2] + b[1])), A.max_(a[1], a[3] + b[1]), A.max_(b[2], a[2] + b[3]), a[3] + b[3])


@pytest.mark.parametrize("n", [1, 2, 33, 129, 1025, 4097, 20000])
def test_fold_non_commutative(n):
    x = ints(n, np.int64, -50, 50)
    xs = A.map(lambda v: A.tup(A.max_(v, 0), A.max_(v, 0), A.max_(v, 0), v), x)
    check(A.fold1(_mss, xs))
    check(A.fold(_mss, A.tup(0, 0, 0, 0), xs))
    m = ints((9, n // 3 + 1), np.int64, -50, 50)
    check(A.fold1(_mss, A.map(lambda v: A.tup(A.max_(v, 0), A.max_(v, 0), A.max_(v, 0), v), m)))


def test_fold_empty_error():
    from accelerate_b200.backend import B200Error
    with pytest.raises(B200Error):
        A.backend.run(A.fold1(add, ints(0)))


# ---- foldSeg -----------------------------------------------------------------------
@pytest.mark.parametrize("nseg,maxlen", [(1, 5), (7, 0), (64, 128), (300, 40), (50, 3000)])
def test_foldseg(nseg, maxlen):
    lens = rng.integers(0, maxlen + 1, size=nseg).astype(np.int32)
    n = int(lens.sum())
    x = ints(n)
    check(A.foldSeg(add, 0, x, lens))
    lens1 = np.maximum(lens, 1)
    x1 = ints(int(lens1.sum()))
    check(A.fold1Seg(add, x1, lens1))
    check(A.fold1Seg(A.max_, floats(int(lens1.sum())), lens1.astype(np.int64)))


def test_foldseg_2d_and_noncommutative():
    lens = np.array([3, 0, 5, 1, 7], np.int64)
    m = ints((6, 16), np.int64, -50, 50)
    check(A.foldSeg(add, 0, m, lens))
    xs = A.map(lambda v: A.tup(A.max_(v, 0), A.max_(v, 0), A.max_(v, 0), v), m)
    check(A.foldSeg(_mss, A.tup(0, 0, 0, 0), xs, lens))


def test_fold1seg_empty_segment_error():
    from accelerate_b200.backend import B200Error
    with pytest.raises(B200Error):
        A.backend.run(A.fold1Seg(add, ints(8), np.array([3, 0, 5], np.int32)))


# ---- scans -------------------------------------------------------------------------
SCAN_SIZES = [0, 1, 2, 3, 4, 5, 64, 65, 127, 128, 129, 511, 512, 513, 4095, 4096, 4097, 8192, 12289, 50001]


@pytest.fixture(params=["auto", "long-row-kernels"])
def scan_path(request, monkeypatch):
    """Short rows are scanned with small tiles; the second pass forces the kernels that long rows
    use (the shared-memory ring, 8192-element tiles) onto the same cases."""
    if request.param == "long-row-kernels":
        monkeypatch.setenv("ACCELERATE_B200_SCAN_NO_SMALL", "1")
    return request.param


@pytest.mark.parametrize("n", SCAN_SIZES)
def test_scans_int(n, scan_path):
    x = ints(n, np.int32, 0, 100)
    if n > 0:
        check(A.scanl1(add, x))
        check(A.scanr1(add, x))
    check(A.scanl(add, 10, x))
    check(A.scanr(add, 10, x))
    check(list(A.scanl_prime(add, 10, x)))
    check(list(A.scanr_prime(add, 10, x)))


@pytest.mark.parametrize("n", [1, 1000, 4096, 70000])
def test_scans_float_and_i64(n, scan_path):
    f = rng.uniform(0, 1, n).astype(np.float32)
    tol = dict(rtol=1e-5 * np.sqrt(n), atol=1e-5 * np.sqrt(n))
    check(list(A.scanl_prime(add, 0.0, f)), **tol)
    check(A.scanl1(add, f), **tol)
    big = rng.integers(np.iinfo(np.int64).min, np.iinfo(np.int64).max, size=n, dtype=np.int64)
    check(A.scanr1(A.max_, big))
    check(A.scanl1(A.min_, big))


def _interval(a, b):
    # non-commutative "interval" monoid (Test/NoFib/Prelude/Scan.hs:745-771)
    return A.tup(a[0], b[1])


@pytest.mark.parametrize("n", [1, 5, 129, 4097, 9000])
def test_scans_non_commutative(n, scan_path):
    x = ints(n, np.int64)
    pairs = A.map(lambda v: A.tup(v, v + 1), x)
    check(A.scanl1(_interval, pairs))
    check(A.scanr1(_interval, pairs))
    check(A.scanl(_interval, A.tup(-1, -2), pairs))
    check(A.scanr(_interval, A.tup(-1, -2), pairs))
    check(list(A.scanl_prime(_interval, A.tup(-1, -2), pairs)))
    check(list(A.scanr_prime(_interval, A.tup(-1, -2), pairs)))
    m = A.map(lambda v: A.tup(A.max_(v, 0), A.max_(v, 0), A.max_(v, 0), v), x)
    check(A.scanl1(_mss, m))
    check(A.scanr1(_mss, m))


@pytest.mark.parametrize("shape", [(1, 1), (3, 5), (31, 257), (4, 4096), (3, 4100), (2, 3, 9), (5, 0), (0, 5), (257, 31)])
def test_scans_rows(shape, scan_path):
    m = ints(shape, np.int32, 0, 100)
    if shape[-1] > 0:
        check(A.scanl1(add, m))
        check(A.scanr1(add, m))
    check(A.scanl(add, 1, m))
    check(A.scanr(add, 1, m))
    check(list(A.scanl_prime(add, 1, m)))
    check(list(A.scanr_prime(add, 1, m)))


def test_scan_wraps_int32(scan_path):
    x = np.full(5000, 2_000_000_000, np.int32)
    check(A.scanl1(add, x))


@pytest.mark.parametrize("ty", ["i8", "u8", "i16", "u16"])
@pytest.mark.parametrize("shape", [(40000,), (16384 + 16,), (3, 16400), (3, 16396), (1, 8196), (2, 8196)])
def test_scans_narrow_types_on_both_kernels(ty, shape, monkeypatch):
    # Long rows of 1- and 2-byte elements: shapes whose row pitch is a multiple of 16 bytes take the
    # shared-memory ring (bulk copies), the others must fall back to the register kernel.
    monkeypatch.setenv("ACCELERATE_B200_SCAN_NO_SMALL", "1")
    dt = A.NP_OF[ty]
    m = rng.integers(0, 3, size=shape).astype(dt)
    check(A.scanl1(add, m))
    check(A.scanr1(add, m))
    check(A.scanr(A.max_, 1, m))
    check(list(A.scanl_prime(add, 1, m)))


def test_scan_descriptor_layouts_do_not_leak_into_each_other():
    # All scans of a context share one scratch buffer of look-back descriptors, told apart by an
    # epoch tag.  Packed 8-byte descriptors, packed 16-byte descriptors and the status/value arrays
    # of tuple scans lay the buffer out differently, so a scan must not take value bits a previous
    # scan left behind for a status word of its own epoch.  The first scan leaves the tile prefixes
    # 1, 2, 3, ... (every small status value among them) in the buffer.
    from accelerate_b200 import backend, language as L
    ctx = backend.Context(0)
    try:
        def run(build, *hosts):
            L.reset_names()
            ps = [L.param(h[0].ndim if isinstance(h, tuple) else h.ndim,
                          tuple(L.TY_OF_NP[x.dtype] for x in h) if isinstance(h, tuple) else L.TY_OF_NP[h.dtype]) for h in hosts]
            prog = A.build_program(build(*ps))
            outs = ctx.execute(prog.text, [ctx.from_host(h) for h in hosts], len(prog.outputs))
            return [o.download() for o in outs]
        tiles = 700
        x = np.zeros(tiles * 8192, np.int32)
        x[::8192] = 1                                            # one per tile: tile prefixes 1..700
        for _ in range(3):
            got, = run(lambda a: A.scanl1(add, a), x)
            assert np.array_equal(got, np.cumsum(x, dtype=np.int32))
            n = 3_000_000
            a, b = ints(n, np.int64), ints(n, np.int64)
            got, = run(lambda p: A.scanl1(_interval, p), (a, b))     # tuple scan: u32 status array
            assert np.array_equal(got[0], np.full(n, a[0])) and np.array_equal(got[1], b)
            big = rng.integers(-1 << 40, 1 << 40, size=2_500_000, dtype=np.int64)
            got, = run(lambda p: A.scanr1(A.max_, p), big)           # 16-byte descriptors
            assert np.array_equal(got, np.maximum.accumulate(big[::-1])[::-1])
            small = ints(70000, np.int32, 0, 3)
            got, = run(lambda p: A.scanl1(add, p), small)            # short rows: small tiles, dense descriptors
            assert np.array_equal(got, np.cumsum(small, dtype=np.int32))
    finally:
        ctx.close()


# ---- errors the reference raises from scalar code ------------------------------------------
def test_integer_division_by_zero_is_reported():
    # quot/rem/div/mod by zero throw DivideByZero in the reference (Interpreter.hs:1328-1344)
    from accelerate_b200.backend import B200Error
    x = ints(1000, np.int32, 1, 50)
    y = x.copy()
    y[777] = 0
    for f in (lambda a, b: a // b, lambda a, b: a % b, lambda a, b: A.quot(a, b), lambda a, b: A.rem(a, b)):
        with pytest.raises(B200Error) as e:
            backend_run(A.zipWith(f, x, y))
        assert e.value.code == 9, e.value
        check(A.zipWith(f, x, x))                                 # the context keeps working
    # a division the scalar code never reaches raises nothing
    check(A.zipWith(lambda a, b: A.cond(b.eq(0), a, a // b), x, y))


def test_permute_target_out_of_bounds_is_reported():
    # toIndex checks every component of the target index (Shape.hs:102-106)
    from accelerate_b200.backend import B200Error
    src = ints(64, np.int32)
    with pytest.raises(B200Error) as e:
        backend_run(A.permute(add, A.fill(10, A.constant(np.int32(0))), lambda ix: A.Just_(A.index(ix[0] % 11)), src))
    assert e.value.code == 5 and "out of bounds" in str(e.value)
    with pytest.raises(B200Error) as e:
        backend_run(A.permute(add, A.fill(A.index(4, 4), A.constant(np.int32(0))), lambda ix: A.Just_(A.index(ix[0] % 4, 1 + ix[0] % 4)), src))
    assert e.value.code == 5                                       # (r, 4) is a valid linear offset but not a valid index
    check(A.permute(add, A.fill(A.index(4, 4), A.constant(np.int32(0))), lambda ix: A.Just_(A.index(ix[0] % 4, ix[0] % 3)), src))


# ---- permute -----------------------------------------------------------------------
@pytest.mark.parametrize("n,bins", [(0, 4), (1, 1), (20, 10), (5000, 37), (100000, 1000), (200000, 70000)])
def test_histogram(n, bins):
    keys = rng.integers(0, bins, size=n).astype(np.int32)
    k = A.use(keys)
    check(A.permute(add, A.fill(bins, A.constant(np.int32(0))), lambda ix: A.Just_(A.index(A.from_integral(k[ix], "i64"))),
                    A.fill(k.shape, A.constant(np.int32(1)))))


@pytest.mark.parametrize("bins", [70001, 65536, 100000])
@pytest.mark.parametrize("vals", ["ones", "mixed"])
def test_permute_add_int32_large_target_packed_fields(bins, vals):
    # (+) into an Int32 target of 51 201 .. 114 688 elements: every element is private to the CTA, the
    # leading ones as 32-bit words, the others as 16-bit fields whose wraps are compensated.  Neighbouring
    # elements of the second kind receive most of the updates (so their fields wrap many times, lower
    # ones carrying into upper ones), the addends include values above 16 bits and negative ones, and
    # the last element of an odd-sized target is hit too.
    n = 3_000_000
    g = np.random.default_rng(bins)
    keys = g.integers(0, bins, size=n).astype(np.int32)
    hot = g.random(n)
    # four neighbouring elements near the end (16-bit fields of both parities), the last element, and one
    # element near the start (which has a 32-bit word of its own)
    for k, (lo, hi) in enumerate([(0.0, 0.15), (0.15, 0.30), (0.30, 0.42), (0.42, 0.55)]):
        keys[(hot >= lo) & (hot < hi)] = bins - 6 + k
    keys[(hot >= 0.55) & (hot < 0.60)] = bins - 1
    keys[(hot >= 0.60) & (hot < 0.70)] = 12344
    if vals == "ones":
        v = np.ones(n, np.int32)
    else:
        v = g.choice(np.array([1, 65535, 70000, -3, 2_000_000_000, 0], np.int32), size=n)
    want = np.zeros(bins, np.int64)
    np.add.at(want, keys, v.astype(np.int64))
    ku = A.use(keys)
    got = backend_run(A.permute(add, A.fill(bins, A.constant(np.int32(5))), lambda ix: A.Just_(A.index(A.from_integral(ku[ix], "i64"))), v))
    assert np.array_equal(got, (want + 5).astype(np.int32))


def test_permute_float_dropped():
    n, bins = 100000, 1 << 10
    keys = rng.integers(0, 1 << 30, size=n).astype(np.int32)
    drop = (rng.uniform(size=n) < 0.1).astype(np.uint8)
    vals = rng.uniform(0, 1, n).astype(np.float32)
    k, d = A.use(keys), A.use(drop)
    acc = A.permute(add, A.fill(bins, A.constant(np.float32(0))),
                    lambda ix: A.cond(d[ix].ne(0), A.Nothing_(1), A.Just_(A.index(A.from_integral(k[ix], "i64") % bins))), vals)
    check(acc, rtol=1e-5 * np.sqrt(n / bins), atol=1e-5 * np.sqrt(n / bins))


def test_permute_minmax_cas_and_scatter():
    n, bins = 20000, 97
    keys = rng.integers(0, bins, size=n).astype(np.int64)
    k = A.use(keys)
    p = lambda ix: A.Just_(A.index(k[ix]))  # noqa: E731
    check(A.permute(A.max_, A.fill(bins, A.constant(np.int32(-5))), p, ints(n)))
    check(A.permute(A.min_, A.fill(bins, A.constant(np.int64(5))), p, ints(n, np.int64)))
    check(A.permute(A.min_, A.fill(bins, A.constant(np.float32(5))), p, floats(n)))          # CAS loop
    check(A.permute(lambda a, b: a * b, A.fill(bins, A.constant(np.int64(1))), p, ints(n, np.int64, 1, 4)))  # CAS loop
    check(A.permute(lambda a, b: a | b, A.fill(bins, A.constant(np.uint32(0))), p, ints(n, np.uint32, 0, 1 << 20)))
    perm = rng.permutation(n).astype(np.int64)
    pu = A.use(perm)
    check(A.permute(lambda a, b: a, A.fill(n, A.constant(np.float32(0))), lambda ix: A.Just_(A.index(pu[ix])), floats(n)))


def test_permute_tuple_lock_and_small_types():
    n, bins = 5000, 13
    keys = rng.integers(0, bins, size=n).astype(np.int64)
    k = A.use(keys)
    p = lambda ix: A.Just_(A.index(k[ix]))  # noqa: E731
    src = A.zip(ints(n, np.int64), ints(n, np.int32, 0, 9))
    f = lambda a, b: A.tup(a[0] + b[0], A.max_(a[1], b[1]))  # noqa: E731
    check(A.permute(f, A.zip(A.fill(bins, A.constant(0)), A.fill(bins, A.constant(np.int32(0)))), p, src))
    check(A.permute(add, A.fill(bins, A.constant(np.int16(0))), p, ints(n, np.int16, -3, 3)))


def test_permute_2d_to_2d():
    m = ints((17, 23), np.int32, 0, 5)
    mu = A.use(m)
    acc = A.permute(add, A.fill(A.index(5, 5), A.constant(np.int32(0))),
                    lambda ix: A.cond((ix[0] + ix[1]) % 3 == 0 if False else ((ix[0] + ix[1]) % 3).eq(0), A.Nothing_(2),
                                      A.Just_(A.index(A.from_integral(mu[ix], "i64"), ix[1] % 5))), mu)
    check(acc)


# ---- stencils ------------------------------------------------------------------------
BOUNDARIES = [A.clamp, A.mirror, A.wrap, A.function(lambda ix: A.constant(np.float32(0.25))), A.constant_boundary(np.float32(-2.0))]


@pytest.mark.parametrize("bnd", range(5))
@pytest.mark.parametrize("shape", [(5, 6), (32, 128), (33, 129), (70, 300), (9, 9)])
def test_stencil_2d_3x3(shape, bnd):
    m = rng.uniform(0, 1, shape).astype(np.float32)
    check(A.stencil(lambda s: 0.25 * (s[0][1] + s[2][1] + s[1][0] + s[1][2]), BOUNDARIES[bnd], m))
    check(A.stencil(lambda s: sum((s[i][j] * float(i * 3 + j + 1) for i in range(3) for j in range(3)), A.constant(np.float32(0))), BOUNDARIES[bnd], m))


@pytest.mark.parametrize("ext", [3, 5, 7, 9])
def test_stencil_1d(ext):
    x = rng.uniform(0, 1, 5000).astype(np.float32)
    for b in BOUNDARIES[:3]:
        check(A.stencil(lambda s: sum((s[i] * float(i + 1) for i in range(ext)), A.constant(np.float32(0))), b, x, extent=(ext,)))


@pytest.mark.parametrize("ext", [5, 7, 9])
def test_stencil_2d_large_patterns(ext):
    m = ints((40, 140), np.int32, 0, 10)
    for b in BOUNDARIES[:3]:
        check(A.stencil(lambda s: sum((s[i][j] * (i * ext + j) for i in range(ext) for j in range(ext)), A.constant(np.int32(0))), b, m,
                        extent=(ext, ext)))


def test_stencil_3d():
    v = rng.uniform(0, 1, (9, 11, 70)).astype(np.float32)
    for b in BOUNDARIES[:3]:
        check(A.stencil(lambda s: s[0][1][1] + s[2][1][1] + s[1][0][1] + s[1][2][1] + s[1][1][0] + s[1][1][2] - 6.0 * s[1][1][1], b, v))


def test_stencil2_gaussian_mirror():
    a = rng.uniform(0, 1, (37, 133)).astype(np.float32)
    b = rng.uniform(0, 1, (35, 140)).astype(np.float32)
    w = [[1, 2, 1], [2, 4, 2], [1, 2, 1]]
    f = lambda s, t: sum((np.float32(w[i][j] / 16.0) * (s[i][j] + t[i][j]) for i in range(3) for j in range(3)), A.constant(np.float32(0)))  # noqa: E731
    check(A.stencil2(f, A.mirror, a, A.mirror, b))


@pytest.mark.parametrize("case", ["stencil2_f32", "stencil2_ragged", "f64_3x3", "zipped_5x5", "f32_odd_width", "i64_wrap_7x3"])
def test_stencil_2d_rows_staged_through_shared_memory(case):
    # arrays wide and tall enough for the kernel that stages input rows in shared memory (at least 8 bytes per
    # point over all inputs, 244 columns, 64 rows besides the halo); the frame around its part comes from the
    # register-window kernel, so every boundary kind is exercised along the seams too
    w = [[1, 2, 1], [2, 4, 2], [1, 2, 1]]
    g2 = lambda s, t: sum((np.float32(w[i][j] / 16.0) * (s[i][j] + t[i][j]) for i in range(3) for j in range(3)), A.constant(np.float32(0)))  # noqa: E731
    if case == "stencil2_f32":
        a = rng.uniform(0, 1, (200, 488)).astype(np.float32)
        b = rng.uniform(0, 1, (200, 488)).astype(np.float32)
        for bnd in BOUNDARIES[:3]:
            check(A.stencil2(g2, bnd, a, A.mirror, b))
    elif case == "stencil2_ragged":
        a = rng.uniform(0, 1, (150, 500)).astype(np.float32)
        b = rng.uniform(0, 1, (131, 488)).astype(np.float32)
        check(A.stencil2(g2, A.clamp, a, A.wrap, b))
        check(A.stencil2(g2, A.function(lambda ix: A.constant(np.float32(7.5))), a, A.clamp, b))
    elif case == "f64_3x3":
        m = rng.uniform(0, 1, (130, 400))
        for bnd in BOUNDARIES[:3]:
            check(A.stencil(lambda s: sum((s[i][j] * float(i * 3 + j + 1) for i in range(3) for j in range(3)), A.constant(np.float64(0))), bnd, m))
    elif case == "zipped_5x5":
        x = rng.uniform(0, 1, (150, 372)).astype(np.float32)
        y = rng.uniform(0, 1, (150, 372)).astype(np.float32)
        z = A.zipWith(lambda u, v: u * 2.0 + v, x, y)
        check(A.stencil(lambda s: sum((s[i][j] * float(i * 5 + j) for i in range(5) for j in range(5)), A.constant(np.float32(0))), A.wrap, z,
                        extent=(5, 5)))
    elif case == "f32_odd_width":
        a = rng.uniform(0, 1, (100, 487)).astype(np.float32)       # rows that are no multiple of four elements: not staged
        check(A.stencil2(g2, A.mirror, a, A.mirror, a))
    else:
        m = ints((140, 368), np.int64, -1000, 1000)
        check(A.stencil(lambda s: sum((s[i][j] * (i * 3 + j) for i in range(7) for j in range(3)), A.constant(np.int64(0))), A.wrap, m, extent=(7, 3)))


def test_stencil_delayed_input_and_jacobi_iterated():
    m = rng.uniform(0, 1, (50, 200)).astype(np.float32)
    jac = lambda s: 0.25 * (s[0][1] + s[2][1] + s[1][0] + s[1][2])  # noqa: E731
    acc = A.map(lambda v: v * 2.0, m)
    for _ in range(5):
        acc = A.stencil(jac, A.clamp, acc)
    check(acc)


# ---- composition ----------------------------------------------------------------------
def test_smvm_like_pipeline():
    # SMVM (Test/NoFib/Spectral/SMVM.hs:77-85): foldSeg over gathered products
    nrows, ncols = 200, 300
    lens = rng.integers(0, 12, nrows).astype(np.int32)
    nnz = int(lens.sum())
    cols = rng.integers(0, ncols, nnz).astype(np.int32)
    vals = floats(nnz)
    vec = floats(ncols)
    v = A.use(vec)
    prods = A.zipWith(lambda i, x: x * v[A.index(A.from_integral(i, "i64"))], cols, vals)
    check(A.foldSeg(add, 0.0, prods, lens), **F32_TOL)


def test_reshape_and_unit():
    x = ints(24)
    check(A.fold(add, 0, A.reshape(A.index(4, 6), x)))
    s = A.fold(add, 0, x)
    check(A.map(lambda v: v + A.the(s), x))


def test_adopt_host_uploads_on_first_use(gpu_ctx):
    # lazy transfer (b200_array_adopt_host): nothing is copied until the array is used
    from accelerate_b200 import language as L
    x, y = ints(1000), floats(1000)
    L.reset_names()
    px, py = L.param(1, "i32"), L.param(1, "f32")
    prog = A.build_program(A.zipWith(lambda a, b: A.from_integral(a, "f32") + b, px, py))
    before = gpu_ctx.stats()["h2d_bytes"]
    dx, dy = gpu_ctx.from_host_lazy(x), gpu_ctx.from_host_lazy(y)
    assert gpu_ctx.stats()["h2d_bytes"] == before
    order = [[px, py].index(next(q for q in (px, py) if q.node is n)) for n in prog.inputs]
    out, = gpu_ctx.execute(prog.text, [[dx, dy][k] for k in order], 1)
    assert gpu_ctx.stats()["h2d_bytes"] == before + x.nbytes + y.nbytes
    assert np.array_equal(out.download(), x.astype(np.float32) + y)
    # a download alone also triggers the copy; an explicit upload replaces an adopted payload
    dz = gpu_ctx.from_host_lazy(x)
    assert np.array_equal(dz.download(), x)
    dw = gpu_ctx.from_host_lazy(x)
    dw.upload([x + 1])
    assert np.array_equal(dw.download(), x + 1)


def test_download_async_arrives_after_sync(gpu_ctx):
    import torch
    x = ints(1 << 20)
    d = gpu_ctx.from_host(x)
    from accelerate_b200 import language as L
    L.reset_names()
    px = L.param(1, "i32")
    prog = A.build_program(A.map(lambda v: v * 3 + 1, px))
    bufs = []
    for _ in range(3):
        out, = gpu_ctx.execute(prog.text, [d], 1)
        t = torch.empty(x.shape, dtype=torch.int32, pin_memory=True)
        out.download_async([t.numpy()])
        out.free()                       # the memory is not reused before the copy has completed
        bufs.append(t)
    gpu_ctx.sync()
    for t in bufs:
        assert np.array_equal(t.numpy(), x * 3 + 1)


def test_bounded_wait_expiry_is_reported_and_the_context_stays_usable(monkeypatch):
    # Every device-side wait has an iteration limit.  With the limit at zero a look-back that does not
    # find its predecessors ready on the first poll gives up: the kernel records a status instead of
    # waiting, the host reports B200_ERR_TIMEOUT, and the context keeps working afterwards.
    from accelerate_b200 import backend, language as L
    x = ints(1 << 20, np.int32, 0, 100)            # 512 tiles on the register kernel (no bulk copies in flight)
    L.reset_names()
    px = L.param(1, "i32")
    prog = A.build_program(A.scanl1(add, px))
    monkeypatch.setenv("ACCELERATE_B200_SPIN_LIMIT", "0")
    ctx = backend.Context(0)
    try:
        d = ctx.from_host(x)
        try:
            out, = ctx.execute(prog.text, [d], 1)
            got = out.download()
            assert np.array_equal(got, np.cumsum(x, dtype=np.int32))     # every predecessor happened to be ready
        except backend.B200Error as e:
            assert e.code == 8, e                                        # B200_ERR_TIMEOUT
        # the same context, same program, on an input of one tile: nothing to wait for
        y = ints(1000, np.int32, 0, 100)
        out, = ctx.execute(prog.text, [ctx.from_host(y)], 1)
        assert np.array_equal(out.download(), np.cumsum(y, dtype=np.int32))
    finally:
        ctx.close()


def test_sixteen_component_tuples():
    # the widest tuples the reference's Elt instances cover (Sugar/Elt.hs: tuples up to 16): one buffer per component
    a = ints(3000, np.int32, -50, 50)
    wide = A.map(lambda v: A.tup(*[v + k for k in range(16)]), a)
    plus = lambda p, q: A.tup(*[p[k] + q[k] for k in range(16)])  # noqa: E731
    zero = A.tup(*[A.constant(np.int32(0)) for _ in range(16)])
    check(wide)
    check(A.fold(plus, zero, wide))
    check(A.scanl1(plus, wide))
    au = A.use(a)
    check(A.permute(plus, A.fill(7, zero), lambda ix: A.Just_(A.index(A.from_integral(au[ix] % 7, "i64"))), wide))


# ---- Half (Type.hs:127): binary16 whose every operation is the Float operation rounded back ---------------
def halves(n):
    x = rng.integers(0, 65536, size=n).astype(np.uint16).view(np.float16)
    x[:8] = np.array([0.0, -0.0, np.inf, -np.inf, 65504, 6e-8, 1.0, 2049], np.float16)
    return x


def test_half_primitives_exact():
    x, y = halves(4096), halves(4096)[::-1].copy()
    xs, ys = A.use(x), A.use(y)
    got = check(A.generate(A.index(4096), lambda ix: A.tup(
        xs[ix] + ys[ix], xs[ix] - ys[ix], xs[ix] * ys[ix], xs[ix] / ys[ix], -xs[ix], abs(xs[ix]), A.signum(xs[ix]),
        A.sqrt(abs(xs[ix])), A.recip(ys[ix]), A.max_(xs[ix], ys[ix]), A.min_(xs[ix], ys[ix]),
        xs[ix] < ys[ix], xs[ix].eq(ys[ix]), A.is_nan(xs[ix]), A.is_infinite(xs[ix]),
        A.bitcast(xs[ix], "u16"), A.pi("f16") * xs[ix], xs[ix] + 0.1)))
    with np.errstate(all="ignore"):
        want = x * y                                   # NumPy's float16 is the same definition: a third opinion
    ok = ~np.isnan(want)
    assert np.array_equal(got[2].view(np.uint16)[ok], want.view(np.uint16)[ok])


def test_half_conversions_exact():
    i = ints(2000, np.int32, -70000, 70000)
    f = (rng.normal(size=2000) * rng.choice([1e-6, 1.0, 300.0, 1e5], size=2000)).astype(np.float32)
    d = f.astype(np.float64) * 1.0000001
    h = rng.uniform(-3000, 3000, size=2000).astype(np.float16)
    h[:6] = np.array([0.5, 1.5, 2.5, -0.5, -1.5, -2.5], np.float16)
    is_, fs, ds, hs = A.use(i), A.use(f), A.use(d), A.use(h)
    check(A.generate(A.index(2000), lambda ix: A.tup(
        A.from_integral(is_[ix], "f16"), A.to_floating(fs[ix], "f16"), A.to_floating(ds[ix], "f16"),
        A.to_floating(hs[ix], "f32"), A.to_floating(hs[ix], "f64"), A.truncate(hs[ix]), A.round_(hs[ix], "i32"),
        A.floor(hs[ix]), A.ceiling(hs[ix]), A.bitcast(A.bitcast(hs[ix], "i16"), "f16"))))


def test_half_transcendentals():
    x = rng.uniform(0.1, 3.0, size=500).astype(np.float16)
    xs = A.use(x)
    # one unit in the last place of a Half at most (the Float results differ in their last place): far
    # inside the reference suite's tolerance for Half, absolute 0.05 / relative 0.5 (Test/Similar.hs:89)
    check(A.generate(A.index(500), lambda ix: A.tup(A.sin(xs[ix]), A.cos(xs[ix]), A.exp(xs[ix]), A.log(xs[ix]),
                                                     A.tanh(xs[ix]), xs[ix] ** 1.5, A.atan2(xs[ix], 2.0))), rtol=2e-3, atol=1e-3)


@pytest.mark.parametrize("n", [0, 1, 300, 5000, 100004])
def test_half_collectives_order_independent(n, monkeypatch):
    # zeros and ones whose sums stay below 2048: every partial sum is a Half whatever the association, so the
    # kernels' tree order must give the sequential result exactly (4096-element rows keep to that too)
    x = (rng.random(n) < 1500.0 / max(n, 1500)).astype(np.float16)
    check(A.fold(add, np.float16(0), x))
    check(A.scanl1(add, x))
    check(list(A.scanr_prime(add, np.float16(0), x)))
    if n:
        check(A.fold1(A.max_, rng.normal(size=n).astype(np.float16)))     # (no NaN: max is a monoid without it)
        k = A.use(ints(n, np.int32, 0, 37))
        check(A.permute(add, A.fill(37, A.constant(np.float16(0))), lambda ix: A.Just_(A.index(A.from_integral(k[ix], "i64"))), x))
        lens = np.full(n // 50, 50, np.int32)
        check(A.foldSeg(add, np.float16(0), x[:lens.sum()], lens))
    monkeypatch.setenv("ACCELERATE_B200_SCAN_NO_SMALL", "1")
    check(A.scanl(add, np.float16(1), x))


def test_half_stencil_and_tuples():
    m = rng.uniform(0, 1, size=(70, 132)).astype(np.float16)
    check(A.stencil(lambda s: (s[0][1] + s[2][1] + s[1][0] + s[1][2]) * 0.25, A.mirror, m))
    v = rng.uniform(-4, 4, size=3001).astype(np.float16)
    check(A.stencil(lambda s: s[0] * 0.25 + s[1] * 0.5 + s[2] * 0.25, A.function(lambda ix: A.constant(np.float16(7))), v, extent=(3,)))
    w = ints(3001, np.int32, -9, 9)
    pairs = A.zip(v, w)
    check(A.map(lambda p: A.tup(p[0] * A.from_integral(p[1], "f16"), p[1]), pairs), embed=True)
    check(A.scanl1(lambda a, b: A.tup(A.max_(a[0], b[0]), a[1] + b[1]), pairs))
