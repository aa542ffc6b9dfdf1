"""Half (Type.hs:127; `half >= 0.3`, accelerate.cabal:335) on the oracle, against NumPy's float16.
Both define an operation on binary16 as the binary32 operation on the converted operands, rounded back
to nearest even, so the arithmetic and the conversions must agree bit for bit; transcendental functions
are compared within the reference suite's tolerance for Half (Test/Similar.hs:89).  The kernels for the
same programs are compiled here (no GPU needed) and run in tests/test_gpu_parity.py."""
import numpy as np

import accelerate_b200 as A
from accelerate_b200 import backend
from oracle import oracle

rng = np.random.default_rng(16)


def bits(a):
    return np.asarray(a).view(np.uint16)


def same_half(got, want):
    assert got.dtype == np.float16 and got.shape == want.shape
    nan = np.isnan(want)
    assert np.array_equal(np.isnan(got), nan)
    assert np.array_equal(bits(got)[~nan], bits(want)[~nan]), (got[~nan][bits(got)[~nan] != bits(want)[~nan]][:5],
                                                                want[~nan][bits(got)[~nan] != bits(want)[~nan]][:5])


def operands(n=4096):
    # every exponent including subnormals, plus the special values
    x = rng.integers(0, 65536, size=n).astype(np.uint16).view(np.float16)
    y = rng.integers(0, 65536, size=n).astype(np.uint16).view(np.float16)
    x[:8] = np.array([0.0, -0.0, np.inf, -np.inf, 65504, 6e-8, 1.0, 2049], np.float16)
    y[:8] = np.array([1.0, 3.0, 1.0, np.inf, 65504, 6e-8, 3.0, 1], np.float16)
    return x, y


def test_half_arithmetic_is_float_arithmetic_rounded_to_nearest_even():
    x, y = operands()
    xs, ys = A.use(x), A.use(y)
    with np.errstate(all="ignore"):
        want = [x + y, x - y, x * y, x / y, -x, np.abs(x), np.sqrt(np.abs(x)), np.float16(1) / y]
    got = oracle.run(A.generate(A.index(len(x)), lambda ix: A.tup(
        xs[ix] + ys[ix], xs[ix] - ys[ix], xs[ix] * ys[ix], xs[ix] / ys[ix], -xs[ix], abs(xs[ix]),
        A.sqrt(abs(xs[ix])), A.recip(ys[ix]))))
    for g, w in zip(got, want):
        same_half(g, w)


def test_half_comparisons_and_selection():
    x, y = operands()
    xs, ys = A.use(x), A.use(y)
    got = oracle.run(A.generate(A.index(len(x)), lambda ix: A.tup(
        xs[ix] < ys[ix], xs[ix] <= ys[ix], xs[ix].eq(ys[ix]), A.is_nan(xs[ix]), A.is_infinite(xs[ix]),
        A.max_(xs[ix], ys[ix]), A.min_(xs[ix], ys[ix]))))
    with np.errstate(all="ignore"):
        assert np.array_equal(got[0], (x < y).astype(np.uint8))
        assert np.array_equal(got[1], (x <= y).astype(np.uint8))
        assert np.array_equal(got[2], (x == y).astype(np.uint8))
        assert np.array_equal(got[3], np.isnan(x).astype(np.uint8))
        assert np.array_equal(got[4], np.isinf(x).astype(np.uint8))
        # GHC's Ord defaults: max x y = if x <= y then y else x; min x y = if x <= y then x else y
        same_half(got[5], np.where(x <= y, y, x))
        same_half(got[6], np.where(x <= y, x, y))


def test_half_conversions():
    i = rng.integers(-70000, 70000, size=2000).astype(np.int32)
    f = (rng.normal(size=2000) * rng.choice([1e-6, 1.0, 300.0, 1e5], size=2000)).astype(np.float32)
    d = f.astype(np.float64) * 1.0000001
    h = rng.uniform(-3000, 3000, size=2000).astype(np.float16)
    h[:6] = np.array([0.5, 1.5, 2.5, -0.5, -1.5, -2.5], np.float16)
    is_, fs, ds, hs = A.use(i), A.use(f), A.use(d), A.use(h)
    got = oracle.run(A.generate(A.index(2000), lambda ix: A.tup(
        A.from_integral(is_[ix], "f16"), A.to_floating(fs[ix], "f16"), A.to_floating(ds[ix], "f16"),
        A.to_floating(hs[ix], "f32"), A.to_floating(hs[ix], "f64"), A.truncate(hs[ix]), A.round_(hs[ix], "i32"),
        A.floor(hs[ix]), A.ceiling(hs[ix]), A.bitcast(hs[ix], "u16"), A.bitcast(A.bitcast(hs[ix], "i16"), "f16"))))
    with np.errstate(all="ignore"):
        same_half(got[0], i.astype(np.float32).astype(np.float16))
        same_half(got[1], f.astype(np.float16))
        same_half(got[2], d.astype(np.float32).astype(np.float16))      # through Float, as fromRational does
    assert np.array_equal(got[3], h.astype(np.float32))
    assert np.array_equal(got[4], h.astype(np.float64))
    assert np.array_equal(got[5], np.trunc(h.astype(np.float32)).astype(np.int64))
    assert np.array_equal(got[6], np.rint(h.astype(np.float32)).astype(np.int32))
    assert np.array_equal(got[7], np.floor(h.astype(np.float32)).astype(np.int64))
    assert np.array_equal(got[8], np.ceil(h.astype(np.float32)).astype(np.int64))
    assert np.array_equal(got[9], bits(h))
    same_half(got[10], h)


def test_half_transcendentals_and_constants():
    x = rng.uniform(0.1, 3.0, size=500).astype(np.float16)
    xs = A.use(x)
    got = oracle.run(A.generate(A.index(500), lambda ix: A.tup(
        A.sin(xs[ix]), A.exp(xs[ix]), A.log(xs[ix]), xs[ix] ** 1.5, A.pi("f16") * xs[ix], xs[ix] + 0.1)))
    x32 = x.astype(np.float32)
    want = [np.sin(x32), np.exp(x32), np.log(x32), x32 ** np.float32(1.5)]
    for g, w in zip(got[:4], want):
        assert g.dtype == np.float16
        assert np.all(np.abs(g.astype(np.float32) - w) <= 2e-3 * np.abs(w) + 1e-3)  # far inside the suite's 0.05 / 0.5
    same_half(got[4], np.float16(np.pi) * x)
    same_half(got[5], x + np.float16(0.1))


def test_half_fold_and_scan_round_after_every_step():
    x = rng.uniform(0, 4, size=300).astype(np.float16)
    acc, run = np.float16(0), []
    for v in x:
        acc = np.float16(acc + v)
        run.append(acc)
    same_half(oracle.run(A.scanl1(lambda a, b: a + b, x)), np.array(run, np.float16))
    same_half(oracle.run(A.fold(lambda a, b: a + b, np.float16(0), x)), np.array(acc, np.float16))
    same_half(oracle.run(A.fold1(A.max_, x)), np.array(x.max(), np.float16))


def test_half_programs_compile():
    x = rng.uniform(0, 4, size=300).astype(np.float16)
    m = rng.uniform(0, 1, size=(40, 64)).astype(np.float16)
    k = rng.integers(0, 50, size=300).astype(np.int32)
    ks = A.use(k)
    add = lambda a, b: a + b
    for term in (A.map(lambda v: A.sin(v) * 2.0 + A.to_floating(A.truncate(v), "f16"), x),
                 A.fold(add, np.float16(0), x), A.scanl1(add, x), A.scanr(A.max_, np.float16(0), x),
                 A.stencil(lambda s: (s[0][1] + s[2][1] + s[1][0] + s[1][2]) * 0.25, A.clamp, m),
                 A.permute(add, A.fill(50, A.constant(np.float16(0))), lambda ix: A.Just_(A.index(A.from_integral(ks[ix], "i64"))), x)):
        assert "ok" in backend.compile_check(A.build_program(term).text)


def test_half_every_bit_pattern_survives_a_copy_and_a_bitcast():
    # Half is a newtype over its 16 bits (Numeric.Half): signalling NaNs and payloads included
    x = np.arange(65536, dtype=np.uint16).view(np.float16)
    xs = A.use(x)
    got = oracle.run(A.generate(A.index(65536), lambda ix: A.tup(A.bitcast(xs[ix], "u16"), xs[ix])))
    assert np.array_equal(got[0], bits(x)) and np.array_equal(bits(got[1]), bits(x))
