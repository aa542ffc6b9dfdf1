"""The oracle's primitive table (Interpreter.hs:1086-1416 over GHC's numeric classes) against references
that share nothing with it: Python's unbounded integers reduced to the type's width, and NumPy for floating
point.  The properties are those of the reference's Map and ZipWith groups (Test/NoFib/Prelude/Map.hs:76-135,
ZipWith.hs:76-150), every integer width and both floating types."""
import numpy as np
import pytest

import accelerate_b200 as A
from oracle import oracle

INTS = ["i8", "i16", "i32", "i64", "u8", "u16", "u32", "u64"]
N = 400


def wrap(v, ty):
    bits = int(ty[1:])
    v &= (1 << bits) - 1
    if ty[0] == "i" and v >> (bits - 1):
        v -= 1 << bits
    return v


def column(vals, ty):
    return np.array([wrap(int(v), ty) for v in vals], dtype=A.NP_OF[ty])


def operands(ty, seed):
    g = np.random.default_rng(seed)
    info = np.iinfo(A.NP_OF[ty])
    x = g.integers(info.min, info.max, size=N, dtype=A.NP_OF[ty], endpoint=True)
    y = g.integers(info.min, info.max, size=N, dtype=A.NP_OF[ty], endpoint=True)
    x[:6] = [info.min, info.max, 0, 1, info.min, info.max]
    y[:6] = [1, info.max, 3, info.min, 2, 1]
    y[y == 0] = 7
    if ty[0] == "i":
        y[(x == info.min) & (y == -1)] = 5          # quot minBound (-1) overflows in GHC: not a defined result
    return x, y, g.integers(0, int(ty[1:]) + 6, size=N).astype(np.int64)


@pytest.mark.parametrize("ty", INTS)
def test_integer_primitives_against_python_integers(ty):
    x, y, s = operands(ty, INTS.index(ty))
    bits, signed = int(ty[1:]), ty[0] == "i"
    xs, ys, ss = A.use(x), A.use(y), A.use(s)
    got = oracle.run(A.generate(A.index(N), lambda ix: A.tup(
        xs[ix] + ys[ix], xs[ix] - ys[ix], xs[ix] * ys[ix], -xs[ix], abs(xs[ix]), A.signum(xs[ix]),
        A.quot(xs[ix], ys[ix]), A.rem(xs[ix], ys[ix]), xs[ix] // ys[ix], xs[ix] % ys[ix],
        xs[ix] & ys[ix], xs[ix] | ys[ix], xs[ix] ^ ys[ix], ~xs[ix], xs[ix] << ss[ix], xs[ix] >> ss[ix],
        A.rotate_l(xs[ix], ss[ix]), A.rotate_r(xs[ix], ss[ix]),
        A.pop_count(xs[ix]), A.count_leading_zeros(xs[ix]), A.count_trailing_zeros(xs[ix]),
        A.max_(xs[ix], ys[ix]), A.min_(xs[ix], ys[ix]), xs[ix] < ys[ix], xs[ix] >= ys[ix], xs[ix].eq(ys[ix]), xs[ix].ne(ys[ix]),
        A.from_integral(xs[ix], "i64"), A.from_integral(xs[ix], "u8"), A.from_integral(xs[ix], "i16"), A.from_integral(xs[ix], "f64"))))
    X, Y, S = [int(v) for v in x], [int(v) for v in y], [int(v) for v in s]
    mask = (1 << bits) - 1

    def trunc_div(a, b):
        q = abs(a) // abs(b)
        return q if (a < 0) == (b < 0) else -q

    def rotl(a, n):
        n %= bits
        u = a & mask
        return ((u << n) | (u >> (bits - n))) & mask if n else u

    def clz(a):
        return bits - (a & mask).bit_length()

    def ctz(a):
        u = a & mask
        return bits if u == 0 else (u & -u).bit_length() - 1
    want = [
        [a + b for a, b in zip(X, Y)], [a - b for a, b in zip(X, Y)], [a * b for a, b in zip(X, Y)], [-a for a in X],
        [abs(a) for a in X], [(a > 0) - (a < 0) for a in X],
        [trunc_div(a, b) for a, b in zip(X, Y)], [a - b * trunc_div(a, b) for a, b in zip(X, Y)],
        [a // b for a, b in zip(X, Y)], [a % b for a, b in zip(X, Y)],                      # Python's // and % floor, as div and mod do
        [a & b for a, b in zip(X, Y)], [a | b for a, b in zip(X, Y)], [a ^ b for a, b in zip(X, Y)], [~a for a in X],
        [(a << n) if n < bits else 0 for a, n in zip(X, S)],
        [(a >> n) if n < bits else (-1 if a < 0 else 0) for a, n in zip(X, S)],             # arithmetic on signed, logical on unsigned
        [rotl(a, n) for a, n in zip(X, S)], [rotl(a, -n) for a, n in zip(X, S)],
    ]
    for k, w in enumerate(want):
        assert np.array_equal(got[k], column(w, ty)), k
    assert np.array_equal(got[18], [bin(a & mask).count("1") for a in X])
    assert np.array_equal(got[19], [clz(a) for a in X])
    assert np.array_equal(got[20], [ctz(a) for a in X])
    assert np.array_equal(got[21], np.maximum(x, y)) and np.array_equal(got[22], np.minimum(x, y))
    assert np.array_equal(got[23], x < y) and np.array_equal(got[24], x >= y)
    assert np.array_equal(got[25], x == y) and np.array_equal(got[26], x != y)
    assert np.array_equal(got[27], column(X, "i64")) and np.array_equal(got[28], column(X, "u8"))
    assert np.array_equal(got[29], column(X, "i16")) and np.array_equal(got[30], x.astype(np.float64))
    assert all(got[k].dtype == np.int64 for k in (18, 19, 20)) and all(got[k].dtype == np.uint8 for k in range(23, 27))
    assert signed or np.array_equal(got[5], (x != 0).astype(x.dtype))


@pytest.mark.parametrize("ty", ["f32", "f64"])
def test_floating_primitives_against_numpy(ty):
    dt = A.NP_OF[ty]
    g = np.random.default_rng(5)
    x = (g.normal(size=N) * 20).astype(dt)
    y = (g.normal(size=N) * 3).astype(dt)
    u = g.uniform(-1, 1, N).astype(dt)
    p = g.uniform(0.01, 50, N).astype(dt)
    x[:6] = [0.5, 1.5, 2.5, -0.5, -1.5, -2.5]
    xs, ys, us, ps = A.use(x), A.use(y), A.use(u), A.use(p)
    got = oracle.run(A.generate(A.index(N), lambda ix: A.tup(
        xs[ix] + ys[ix], xs[ix] - ys[ix], xs[ix] * ys[ix], xs[ix] / ys[ix], -xs[ix], abs(xs[ix]), A.signum(xs[ix]), A.recip(ys[ix]),
        A.sqrt(ps[ix]), A.truncate(xs[ix]), A.round_(xs[ix]), A.floor(xs[ix]), A.ceiling(xs[ix]),
        A.max_(xs[ix], ys[ix]), A.min_(xs[ix], ys[ix]), xs[ix] < ys[ix], xs[ix].eq(ys[ix]),
        A.sin(xs[ix]), A.cos(xs[ix]), A.tan(us[ix]), A.asin(us[ix]), A.acos(us[ix]), A.atan(xs[ix]), A.sinh(us[ix]), A.cosh(us[ix]),
        A.tanh(xs[ix]), A.asinh(xs[ix]), A.acosh(ps[ix] + 1), A.atanh(us[ix] * 0.99), A.exp(us[ix]), A.log(ps[ix]),
        ps[ix] ** us[ix], A.atan2(xs[ix], ys[ix]), A.log_base(ps[ix] + 1.5, ps[ix]))))
    with np.errstate(all="ignore"):
        exact = [x + y, x - y, x * y, x / y, -x, np.abs(x), np.sign(x), dt(1) / y, np.sqrt(p),
                 np.trunc(x).astype(np.int64), np.rint(x).astype(np.int64), np.floor(x).astype(np.int64), np.ceil(x).astype(np.int64),
                 np.maximum(x, y), np.minimum(x, y), (x < y).astype(np.uint8), (x == y).astype(np.uint8)]
        close = [np.sin(x), np.cos(x), np.tan(u), np.arcsin(u), np.arccos(u), np.arctan(x), np.sinh(u), np.cosh(u), np.tanh(x),
                 np.arcsinh(x), np.arccosh(p + dt(1)), np.arctanh(u * dt(0.99)), np.exp(u), np.log(p), p ** u, np.arctan2(x, y),
                 np.log(p) / np.log(p + dt(1.5))]
    for k, w in enumerate(exact):
        assert got[k].dtype == w.dtype and np.array_equal(got[k], w), k
    eps = np.finfo(dt).eps
    for k, w in enumerate(close):
        gk = got[len(exact) + k]
        assert gk.dtype == dt and np.all(np.abs(gk - w) <= 8 * eps * np.maximum(np.abs(w), 1)), k
