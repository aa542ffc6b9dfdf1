"""Seeded random shapes around the places where the kernels switch strategy: the row-staged stencil
against the plain one (column counts that are and are not multiples of four, differing extents of
stencil2's two arrays, every boundary), the ring scans against the small scans (lengths a few elements
either side of a tile), the histogram's 16-bit private bins (sizes either side of the shared-memory
limits, with counts that overflow 16 bits), row windows of one and two ranges, and ragged segments.
The same generators were run for two thousand cases before these seeds were fixed; the property is
the one the reference's nofib suite checks (Test/Similar.hs:35-37: exact for integers, tolerance for
floating point) with the oracle or NumPy as the expected value."""
import numpy as np
import pytest

import accelerate_b200 as A
from accelerate_b200 import language as L
from tests.util import check

pytestmark = pytest.mark.gpu

W = [[1, 2, 1], [2, 4, 2], [1, 2, 1]]
BOUNDARIES = [A.clamp, A.mirror, A.wrap]


def add(a, b):
    return a + b


def gauss2(s, t):
    return sum((np.float32(W[i][j] / 16.0) * (s[i][j] + t[i][j]) for i in range(3) for j in range(3)),
               A.constant(np.float32(0)))


def rng(kind, seed):
    return np.random.default_rng([kind, seed])


@pytest.mark.parametrize("seed", range(12))
def test_stencil2_random_extents(seed):
    g = rng(0, seed)
    r, c = int(g.integers(3, 260)), int(g.integers(3, 180)) * int(g.choice([1, 4]))
    r2, c2 = r + int(g.integers(0, 9)), c + 4 * int(g.integers(0, 5))
    a = g.uniform(0, 1, (r, c)).astype(np.float32)
    b = g.uniform(0, 1, (r2, c2)).astype(np.float32)
    check(A.stencil2(gauss2, BOUNDARIES[g.integers(3)], a, BOUNDARIES[g.integers(3)], b))


@pytest.mark.parametrize("seed", range(6))
def test_stencil_f64_random_extents(seed):
    g = rng(1, seed)
    r, c = int(g.integers(60, 200)), 4 * int(g.integers(50, 130))
    m = g.uniform(0, 1, (r, c))
    e = int(g.choice([3, 5]))

    def f(s):
        return sum((s[i][j] * float(i * 3 + j + 1) for i in range(e) for j in range(3)), A.constant(np.float64(0)))

    check(A.stencil(f, BOUNDARIES[g.integers(3)], m, extent=(e, 3)))


@pytest.mark.parametrize("seed", range(24))
def test_scan_random_lengths_near_tiles(seed, monkeypatch):
    monkeypatch.setenv("ACCELERATE_B200_SCAN_NO_SMALL", "1")
    g = rng(2, seed)
    dt = [np.int32, np.int64, np.float32, np.int16, np.uint8][g.integers(5)]
    rows = int(g.choice([1, 1, 2, 3, 7]))
    m = int(g.choice([4096, 8192, 16384, 32768])) * int(g.integers(1, 4)) + int(g.choice([0, 0, 4, 8, -4, 1, 13]))
    x = g.integers(0, 50, size=(rows, m) if rows > 1 else (m,)).astype(dt)
    z = np.array(3).astype(dt)[()]
    tol = dict(rtol=1e-4, atol=1e-2) if dt == np.float32 else {}
    which = seed % 6
    term = [lambda: A.scanl1(add, x), lambda: A.scanr1(add, x), lambda: A.scanl(add, z, x),
            lambda: A.scanr(add, z, x), lambda: list(A.scanl_prime(add, z, x)),
            lambda: list(A.scanr_prime(add, z, x))][which]()
    check(term, **tol)


@pytest.mark.parametrize("out_n", [51200, 51201, 65536, 70001, 114688, 114689])
@pytest.mark.parametrize("hot", [0.0, 0.9])
def test_histogram_private_bin_limits(out_n, hot, gpu_ctx):
    from accelerate_b200 import backend
    g = rng(3, out_n + int(hot * 10))
    total = out_n * int(g.integers(8, 11))
    k = g.integers(0, out_n, size=total).astype(np.int32)
    k[g.random(total) < hot] = int(g.integers(0, out_n))
    # values far above 65535 in one bin: the 16-bit private counters must spill without losing a carry
    v = g.integers(-3, 70000, size=total).astype(np.int32) if out_n % 2 else np.ones(total, np.int32)
    ku = A.use(k)
    got = backend.run(A.permute(add, A.fill(out_n, A.constant(np.int32(0))),
                                lambda ix: A.Just_(A.index(A.from_integral(ku[ix], "i64"))), v), gpu_ctx)
    want = np.zeros(out_n, np.int64)
    np.add.at(want, k, v.astype(np.int64))
    assert np.array_equal(got, want.astype(np.int32))


@pytest.mark.parametrize("seed", range(10))
def test_row_windows_random_cuts(seed, gpu_ctx):
    g = rng(4, seed)
    r, c = int(g.integers(8, 200)), int(g.integers(4, 400))
    m = g.uniform(0, 1, (r, c)).astype(np.float32)
    L.reset_names()
    text = A.build_program(A.stencil(lambda s: 0.25 * (s[0][1] + s[2][1] + s[1][0] + s[1][2]),
                                     BOUNDARIES[g.integers(3)], L.param(2, "f32"))).text
    a = gpu_ctx.from_host(m)
    full, = gpu_ctx.execute(text, [a], 1)
    want = full.download()
    cuts = sorted(int(x) for x in g.integers(0, r + 1, size=4))
    out = gpu_ctx.from_host(np.zeros_like(m))
    exp = np.zeros_like(m)
    if cuts[0] < cuts[1] and cuts[2] < cuts[3]:
        gpu_ctx.run_rows2(text, [a], out, cuts[0], cuts[1], cuts[2], cuts[3])
        exp[cuts[0]:cuts[1]] = want[cuts[0]:cuts[1]]
        exp[cuts[2]:cuts[3]] = want[cuts[2]:cuts[3]]
    else:
        gpu_ctx.run_rows(text, [a], out, cuts[0], cuts[3])
        exp[cuts[0]:cuts[3]] = want[cuts[0]:cuts[3]]
    assert np.array_equal(out.download(), exp)


@pytest.mark.parametrize("seed", range(8))
def test_foldseg_random_ragged_segments(seed):
    g = rng(5, seed)
    segs = int(g.integers(1, 3000))
    lens = g.integers(0, 60, size=segs).astype(np.int32)
    x = g.integers(-100, 100, size=int(lens.sum())).astype(np.int32)
    check(A.foldSeg(add, 0, x, lens))
