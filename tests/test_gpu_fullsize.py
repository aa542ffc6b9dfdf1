"""The benchmark's workloads at their full configured sizes, checked on the host.

At these sizes (2^28 .. 2^30 elements) the tree-walking oracle would take hours, so the
checks are vectorised NumPy restatements of the same definitions (integer work bit-exact,
wrapping like the reference's Int32/Int64; floating point within the tolerance stated at
each test) plus size-independent properties for the 100-fold iterated stencil, where even
NumPy is too slow: a constant field is a fixed point, and scaling the input by a power of
two scales the output exactly.
The inputs are the seeded arrays bench.py uses.
"""
import importlib.util
import os

import numpy as np
import pytest

import accelerate_b200 as A
from accelerate_b200 import language as L

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def bench():
    spec = importlib.util.spec_from_file_location("bench_for_tests", os.path.join(ROOT, "bench.py"))
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    return m


@pytest.fixture(scope="module")
def workloads(bench):
    return {w.name: w for w in bench.suite(0)}


def run(ctx, build, host):
    """Upload, run, download, free; returns a list of host arrays."""
    L.reset_names()
    params = [L.param(h.ndim, L.TY_OF_NP[h.dtype]) for h in host]
    prog = L.build_program(build(*params))
    order = [next(i for i, q in enumerate(params) if q.node is n) for n in prog.inputs]
    dev = [ctx.from_host(host[k]) for k in order]
    outs = ctx.execute(prog.text, dev, len(prog.outputs))
    res = [o.download() for o in outs]
    for d in dev + list(outs):
        d.free()
    return res


def test_fold1seg_int32_2p28(gpu_ctx, workloads):
    w = workloads["fold1seg_add_i32"]
    vals, lens = [f() for f in w.inputs]
    assert vals.size == 1 << 28 and int(lens.sum()) == vals.size and lens.min() >= 1
    got, = run(gpu_ctx, w.build, [vals, lens])
    starts = np.concatenate([[0], np.cumsum(lens[:-1], dtype=np.int64)])
    want = np.add.reduceat(vals, starts, dtype=np.int32)        # wraps like Int32
    assert got.dtype == np.int32 and np.array_equal(got, want)


def test_fold_max_rows_65536x4096(gpu_ctx, workloads):
    w = workloads["fold_max_rows_f32"]
    m, = [f() for f in w.inputs]
    assert m.shape == (65536, 4096)
    got, = run(gpu_ctx, w.build, [m])
    assert np.array_equal(got, m.max(axis=1))                   # max is exact in any order


def test_scanl1_int32_2p30_wraps(gpu_ctx, workloads):
    w = workloads["scanl1_add_i32"]
    x, = [f() for f in w.inputs]
    assert x.size == 1 << 30
    got, = run(gpu_ctx, w.build, [x])
    want = np.cumsum(x, dtype=np.int32)                          # two's-complement wrap, as Int32 (+)
    assert int(np.cumsum(x[: 1 << 27], dtype=np.int64)[-1]) > np.iinfo(np.int32).max   # the sums do overflow
    assert np.array_equal(got, want)


def test_scanl_prime_float_2p28(gpu_ctx, workloads):
    w = workloads["scanl_prime_add_f32"]
    x, = [f() for f in w.inputs]
    n = x.size
    assert n == 1 << 28
    prefix, total = run(gpu_ctx, w.build, [x])
    ref = np.cumsum(x, dtype=np.float64)
    # exclusive prefix sums and the total; tolerance 1e-5 * sqrt(n) relative for fp32 scans
    tol = 1e-5 * np.sqrt(n)
    assert prefix.shape == (n,) and prefix[0] == 0.0
    err = np.abs(prefix[1:].astype(np.float64) - ref[:-1]) / np.maximum(ref[:-1], 1.0)
    assert float(err.max()) <= tol
    assert abs(float(total) - ref[-1]) <= tol * ref[-1]


def test_scanr1_max_int64_2p28(gpu_ctx, workloads):
    w = workloads["scanr1_max_i64"]
    x, = [f() for f in w.inputs]
    assert x.size == 1 << 28 and x.dtype == np.int64
    got, = run(gpu_ctx, w.build, [x])
    want = np.maximum.accumulate(x[::-1])[::-1]
    assert np.array_equal(got, want)


@pytest.mark.parametrize("layout", ["permute_hist_i32", "permute_hist_i32_shuffled"])
def test_histogram_zipf_2p30(gpu_ctx, workloads, layout):
    # both layouts of the bins: frequent keys at the start of the target (inside the partial 32-bit private
    # copy) and scattered over it by a fixed shuffle (the device-side sample then picks the 16-bit fields)
    w = workloads[layout]
    keys, = [f() for f in w.inputs]
    assert keys.size == 1 << 30
    got, = run(gpu_ctx, w.build, [keys])
    want = np.bincount(keys, minlength=w.bins).astype(np.int32)
    assert got.shape == (w.bins,) and np.array_equal(got, want)
    assert int(got.astype(np.int64).sum()) == keys.size


def test_permute_add_float_2p30_with_dropped_indices(gpu_ctx, workloads):
    w = workloads["permute_add_f32"]
    keys, vals = [f() for f in w.inputs]
    n, bins = keys.size, w.bins
    assert n == 1 << 30
    got, = run(gpu_ctx, w.build, [keys, vals])
    keep = keys >= 0
    assert 0.05 < 1.0 - keep.mean() < 0.15                      # about 10 % of the elements are ignored
    want = np.bincount(keys[keep].astype(np.int64) % bins, weights=vals[keep].astype(np.float64), minlength=bins)
    # ~920 values per bin summed in arbitrary order: 1e-5 * sqrt(n / bins) relative per bin
    tol = 1e-5 * np.sqrt(n / bins)
    assert float((np.abs(got.astype(np.float64) - want) / np.maximum(want, 1.0)).max()) <= tol


def jacobi_np(x):
    p = np.pad(x, 1, mode="edge")                               # clamp
    return np.float32(0.25) * (((p[:-2, 1:-1] + p[2:, 1:-1]) + p[1:-1, :-2]) + p[1:-1, 2:])


def test_jacobi_16384_two_iterations_bit_exact(gpu_ctx, workloads, bench):
    g, = [f() for f in workloads["jacobi5_clamp_x100_f32"].inputs]
    assert g.shape == (16384, 16384)
    got, = run(gpu_ctx, lambda m: A.stencil(bench.jacobi, A.clamp, A.stencil(bench.jacobi, A.clamp, m)), [g])
    want = jacobi_np(jacobi_np(g))
    assert np.array_equal(got, want)                             # same expression order, no fused multiply-add


def test_jacobi_16384_x100_properties(gpu_ctx, workloads):
    w = workloads["jacobi5_clamp_x100_f32"]
    g, = [f() for f in w.inputs]
    out, = run(gpu_ctx, w.build, [g])
    # averaging never leaves the input's range and contracts it
    assert out.min() >= g.min() and out.max() <= g.max() and (out.max() - out.min()) < (g.max() - g.min())
    # scaling by a power of two is exact in binary floating point at every step
    out2, = run(gpu_ctx, w.build, [g * np.float32(4.0)])
    assert np.array_equal(out2, out * np.float32(4.0))
    del out2
    # a constant field is a fixed point under the clamp boundary (0.25 * 4c == c exactly)
    c = np.full_like(g, np.float32(0.625))
    outc, = run(gpu_ctx, w.build, [c])
    assert np.array_equal(outc, c)


def test_stencil2_gauss_mirror_16384(gpu_ctx, workloads, bench):
    w = workloads["stencil2_gauss_mirror_f32"]
    a, b = [f() for f in w.inputs]
    got, = run(gpu_ctx, w.build, [a, b])
    pa, pb = np.pad(a, 1, mode="reflect"), np.pad(b, 1, mode="reflect")     # mirror: -1 -> 1, n -> n-2
    n0, n1 = a.shape
    want = np.zeros_like(a)
    for i in range(3):
        for j in range(3):
            want = want + np.float32(bench.GAUSS[i][j] / 16.0) * (pa[i:i + n0, j:j + n1] + pb[i:i + n0, j:j + n1])
    # stencils: at most 1 ulp per point; with the same expression order and no fused multiply-add
    # the results are in fact identical
    assert np.array_equal(got, want)


# Long rows in several rows: the shared-memory ring and the 8192-element register tiles with partial
# last tiles, seeds, right-to-left order and row boundaries, at sizes the small-case tests do not reach.
def _scan_np(x, right, seed, op):
    acc = {"add": np.add, "max": np.maximum}[op].accumulate
    y = x[..., ::-1] if right else x
    if seed is not None:
        y = np.concatenate([np.full(y.shape[:-1] + (1,), seed, y.dtype), y], axis=-1)
    r = acc(y, axis=-1, dtype=y.dtype) if op == "add" else acc(y, axis=-1)
    return r[..., ::-1] if right else r


@pytest.mark.parametrize("name,shape,dtype", [
    ("scanl1", (4, (1 << 24) + 4), np.int32),        # ring, partial last tile in every row
    ("scanr1", (2, 1 << 24), np.int32),              # ring, right to left
    ("scanl", (1, (1 << 25) + 3), np.int32),         # ring, seeded: n+1 results
    ("scanr", (2, (1 << 22) + 3), np.int32),         # seeded, right to left, rows of n+1 results
    ("scanl'", (3, (1 << 23) + 8), np.int32),        # ring, totals in a second array
    ("scanr'", (2, 1 << 23), np.int64),              # register kernel, 8-byte elements
    ("scanl1max", (5, (1 << 22) + 12), np.int64),
])
def test_long_rows_scans(gpu_ctx, name, shape, dtype):
    g = np.random.default_rng(7)
    x = g.integers(0, 100, size=shape).astype(dtype) if dtype == np.int32 else g.integers(-(1 << 62), 1 << 62, size=shape, dtype=np.int64)
    add = lambda a, b: a + b  # noqa: E731
    if name == "scanl1":
        got, = run(gpu_ctx, lambda a: A.scanl1(add, a), [x]); want = _scan_np(x, False, None, "add")
    elif name == "scanr1":
        got, = run(gpu_ctx, lambda a: A.scanr1(add, a), [x]); want = _scan_np(x, True, None, "add")
    elif name == "scanl":
        got, = run(gpu_ctx, lambda a: A.scanl(add, 7, a), [x]); want = _scan_np(x, False, 7, "add")
    elif name == "scanr":
        got, = run(gpu_ctx, lambda a: A.scanr(add, 7, a), [x]); want = _scan_np(x, True, 7, "add")
    elif name == "scanl'":
        got, tot = run(gpu_ctx, lambda a: list(A.scanl_prime(add, 7, a)), [x])
        full = _scan_np(x, False, 7, "add")
        want = full[..., :-1]
        assert np.array_equal(tot, full[..., -1])
    elif name == "scanr'":
        got, tot = run(gpu_ctx, lambda a: list(A.scanr_prime(A.max_, -(1 << 63), a)), [x])
        full = _scan_np(x, True, -(1 << 63), "max")
        want = full[..., 1:]
        assert np.array_equal(tot, full[..., 0])
    else:
        got, = run(gpu_ctx, lambda a: A.scanl1(A.max_, a), [x]); want = _scan_np(x, False, None, "max")
    assert got.shape == want.shape and np.array_equal(got, want)
