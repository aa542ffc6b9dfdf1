"""Programs with array-level control flow (Acond, Awhile, Apply, Use), shared by the oracle
tests and the GPU parity tests.  Each case is ``(term, expected)`` with the expected value
computed independently in NumPy."""
import numpy as np

import accelerate_b200 as A

add = lambda a, b: a + b  # noqa: E731


def jacobi(s):
    return 0.25 * (s[0][1] + s[2][1] + s[1][0] + s[1][2])


def jacobi_np(g, iters):
    for _ in range(iters):
        p = np.pad(g, 1, mode="edge")
        g = np.float32(0.25) * (((p[:-2, 1:-1] + p[2:, 1:-1]) + p[1:-1, :-2]) + p[1:-1, 2:])
    return g


def radixsort(xs, bits=16):
    """The reference's test program for array pipelines (Test/NoFib/Spectral/RadixSort.hs:167-180):
    one stable split per bit, chained with ``>->``; the sign bit is flipped on the last pass
    (radixOfSigned, :139-147)."""
    def radix_pass(k):
        def go(v):
            def radix(e):
                x = e ^ A.min_bound(e.ty) if k == bits - 1 else e
                return A.from_integral((x >> k) & 1, "i64")
            flags = A.map(radix, v)
            idown = A.scanl_prime(add, 0, A.map(lambda f: f ^ 1, flags))[0]                    # prescanl
            iup = A.map(lambda i: v.size() - 1 - i, A.scanr_prime(add, 0, flags)[0])           # prescanr
            index = A.zipWith(lambda f, du: A.cond(f.eq(0), du[0], du[1]), flags, A.zip(idown, iup))
            return A.permute(lambda new, old: new, v, lambda ix: A.Just_(A.index(index[ix])), v)
        return go
    f = radix_pass(0)
    for k in range(1, bits):
        f = A.pipe(f, radix_pass(k))
    return f(A.use(xs))


def cases():
    g = np.random.default_rng(3)
    out = {}
    x = g.integers(1, 50, size=300).astype(np.int64)
    # Awhile with a data-dependent trip count: double until the sum passes a bound
    want = x.copy()
    while want.sum() < 10_000_000:
        want = want * 2
    out["awhile_double_until"] = (A.awhile(lambda s: A.unit(A.the(A.sum(s)) < 10_000_000), lambda s: A.map(lambda v: v * 2, s), x), want)
    # Awhile over a pair of arrays: a Jacobi grid and an iteration counter (a fixed trip count written as a loop)
    grid = g.random(size=(37, 53), dtype=np.float32)
    for iters in (0, 1, 10):
        t = A.awhile(lambda s: A.unit(A.the(s[1]) < iters),
                     lambda s: (A.stencil(jacobi, A.clamp, s[0]), A.unit(A.the(s[1]) + 1)),
                     (grid, A.unit(A.constant(np.int64(0)))))
        out[f"awhile_jacobi_{iters}"] = (list(t), [jacobi_np(grid, iters), np.array(iters, np.int64)])
    # Acond: both branches, the predicate reads an array; only the chosen branch may run (the other divides by zero)
    zeros = np.zeros(300, np.int64)
    out["acond_then"] = (A.acond(A.the(A.sum(x)) > 5, A.map(lambda v: v + 1, x), A.zipWith(lambda a, b: a // b, x, zeros)), x + 1)
    out["acond_else"] = (A.acond(A.the(A.sum(x)) < 5, A.zipWith(lambda a, b: a // b, x, zeros), A.scanl1(add, x)), np.cumsum(x))
    # a node both branches need is computed once, in front of the Acond
    shared = A.scanl1(add, x)
    out["acond_shared"] = (A.acond(A.the(A.sum(x)) > 5, A.map(lambda v: v + 1, shared), A.map(lambda v: v - 1, shared)), np.cumsum(x) + 1)
    # nested: a loop whose step contains a conditional; loop-invariant nodes are hoisted
    inv = A.map(lambda v: v % 7, x)

    def step(s):
        big = A.the(A.maximum(s)) > 1000
        return A.acond(big, A.map(lambda v: v // 3, s), A.zipWith(add, s, A.zipWith(add, s, inv)))
    want = x.copy()
    k = 0
    while want.sum() < 200_000 and k < 1000:
        want = want // 3 if want.max() > 1000 else want + want + x % 7
        k += 1
    out["awhile_nested_acond"] = (A.awhile(lambda s: A.unit(A.the(A.sum(s)) < 200_000), step, x), want)
    # Apply / pipelines: radix sort (16 chained array functions)
    keys = g.integers(-2000, 2000, size=128).astype(np.int16)
    out["apply_radixsort_i16"] = (radixsort(keys), np.sort(keys))
    out["apply_radixsort_empty"] = (radixsort(np.zeros(0, np.int16)), np.zeros(0, np.int16))
    out["apply_two_results"] = (list(A.apply(lambda a, b: (A.zipWith(add, a, b), A.sum(a)), x, x)), [x + x, np.array(x.sum())])
    return out
