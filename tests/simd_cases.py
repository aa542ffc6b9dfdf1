"""The reference's SIMD properties (Test/NoFib/Prelude/SIMD.hs:43-170): `extract` maps a projection of
`unpackVec{2,3,4}'` over an array of vectors, `inject` zips n arrays of scalars into an array of vectors;
every scalar type, and beyond the reference a rank-2 array, a fold over vectors and a scalar of a vector.
An array of `Vec n t` is an ndarray of t with one more axis of length n (Array/Data.hs:108-119), so the
expected values are NumPy slices and stacks, the counterpart of the reference's list functions."""
import numpy as np

import accelerate_b200 as A

TYPES = ["i8", "i16", "i32", "i64", "u8", "u16", "u32", "u64", "f16", "f32", "f64"]


def data(ty, shape, seed):
    g = np.random.default_rng(seed)
    dt = A.NP_OF[ty]
    if np.issubdtype(dt, np.integer):
        info = np.iinfo(dt)
        return g.integers(info.min, info.max, size=shape, dtype=dt, endpoint=True)
    return (g.normal(size=shape) * 100).astype(dt)


def cases():
    out = {}
    for ty in TYPES:
        for n in (2, 3, 4):
            x = data(ty, (257, n), 100 * n + TYPES.index(ty))
            xs = A.use(x, elt=A.vec(n, ty))
            for k in range(n):
                # test_extract_v{n}: map (view _k . unpackVec') xs
                out[f"extract_v{n}_{ty}_{k + 1}"] = (A.map(lambda v, k=k: A.vec_unpack(v)[k], xs), x[:, k].copy())
            parts = [data(ty, (301 - 7 * j,), 7 * n + j) for j in range(n)]        # zipWith: the shortest wins
            m = min(len(p) for p in parts)
            if n == 2:
                term = A.zipWith(lambda a, b: A.vec_pack(a, b), *parts)
            elif n == 3:
                term = A.zipWith3(lambda a, b, c: A.vec_pack(a, b, c), *parts)
            else:
                term = A.zipWith4(lambda a, b, c, d: A.vec_pack(a, b, c, d), *parts)
            out[f"inject_v{n}_{ty}"] = (term, np.stack([p[:m] for p in parts], axis=-1))
    x = data("f32", (19, 33, 4), 5)
    xs = A.use(x, elt=A.vec(4, "f32"))
    out["rank2_swizzle_v4_f32"] = (A.map(lambda v: A.vec_pack(*list(A.vec_unpack(v))[::-1]), xs), x[..., ::-1].copy())
    y = data("i32", (1000, 3), 6)
    ys = A.use(y, elt=A.vec(3, "i32"))
    plus = lambda a, b: A.vec_pack(*[p + q for p, q in zip(A.vec_unpack(a), A.vec_unpack(b))])  # noqa: E731
    zero = A.vec_pack(*[A.constant(np.int32(0))] * 3)
    out["fold_sum_v3_i32"] = (A.fold(plus, zero, ys), y.sum(axis=0, dtype=np.int32))
    out["scanl1_sum_v3_i32"] = (A.scanl1(plus, ys), np.cumsum(y, axis=0, dtype=np.int32))
    c = data("f64", (64, 2), 7)                      # Complex Double is a Vec2 (Data/Complex.hs:117)
    cs = A.use(c, elt=A.vec(2, "f64"))

    def cmul(a, b):
        (ar, ai), (br, bi) = A.vec_unpack(a), A.vec_unpack(b)
        return A.vec_pack(ar * br - ai * bi, ar * bi + ai * br)
    re, im = c[:, 0], c[:, 1]
    out["complex_square_v2_f64"] = (A.zipWith(cmul, cs, cs), np.stack([re * re - im * im, re * im + im * re], axis=-1))
    return out
