"""The reference's own known-answer cases for the hot path, restated with the
Python front end.  Expected values live in tests/golden/reference_vectors.json
(extracted from the reference's files by tests/golden/make_golden.py); each
case cites where its program and inputs are written in the reference
(paths relative to src/Data/Array/Accelerate/)."""
import json
import os

import numpy as np

import accelerate_b200 as A

HERE = os.path.dirname(os.path.abspath(__file__))
VECTORS = json.load(open(os.path.join(HERE, "golden", "reference_vectors.json")))
add = lambda a, b: a + b  # noqa: E731
I = np.int64  # Haskell Int


def _mss(x, y):
    # Language.hs:501-508
    return A.tup(A.max_(x[0], A.max_(y[0], x[2] + y[1])), A.max_(x[1], x[3] + y[1]), A.max_(y[2], x[2] + y[3]), x[3] + y[3])


def _issue137():
    # Test/NoFib/Issues/Issue137.hs:37-56
    sz = 3000
    interm = np.array([8 - (a % 17) for a in range(1, sz + 1)], I)
    ms = np.array([a // 8 for a in range(1, sz + 1)], I)
    inf = 10000
    infs = A.generate(A.index(384), lambda ix: A.tup(A.constant(inf), A.constant(inf)))
    inp = A.map(lambda v: A.tup(abs(v), A.constant(inf)), interm)
    msa = A.use(ms)

    def f(a, b):
        return A.cond(a[0] <= b[0], A.tup(a[0], A.min_(a[1], b[0])), A.tup(b[0], A.min_(b[1], a[0])))
    return A.permute(f, infs, lambda ix: A.Just_(A.index(msa[ix])), inp)


def _gather_if(frm, mask, pred, over, xs):
    # Test/NoFib/Issues/Issue185.hs:112-124
    g = A.zip(A.gather(frm, xs), over)
    pf = A.map(pred, mask)
    return A.zipWith(lambda ok, gv: A.cond(ok, gv[0], gv[1]), pf, g)


def _merge(e1, e2):
    # Test/NoFib/Issues/Issue228.hs:58-68
    return A.tup(e1[0] * e2[0], e1[0] * e2[1] + e1[1])


def _efloat_add(a, b):
    # Test/NoFib/Issues/Issue114.hs:52-59
    val = a[0] + b[0]
    det = val - a[0]
    err = a[0] - (val - det) + (b[0] - det) + a[1] + b[1]
    return A.tup(val, err)


def cases():
    vec10 = np.arange(10, dtype=I)
    mat5x10 = np.arange(50, dtype=I).reshape(5, 10)
    mat4x10 = np.arange(40, dtype=I).reshape(4, 10)
    xs3x5 = np.arange(15, dtype=I).reshape(3, 5)
    ys5x10 = np.arange(1, 51, dtype=I).reshape(5, 10)
    hist = np.array([0, 0, 1, 2, 1, 1, 2, 4, 8, 3, 4, 9, 8, 3, 2, 5, 5, 3, 1, 2], I)
    hu = A.use(hist)
    mss_in = np.array([-2, 1, -3, 4, -1, 2, 1, -5, 4, 0], I)
    m34 = np.array([1, 4, 3, 8, 0, 2, 8, 4, 7, 9, 8, 8], I).reshape(3, 4)
    to = np.array([1, 3, 7, 2, 5, 8], I)
    frm = np.array([1, 3, 7, 2, 5, 3], I)
    mask = np.array([3, 4, 9, 2, 7, 5], np.int32)
    zeros9 = np.zeros(9, I)
    in7 = np.array([1, 9, 6, 4, 4, 2, 5], I)
    in3 = np.array([1, 9, 6], I)
    in9 = np.array([1, 9, 6, 4, 4, 2, 0, 1, 2], I)
    gt4 = lambda v: v > 4  # noqa: E731
    matu = A.use(mat5x10)
    sp, ss = A.scanl_prime(add, 0, vec10)
    mp, ms = A.scanl_prime(add, 0, mat4x10)
    t4 = np.arange(10, dtype=I)
    efl = (np.full(100, 1.01, np.float32), np.zeros(100, np.float32))
    seg4 = np.array([1, 4, 0, 3], I)
    spr, sps = A.scanl_primeSeg(add, 0, mat5x10, seg4)
    rpr, rps = A.scanr_primeSeg(add, 0, mat5x10, seg4)
    c = {
        "generate_plus1": A.generate(A.index(10), lambda ix: ix[0] + 1),                              # Language.hs:288
        "map_plus1": A.map(lambda x: x + 1, vec10),                                                   # Language.hs:412-416
        "zipWith_plus": A.zipWith(add, xs3x5, ys5x10),                                                # Language.hs:430-446
        "fold_plus_42": A.fold(add, 42, mat5x10),                                                     # Language.hs:473-482
        "maximum_segment_sum": A.map(lambda t: t[0], A.fold1(_mss, A.map(lambda x: A.let_(A.max_(x, 0), lambda y: A.tup(y, y, y, x)), mss_in))),
        "scanl_vec": A.scanl(add, 10, vec10),                                                         # Language.hs:595-596
        "scanl_mat": A.scanl(add, 0, mat4x10),                                                        # Language.hs:599-600
        "scanl_prime_vec_res": sp, "scanl_prime_vec_sum": ss,                                         # Language.hs:623-627
        "scanl_prime_mat_res": mp, "scanl_prime_mat_sums": ms,                                        # Language.hs:630-638
        "scanl1_mat": A.scanl1(add, mat4x10),                                                         # Language.hs:653-654
        "permute_histogram": A.permute(add, A.fill(10, A.constant(0)), lambda ix: A.Just_(A.index(hu[ix])), A.fill(hu.shape, A.constant(1))),
        "permute_identity": A.permute(lambda a, b: a, A.fill(A.index(5, 5), A.constant(0)), lambda ix: A.Just_(A.index(ix[0], ix[0])),
                                      A.fill(A.index(5), A.constant(1))),                             # Language.hs:734-743
        "backpermute_transpose": A.backpermute(A.index(matu.shape[1], matu.shape[0]), lambda ix: A.index(ix[1], ix[0]), matu),
        "foldSeg_mat": A.foldSeg(add, 0, mat5x10, np.array([1, 4, 0, 3], I)),                         # Prelude.hs:689-702
        "scanlSeg_mat": A.scanlSeg(add, 0, mat5x10, seg4),                                            # Prelude.hs:954-977
        "scanl_primeSeg_res": spr, "scanl_primeSeg_sums": sps,                                        # Prelude.hs:1023-1050
        "scanl1Seg_mat": A.scanl1Seg(add, mat5x10, seg4),                                             # Prelude.hs:1121-1136
        "scanrSeg_mat": A.scanrSeg(add, 0, mat5x10, seg4),                                            # Prelude.hs:1183-1198
        "scanr_primeSeg_res": rpr, "scanr_primeSeg_sums": rps,                                        # Prelude.hs:1232-1257
        "scanr1Seg_mat": A.scanr1Seg(add, mat5x10, seg4),                                             # Prelude.hs:1296-1313
        "sum_mat": A.sum(np.arange(10, dtype=I).reshape(2, 5)),                                       # Prelude.hs:822-823
        "minimum_mat": A.minimum(m34), "maximum_mat": A.maximum(m34),                                 # Prelude.hs:849-877
        "gather": A.gather(frm, in9),                                                                 # Prelude.hs:1696-1698
        "scatter": A.scatter(to, A.fill(10, A.constant(0)), in7),                                     # Prelude.hs:1750-1752
        "issue137_ref1": _issue137(),
        "issue185_ref1": A.scatter(to, zeros9, in7),                                                  # Issue185.hs:49-54
        "issue185_ref2": A.scatter(to, zeros9, in3),                                                  # Issue185.hs:60-65
        "issue185_ref3": A.scatterIf(to, mask, gt4, zeros9, in7),                                     # Issue185.hs:71-80
        "issue185_ref4": A.scatterIf(to, mask, gt4, zeros9, in3),                                     # Issue185.hs:86-95
        "issue185_ref5": A.gather(frm, in9),                                                          # Issue185.hs:101-105
        "issue185_ref6": _gather_if(frm, mask, gt4, np.full(6, 6, I), in9),                           # Issue185.hs:111-124
        "issue228_ref1": A.fold(_merge, A.tup(1, 0), (np.array([1, 0, 1], I), np.array([1, 0, 1], I))),   # Issue228.hs:36-50
        "issue362_e1": A.scanl1(lambda x, y: A.tup(*[x[i] + y[i] for i in range(4)]), tuple([t4] * 4)),   # Issue362.hs:39-47
        "issue362_e2": A.scanl1(lambda x, y: A.tup(*[x[i] + y[i] for i in range(5)]), tuple([t4] * 5)),   # Issue362.hs:54-62
        "issue114_ref1": A.fold1(_efloat_add, efl),                                                    # Issue114.hs:61-77
    }
    return c


def _primes(n):
    # the sieve of Prelude.hs:2478-2508: awhile over (primes so far, upper bound), each trip expanding the
    # known primes into their multiples, knocking those out with a permute, filtering what is left
    n = A.constant(n)
    limit = A.truncate(A.sqrt(A.from_integral(n + 1, "f32")))

    def step(st):
        old, c = st
        c1 = A.the(c)
        c2 = A.cond(c1 < limit, c1 * c1, n + 1)
        sieves = A.compute(A.map(lambda v: v - c1, A.expand(lambda p: A.quot(c2 - p, p), lambda p, i: (2 + i) * p, old)))
        m = c2 - c1
        put = lambda ix: A.let_(sieves[ix], lambda s: A.cond(A.land(s >= 0, s < m), A.Just_(A.index(s)), A.Nothing_(1)))  # noqa: E731
        left = A.permute(lambda a, b: a, A.enumFromN(A.index(m), c1), put, A.fill(sieves.shape, A.constant(0)))
        return (A.append(old, A.filter_(lambda v: v > 0, left)[0]), A.unit(c2))
    return A.awhile(lambda st: A.map(lambda c: c < n + 1, st[1]), step, (A.use(np.zeros(0, I)), A.unit(A.constant(2))))[0]


def prelude_cases():
    """Further haddock examples of Language.hs and Prelude.hs: combinators the reference builds from
    the operations of the hot path (backpermute, generate, fold, scanl', permute), restated through the
    Python front end's own versions of them."""
    F = np.float32
    vec10 = np.arange(10, dtype=I)
    mat5x10 = np.arange(50, dtype=I).reshape(5, 10)
    cube = np.arange(60, dtype=I).reshape(3, 4, 5)
    box = np.arange(30, dtype=I).reshape(2, 3, 5)
    evens = np.array([1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 1, 1, 1, 1, 1, 2, 2, 2, 2, 2, 2, 4, 6, 8, 10, 12, 14, 16, 18, 20,
                      1, 3, 5, 7, 9, 11, 13, 15, 17, 19], I).reshape(4, 10)
    even = lambda v: (v % 2).eq(0)  # noqa: E731
    odd = lambda v: (v % 2).ne(0)  # noqa: E731
    one10 = np.arange(1, 11, dtype=I)
    m10x3 = np.arange(30, dtype=I).reshape(10, 3)
    m10x5 = np.arange(50, dtype=I).reshape(10, 5)
    fv, fc = A.filter_(even, one10)
    mv, mc = A.filter_(odd, evens)
    gt4 = lambda v: v > 4  # noqa: E731
    return {
        "replicate_rows": A.replicate((4, A.All), vec10),                                             # Language.hs:196
        "replicate_cols": A.replicate((A.All, 4), vec10),                                             # Language.hs:205
        "replicate_two": A.replicate((2, A.All, 3), vec10),                                           # Language.hs:221
        "replicate_rep0_unit": A.replicate((10,), A.unit(A.constant(42))),                            # Language.hs:228-235
        "replicate_rep0_vec": A.replicate((A.All, 5), vec10),                                         # Language.hs:237
        "replicate_rep1_vec": A.replicate((5, A.All), vec10),                                         # Language.hs:252-257
        "generate_const": A.generate(A.index(3), lambda ix: A.constant(F(1.2))),                      # Language.hs:278
        "fill_3": A.fill(A.index(3), F(1.2)),                                                         # Language.hs:283
        "slice_row": A.slice(mat5x10, (2, A.All)),                                                    # Language.hs:352
        "slice_point": A.slice(mat5x10, (4, 2)),                                                      # Language.hs:358
        "slice_sl0_vec": A.slice(vec10, (4,)),                                                        # Language.hs:365-372
        "slice_sl0_mat": A.slice(mat5x10, (A.All, 4)),                                                # Language.hs:375
        "slice_sl1_mat": A.slice(mat5x10, (4, A.All)),                                                # Language.hs:380-385
        "slice_sl1_cube": A.slice(cube, (A.All, 2, A.All)),                                           # Language.hs:388-392
        "indexed_vec": A.indexed(np.arange(5, dtype=F)),                                              # Prelude.hs:161-162
        "indexed_mat": A.indexed(np.arange(12, dtype=F).reshape(3, 4)),                               # Prelude.hs:165-166
        "zip_mats": A.zip(mat5x10, np.arange(50, dtype=F).reshape(10, 5)),                            # Prelude.hs:425-427
        "foldAll_vec": A.foldAll(add, F(42), np.arange(10, dtype=F)),                                 # Prelude.hs:656-657
        "foldAll_mat": A.foldAll(add, F(0), np.arange(50, dtype=F).reshape(5, 10)),                   # Prelude.hs:660-661
        "all_even": A.all_(even, evens), "any_even": A.any_(even, evens),                             # Prelude.hs:769-797
        "product_mat": A.product(np.arange(10, dtype=I).reshape(2, 5)),                               # Prelude.hs:834-835
        "prescanl_vec": A.prescanl(add, 0, one10),                                                    # Prelude.hs:895-896
        "postscanl_vec": A.postscanl(add, 42, one10),                                                 # Prelude.hs:912-913
        "fill_10": A.fill(A.index(10), F(0)),                                                         # Prelude.hs:1443
        "enumFromN_mat": A.enumFromN(A.index(5, 10), A.constant(0)),                                  # Prelude.hs:1452
        "enumFromStepN_mat": A.enumFromStepN(A.index(5, 10), F(0), F(0.5)),                           # Prelude.hs:1470
        "append_mats": A.append(mat5x10, m10x3),                                                      # Prelude.hs:1495-1518
        "concatOn_1": A.concatOn(1, mat5x10, m10x5), "concatOn_2": A.concatOn(2, mat5x10, m10x5),     # Prelude.hs:1541-1570
        "filter_even_vec_0": fv, "filter_even_vec_1": fc,                                             # Prelude.hs:1619-1624
        "filter_odd_mat_0": mv, "filter_odd_mat_1": mc,                                               # Prelude.hs:1626-1635
        "gatherIf": A.gatherIf(np.array([1, 3, 7, 2, 5, 3], I), np.array([3, 4, 9, 2, 7, 5], I), gt4, np.full(6, 6, F),
                               np.array([1, 9, 6, 4, 4, 2, 0, 1, 2], F)),                             # Prelude.hs:1719-1724
        "scatterIf": A.scatterIf(np.array([1, 3, 7, 2, 5, 8], I), np.array([3, 4, 9, 2, 7, 5], I), gt4, A.fill(10, A.constant(0)),
                                 np.array([1, 9, 6, 4, 4, 2, 5], I)),                                 # Prelude.hs:1774-1778
        "reverseOn_1": A.reverseOn(1, mat5x10), "reverseOn_2": A.reverseOn(2, mat5x10),               # Prelude.hs:1815-1838
        "transposeOn_mat": A.transposeOn(1, 2, mat5x10),                                              # Prelude.hs:1868
        "transposeOn_box_12": A.transposeOn(1, 2, box), "transposeOn_box_23": A.transposeOn(2, 3, box),
        "transposeOn_box_13": A.transposeOn(1, 3, box),                                               # Prelude.hs:1881-1892
        "take_5": A.take(5, mat5x10), "drop_7": A.drop(7, mat5x10),                                   # Prelude.hs:1925, 1952
        "init_mat": A.init(mat5x10), "tail_mat": A.tail(mat5x10),                                     # Prelude.hs:1978, 2004
        "primes_100": _primes(100),                                                                   # Prelude.hs:2478-2512
    }


ISSUE119 = json.load(open(os.path.join(HERE, "golden", "issue119.json")))


def _i119(key, dtype):
    v = ISSUE119[key]
    return np.array(v["values"], dtype=dtype).reshape(tuple(v["shape"]))


def _issue102():
    # Test/NoFib/Issues/Issue102.hs:36-63: a DFT written with reshape, replicate and fold
    p, lts, rts, rustride = 3, 1, 1, 1
    v = A.fill(A.index(p - 1), A.constant(2))
    ru = A.fill(A.index(p - 1), A.constant(1))
    x1 = A.reshape(A.index(lts, p - 1, rts), v)
    y = A.generate(A.index(lts, p, rts), lambda ix: A.cond(ix[1].eq(0), A.constant(0), x1[A.index(ix[0], ix[1] - 1, ix[2])]))
    y1 = A.reshape(A.index(lts, p, rts), A.flatten(y))
    dftrus = A.generate(A.index(p, p), lambda ix: ru[A.index((ix[0] * ix[1] * rustride) % p)])
    coeffs = A.compute(A.replicate((lts, A.All, rts, A.All), dftrus))
    inputs = A.generate(coeffs.shape, lambda ix: y1[A.index(ix[0], ix[3], ix[2])])
    ans = A.flatten(A.fold(add, A.constant(0), A.zipWith(lambda a, b: a * b, coeffs, inputs)))
    return A.reshape(A.use(y).shape, ans)


def _issue287_f(x, y):
    # Test/NoFib/Issues/Issue287.hs:52-64
    return A.tup(A.max_(x[0], x[5] + y[1]), x[1], x[2], y[3] * x[3], x[4], y[5])


def issue_cases():
    """More of the reference's regression tests (Test/NoFib/Issues/): `(term, expected)` with the expected
    value as the test states it (the literals of Issue102 and Issue119 come from the fixture files)."""
    out = {}
    out["issue102"] = (_issue102(), np.array(VECTORS["issue102_ref1"]["values"], I).reshape(1, 3, 1))
    # Issue119.hs:48-98: foldAll / fold of Int32 and Int64 matrices (sums that wrap in Int32)
    for k, dt in (("1", np.int32), ("2", np.int32), ("3", np.int64), ("4", np.int64)):
        out[f"issue119_{k}"] = (A.foldAll(add, dt(0), _i119(f"{k}_xs", dt)), _i119(f"{k}_ref", dt))
    out["issue119_5"] = (A.fold(add, np.int32(0), _i119("5_xs", np.int32)), _i119("5_ref", np.int32))
    # Issue119.hs:100-186: the six segmented scans over Int64 with Int32 segment descriptors
    seg = lambda k: _i119(f"{k}_seg", np.int32)  # noqa: E731
    xs = lambda k: _i119(f"{k}_xs", np.int64)  # noqa: E731
    out["issue119_6"] = (A.scanl1Seg(add, xs(6), seg(6)), _i119("6_ref", np.int64))
    out["issue119_7"] = (A.scanr1Seg(add, xs(7), seg(7)), _i119("7_ref", np.int64))
    out["issue119_8"] = (A.scanlSeg(add, np.int64(0), xs(8), seg(8)), _i119("8_ref", np.int64))
    out["issue119_9"] = (A.scanrSeg(add, np.int64(0), xs(9), seg(9)), _i119("9_ref", np.int64))
    p10, r10 = A.scanl_primeSeg(add, np.int64(0), xs(10), seg(10))
    out["issue119_10_ps"], out["issue119_10_rs"] = (p10, _i119("10_ps", np.int64)), (r10, _i119("10_rs", np.int64))
    p11, r11 = A.scanr_primeSeg(add, np.int64(0), xs(11), seg(11))
    out["issue119_11_ps"], out["issue119_11_rs"] = (p11, _i119("11_ps", np.int64)), (r11, _i119("11_rs", np.int64))
    out["issue123"] = (A.fold(add, 0, A.fill(A.index(100), A.constant(1))), np.array(100, I))        # Issue123.hs:30-41
    # Issue168.hs:29-58: iterate on tuples
    q1 = lambda t: A.tup(A.constant(np.float32(3)), t[0])  # noqa: E731
    d1 = A.tup(A.constant(np.float32(2)), A.constant(np.float32(1)))
    out["issue168_A"] = (A.fill(A.index(1), q1(d1)), (np.array([3], np.float32), np.array([2], np.float32)))
    out["issue168_B"] = (A.fill(A.index(1), A.iterate(1, q1, d1)), (np.array([3], np.float32), np.array([2], np.float32)))
    d3 = A.tup(*[A.constant(np.float32(v)) for v in (6, 5, 4, 3, 2, 1)])
    out["issue168_C"] = (A.fill(A.index(1), A.iterate(1, lambda t: A.tup(*[t[5 - k] for k in range(6)]), d3)),
                         tuple(np.array([v], np.float32) for v in (1, 2, 3, 4, 5, 6)))
    # Issue184.hs:36-63, Issue187.hs:31-52: what a conditional does not choose is not evaluated, so the
    # read at linear index -1 never happens
    v5 = A.use(np.array([1, 2, 3, 4, 5], I))
    want184 = np.zeros(1000, I)
    want184[:5] = [1, 4, 9, 16, 25]
    out["issue184_A"] = (A.generate(A.index(1000), lambda ix: A.cond(ix[0] < 5, A.let_(v5.linear(ix[0]), lambda y: y * y), A.constant(0))), want184)
    one = A.constant(1)
    out["issue184_B"] = (A.unit(A.or_(one.eq(1), v5.linear(-1).eq(1))), np.array(1, np.uint8))
    out["issue184_C"] = (A.unit(A.and_(one.ne(1), v5.linear(-1).eq(1))), np.array(0, np.uint8))
    out["issue187_A"] = (A.generate(A.index(), lambda ix: A.or_(one.eq(1), v5.linear(-1).eq(1))), np.array(1, np.uint8))
    x1 = A.unit(one)
    out["issue187_B"] = (A.generate(A.index(), lambda ix: A.or_(one.eq(A.the(x1)), A.let_(v5.linear(-1), lambda y: (y * y).eq(1)))),
                         np.array(1, np.uint8))
    # Issue287.hs:34-50: scans of six-component tuples of zeros stay zeros
    z6 = tuple(np.zeros(4, I) for _ in range(6))
    s22 = np.array([2, 2], I)
    out["issue287_A"] = (A.scanl1(_issue287_f, z6), z6)
    out["issue287_B"] = (A.scanl1Seg(lambda a, b: b, z6, s22), z6)
    out["issue287_C"] = (A.scanl1Seg(_issue287_f, z6, s22), z6)
    # Issue288.hs:29-37: a while whose condition is False from the start is the identity
    t10 = (np.arange(1, 11, dtype=I), np.arange(1, 11, dtype=I))
    out["issue288"] = (A.map(lambda e: A.while_(lambda _: A.constant(False), lambda v: v, e), t10), t10)
    # Issue407.hs:29-47
    for ty, dt in (("f32", np.float32), ("f64", np.float64)):
        with np.errstate(all="ignore"):
            fl = np.array([np.nan, -np.inf, np.nan, 0.1, np.inf, 0.5, np.inf], dt)
        out[f"issue407_isnan_{ty}"] = (A.map(A.is_nan, fl), np.array([1, 0, 1, 0, 0, 0, 0], np.uint8))
        out[f"issue407_isinf_{ty}"] = (A.map(A.is_infinite, fl), np.array([0, 1, 0, 0, 1, 0, 1], np.uint8))
        # Issue409.hs:29-50: y + tanh ((-y) * y) with y = recip x shared, at x = 1
        f409 = lambda x: A.let_(A.recip(x), lambda y: y + A.tanh((-y) * y))  # noqa: E731
        out[f"issue409_{ty}"] = (A.map(f409, np.array(1, dt)), np.array(dt(1) + np.tanh(dt(-1)), dt))
    # Issue436.hs:31-56: filter (const True) of take 3
    b5 = np.array([1, 0, 1, 0, 1], np.uint8)
    r1, n1 = A.filter_(lambda _: A.constant(True), A.take(3, b5))
    out["issue436_A_0"], out["issue436_A_1"] = (r1, np.array([1, 0, 1], np.uint8)), (n1, np.array(3, I))
    b55 = np.resize(np.array([1, 0], np.uint8), 25).reshape(5, 5)
    r2, n2 = A.filter_(lambda _: A.constant(True), A.take(3, b55))
    out["issue436_B_0"] = (r2, np.array([1, 0, 1, 0, 1, 0, 1, 0, 1, 0, 1, 0, 1, 0, 1], np.uint8))
    out["issue436_B_1"] = (n2, np.full(5, 3, I))
    # Issue439.hs:28-37
    out["issue439"] = (A.compute(A.map(lambda v: v * 2, A.compute(A.fill(A.index(), A.constant(np.float32(1)))))), np.array(2, np.float32))
    return out


def expected(key, got):
    """The reference's expected value in the layout `got` has (ndarray or tuple of leaves)."""
    v = VECTORS[key]
    shape = tuple(v["shape"])
    if isinstance(got, tuple):
        cols = list(zip(*v["values"]))
        return tuple(np.array(c, dtype=g.dtype).reshape(shape) for c, g in zip(cols, got))
    return np.array(v["values"], dtype=got.dtype).reshape(shape)


def extra_cases():
    """Known answers given in closed form by the reference's tests."""
    out = {}
    # Test/NoFib/Misc/Scanl1.hs:32-39: scanl1 (+) over [1..] of shape 257 x 31
    sh = (257, 31)
    arr = np.arange(1, sh[0] * sh[1] + 1, dtype=I).reshape(sh)
    i, j = np.indices(sh)
    intsum = lambda n, m: m * (m + 1) // 2 - (n - 1) * n // 2  # noqa: E731
    out["misc_scanl1"] = (A.scanl1(add, arr), intsum(1 + i * 31, 1 + i * 31 + j).astype(I))
    # Test/NoFib/Issues/Issue364.hs:52-54, 66-99: scanl of the interval monoid at sizes 64 and 65
    for n in (64, 65):
        for dt in (np.int8, np.int16, np.int32, np.int64, np.float32, np.float64):
            t = A.TY_OF_NP[np.dtype(dt)]
            one = A.tup(A.constant(dt(-1), t), A.constant(dt(-1), t))
            top = A.tup(A.constant(dt(-2), t), A.constant(dt(-2), t))

            def teq(x, y):
                return A.land(x[0].eq(y[0]), x[1].eq(y[1]))

            def iappend(x, y, one=one, top=top):
                return A.cond(teq(x, one), y, A.cond(teq(y, one), x, A.cond(A.lor(teq(x, top), teq(y, top)), top,
                              A.cond((x[1] + 1).eq(y[0]), A.tup(x[0], y[1]), top))))
            iv = np.arange(n).astype(dt)
            term = A.scanl(iappend, one, (iv, iv))
            exp = (np.concatenate([[-1], np.zeros(n)]).astype(dt), np.concatenate([[-1], np.arange(n)]).astype(dt))
            out[f"issue364_{t}_{n}"] = (term, exp)
    # Test/NoFib/Issues/Issue114.hs:79-84: compensated prefix sums (compared with the suite's Float tolerance)
    efl = (np.full(100, 1.01, np.float32), np.zeros(100, np.float32))
    exp = (np.array([1.01 * k for k in range(1, 101)], np.float32), np.zeros(100, np.float32))
    out["issue114_ref2"] = (A.scanl1(_efloat_add, efl), exp)
    # Test/NoFib/Misc/Cache.hs:43-73: two kernels that differ only in the expression computing their
    # extent (host-side, not part of the kernel) and in which arrays that expression mentions; a kernel
    # cache that ignores the extent must still pass the right parameters to each
    a10 = A.use(np.arange(10, dtype=np.float32))
    b10 = A.use(np.arange(10, 20, dtype=np.float32))
    c = A.compute(A.generate(A.index(a10.shape[0] + b10.shape[0]), lambda ix: a10[A.index(A.rem(ix[0], 10))]))
    d = A.compute(A.generate(A.index(3 * a10.shape[0]), lambda ix: a10[A.index(A.rem(ix[0], 10))]))
    out["misc_cache_generate"] = (A.zipWith(add, A.sum_(c), A.sum_(d)), np.array(5 * 45, np.float32))
    c = A.compute(A.backpermute(A.index(A.min_(a10.shape[0], b10.shape[0])), lambda ix: ix, a10))
    d = A.compute(A.backpermute(A.index(a10.shape[0]), lambda ix: ix, a10))
    out["misc_cache_backpermute"] = (A.zipWith(add, A.sum_(c), A.sum_(d)), np.array(2 * 45, np.float32))
    # Test/NoFib/Issues/Issue93.hs:30-37
    xs = np.array([[5]], I)
    out["issue93"] = (A.permute(lambda c, _: c, A.fill(A.use(xs).shape, A.constant(0)), lambda ix: A.Just_(ix), xs), xs)
    return out
