"""List-and-loop references for stencils, in the manner of the reference's own test
oracle for its backends (Test/NoFib/Prelude/Stencil.hs): ``stencil3Ref`` ... ``stencil9Ref``,
``stencil3x3Ref`` ... ``stencil9x9Ref``, ``stencil3x3x3Ref`` (:442-634) build, for every output
index, the neighbourhood as nested tuples (outermost dimension outermost, offsets -r..+r) by
asking ``bound`` (:637-669) for every tap, and hand it to the stencil function; the random
"patterns" (:350-438) are sums over a random subsequence of the taps of every innermost row.

Plain Python loops over lists on purpose: nothing here shares code or idiom (padding,
slicing) with the oracle or the kernels it is used to check.
"""
import itertools


def bound(bnd, sh, ix):
    """Stencil.hs:637-669.  ``bnd``: "clamp" | "mirror" | "wrap" | ("constant", e).
    Returns ("value", e) for a constant boundary hit in any dimension, else ("index", ix')."""
    out = []
    for sz, i in zip(sh, ix):
        if i < 0:
            if bnd == "clamp":
                out.append(0)
            elif bnd == "mirror":
                out.append(-i)
            elif bnd == "wrap":
                out.append(sz + i)
            else:
                return ("value", bnd[1])
        elif i >= sz:
            if bnd == "clamp":
                out.append(sz - 1)
            elif bnd == "mirror":
                out.append(sz - (i - sz + 2))
            elif bnd == "wrap":
                out.append(i - sz)
            else:
                return ("value", bnd[1])
        else:
            out.append(i)
    return ("index", tuple(out))


def _at(nested, ix):
    for i in ix:
        nested = nested[i]
    return nested


def neighbourhood(arr, sh, bnd, ix, extent):
    """Nested tuples of the taps around ``ix``: extent[d] taps in dimension d, outermost first."""
    def go(d, prefix):
        if d == len(sh):
            kind, v = bound(bnd, sh, prefix)
            return v if kind == "value" else _at(arr, v)
        r = extent[d] // 2
        return tuple(go(d + 1, prefix + (ix[d] + o,)) for o in range(-r, r + 1))
    return go(0, ())


def stencil_ref(st, bnd, arr, sh, extent):
    """``stencil<extent>Ref st bnd arr`` as nested lists of shape ``sh``."""
    def build(d, prefix):
        if d == len(sh):
            return st(neighbourhood(arr, sh, bnd, prefix, extent))
        return [build(d + 1, prefix + (i,)) for i in range(sh[d])]
    return build(0, ())


def stencil2_ref(st, bnd1, arr1, sh1, ext1, bnd2, arr2, sh2, ext2):
    """Two neighbourhoods per point of the intersection of the two shapes (Interpreter.hs:652-668)."""
    sh = tuple(min(a, b) for a, b in zip(sh1, sh2))

    def build(d, prefix):
        if d == len(sh):
            return st(neighbourhood(arr1, sh1, bnd1, prefix, ext1), neighbourhood(arr2, sh2, bnd2, prefix, ext2))
        return [build(d + 1, prefix + (i,)) for i in range(sh[d])]
    return build(0, ())


def random_pattern(rnd, extent):
    """Which taps of every innermost row take part (pattern3 ... pattern3x3x3, :350-438): one
    subsequence of range(extent[-1]) per row, nested like the outer dimensions."""
    def go(d):
        if d == len(extent) - 1:
            return [k for k in range(extent[d]) if rnd.random() < 0.5]
        return [go(d + 1) for _ in range(extent[d])]
    return go(0)


def apply_pattern(pattern, nb, zero, depth):
    """Sum of the chosen taps, rows summed in order (the reference sums the rows' sums)."""
    if depth == 1:
        acc = zero
        for k in pattern:
            acc = acc + nb[k]
        return acc
    acc = zero
    for p, sub in zip(pattern, nb):
        acc = acc + apply_pattern(p, sub, zero, depth - 1)
    return acc
