"""Host-side mirror of the reference's array-language interface for the hot path.

The reference's front end (``Data.Array.Accelerate.Language`` /
``Data.Array.Accelerate.Prelude``) is a Haskell EDSL whose terms go through
sharing recovery and fusion (``Data/Array/Accelerate/Trafo.hs:63-85``) before
a backend sees them.  No Haskell toolchain exists where this backend is built
and tested, so this module provides the same operators with the same argument
order and meaning in Python, and produces the *post-fusion* form directly:

* producers (``generate``/``map``/``zipWith``/``backpermute``/``fill`` ...) stay
  *delayed* (an extent expression plus an index function) and are embedded into
  their consumer, as ``Trafo/Fusion.hs:161-216`` arranges;
* consumers (``fold*``, ``scan*``, ``permute``, ``stencil*``) become manifest
  nodes of the program text handed to the backend.

The result of building a term is the S-expression program text that both the
B200 backend (``accelerate_b200.backend``) and the CPU oracle accept.
"""
from __future__ import annotations

import itertools
import re
import numpy as np

# ----------------------------------------------------------------------------
# Types.  Scalars are strings; tuples are Python tuples of types.
# ``Int`` is 64-bit (Array/Data.hs:380-384); ``Bool`` is a Word8 tag.
# ----------------------------------------------------------------------------
SCALARS = ("i8", "i16", "i32", "i64", "u8", "u16", "u32", "u64", "f32", "f64", "f16")
NP_OF = {
    "i8": np.int8, "i16": np.int16, "i32": np.int32, "i64": np.int64,
    "u8": np.uint8, "u16": np.uint16, "u32": np.uint32, "u64": np.uint64,
    "f32": np.float32, "f64": np.float64, "f16": np.float16,   # Half (Type.hs:127)
}
TY_OF_NP = {np.dtype(v): k for k, v in NP_OF.items()}
TY_OF_NP[np.dtype(np.bool_)] = "u8"
INT, BOOL = "i64", "u8"


def is_float(t):
    return t in ("f32", "f64", "f16")


def is_scalar(t):
    return isinstance(t, str)


def vec(n, t):
    """``Vec n t`` (Type.hs:140-152), n in 2, 3, 4, 8, 16.  To this module it is one opaque element type:
    an ndarray of such elements has one more, innermost, axis of length n, the reference's layout for it
    (Array/Data.hs:108-119); ``vec_unpack`` / ``vec_pack`` convert to and from the tuple of components."""
    if n not in (2, 3, 4, 8, 16) or t not in SCALARS:
        raise TypeError("vec(n, t): n in 2, 3, 4, 8, 16 and t a scalar type")
    return f"(vec {n} {t})"


def vec_parts(t):
    """``(n, component type)`` of a vector type, else None."""
    if isinstance(t, str) and t.startswith("(vec "):
        _, n, c = t[1:-1].split()
        return int(n), c
    return None


def ty_sx(t):
    if is_scalar(t):
        return t
    return "(tup" + "".join(" " + ty_sx(c) for c in t) + ")"


def flatten_ty(t):
    if is_scalar(t):
        return [t]
    out = []
    for c in t:
        out += flatten_ty(c)
    return out


def shape_ty(rank):
    return tuple([INT] * rank)


_counter = itertools.count()


def _fresh(prefix):
    return f"{prefix}{next(_counter)}"


def reset_names():
    """Restart name generation (makes program text deterministic per trace)."""
    global _counter
    _counter = itertools.count()


# ----------------------------------------------------------------------------
# Scalar expressions (AST.hs:524-645 OpenExp; primitives AST.hs:661-753)
# ----------------------------------------------------------------------------
def _lit(t, v):
    if is_float(t):
        f = float(np.float32(v)) if t == "f32" else (float(np.float16(v)) if t == "f16" else float(v))
        if f != f:
            s = "nan"
        elif f in (float("inf"), float("-inf")):
            s = "inf" if f > 0 else "-inf"
        else:
            s = f.hex()
        return f"(const {t} {s})"
    return f"(const {t} {int(NP_OF[t](v))})"


class Exp:
    """A typed scalar expression.  ``deps`` are the manifest arrays it reads."""

    __slots__ = ("ty", "sx", "deps", "parts")
    __array_priority__ = 1000

    def __init__(self, ty, sx, deps=frozenset(), parts=None):
        self.ty, self.sx, self.deps, self.parts = ty, sx, frozenset(deps), parts

    # -- tuples ------------------------------------------------------------
    def __getitem__(self, i):
        if is_scalar(self.ty):
            raise TypeError("projection from a scalar expression")
        if self.parts is not None:
            return self.parts[i]
        return Exp(self.ty[i], f"(prj {i} {self.sx})", self.deps)

    def __len__(self):
        if is_scalar(self.ty):
            raise TypeError("scalar expression has no length")
        return len(self.ty)

    def __iter__(self):
        return (self[i] for i in range(len(self)))

    # -- arithmetic --------------------------------------------------------
    def _bin(self, op, other, swap=False, result=None):
        o = lift(other, self.ty)
        a, b = (o, self) if swap else (self, o)
        if a.ty != b.ty:
            raise TypeError(f"{op}: operand types differ: {a.ty} vs {b.ty}")
        return Exp(result or a.ty, f"(prim {op} {a.ty} {a.sx} {b.sx})", a.deps | b.deps)

    def _un(self, op, result=None):
        return Exp(result or self.ty, f"(prim {op} {self.ty} {self.sx})", self.deps)

    def __add__(self, o): return self._bin("add", o)
    def __radd__(self, o): return self._bin("add", o, True)
    def __sub__(self, o): return self._bin("sub", o)
    def __rsub__(self, o): return self._bin("sub", o, True)
    def __mul__(self, o): return self._bin("mul", o)
    def __rmul__(self, o): return self._bin("mul", o, True)
    def __neg__(self): return self._un("neg")
    def __abs__(self): return self._un("abs")
    def __truediv__(self, o): return self._bin("fdiv", o)
    def __rtruediv__(self, o): return self._bin("fdiv", o, True)
    def __floordiv__(self, o): return self._bin("idiv", o)      # Haskell `div`
    def __mod__(self, o): return self._bin("mod", o)            # Haskell `mod`
    def __and__(self, o): return self._bin("band", o)
    def __or__(self, o): return self._bin("bor", o)
    def __xor__(self, o): return self._bin("bxor", o)
    def __invert__(self): return self._un("bnot")
    def __lshift__(self, o): return _shift("shl", self, o)
    def __rshift__(self, o): return _shift("shr", self, o)
    def __pow__(self, o): return self._bin("fpow", o)
    def __lt__(self, o): return self._bin("lt", o, result=BOOL)
    def __gt__(self, o): return self._bin("gt", o, result=BOOL)
    def __le__(self, o): return self._bin("le", o, result=BOOL)
    def __ge__(self, o): return self._bin("ge", o, result=BOOL)
    def eq(self, o): return self._bin("eq", o, result=BOOL)
    def ne(self, o): return self._bin("ne", o, result=BOOL)
    __hash__ = object.__hash__

    def __bool__(self):
        raise TypeError("an embedded expression has no Python truth value; use cond()")


def _shift(op, a, n):
    n = lift(n, INT)
    return Exp(a.ty, f"(prim {op} {a.ty} {a.sx} {n.sx})", a.deps | n.deps)


def constant(v, ty=None):
    """``constant`` (Smart.hs): embed a host value."""
    if isinstance(v, Exp):
        return v
    if isinstance(v, tuple):
        tys = ty if ty is not None else [None] * len(v)
        return tup(*[constant(x, t) for x, t in zip(v, tys)])
    if ty is None:
        if isinstance(v, (bool, np.bool_)):
            ty = BOOL
        elif isinstance(v, (int, np.integer)) and not isinstance(v, np.generic):
            ty = INT
        elif isinstance(v, float):
            ty = "f64"
        else:
            ty = TY_OF_NP[np.dtype(type(v))]
    return Exp(ty, _lit(ty, v))


def lift(v, ty):
    """Embed ``v`` at type ``ty`` unless it is an expression already."""
    if isinstance(v, Exp):
        return v
    if isinstance(v, tuple):
        return tup(*[lift(x, t) for x, t in zip(v, ty)])
    return Exp(ty, _lit(ty, v))


def tup(*xs):
    xs = [x if isinstance(x, Exp) else constant(x) for x in xs]
    deps = frozenset().union(*[x.deps for x in xs]) if xs else frozenset()
    return Exp(tuple(x.ty for x in xs), "(tup" + "".join(" " + x.sx for x in xs) + ")", deps, parts=list(xs))


def index(*ix):
    """``Z :. i :. j`` — outermost first, innermost last."""
    return tup(*[lift(i, INT) for i in ix])


index0 = index()


def let_(e, body):
    """Explicit sharing of a scalar sub-expression."""
    v = _fresh("v")
    r = body(Exp(e.ty, f"(var {v})", e.deps))
    return Exp(r.ty, f"(let {v} {e.sx} {r.sx})", e.deps | r.deps)


def cond(c, t, e):
    t = t if isinstance(t, Exp) else constant(t)
    e = lift(e, t.ty)
    if t.ty != e.ty:
        raise TypeError("cond: branch types differ")
    return Exp(t.ty, f"(cond {c.sx} {t.sx} {e.sx})", c.deps | t.deps | e.deps)


def while_(p, f, x):
    x = x if isinstance(x, Exp) else constant(x)
    pv, fv = _fresh("v"), _fresh("v")
    pe = p(Exp(x.ty, f"(var {pv})"))
    fe = f(Exp(x.ty, f"(var {fv})"))
    sx = (f"(while (lam (({pv} {ty_sx(x.ty)})) {pe.sx}) (lam (({fv} {ty_sx(x.ty)})) {fe.sx}) {x.sx})")
    return Exp(x.ty, sx, x.deps | pe.deps | fe.deps)


def _prim1(op):
    def f(x):
        return x._un(op)
    f.__name__ = op
    return f


for _n in ("sin cos tan asin acos atan sinh cosh tanh asinh acosh atanh exp sqrt log recip").split():
    globals()[_n] = _prim1(_n)
signum = _prim1("sig")


def iterate(n, f, z):
    """``iterate n f z`` (Prelude.hs:2320-2328): ``f`` applied ``n`` times, as a ``while`` over (count, value)."""
    z = z if isinstance(z, Exp) else constant(z)
    n = lift(n, INT)
    return while_(lambda v: v[0] < n, lambda v: tup(v[0] + 1, f(v[1])), tup(constant(0), z))[1]


def is_nan(x): return x._un("isnan", BOOL)
def is_infinite(x): return x._un("isinf", BOOL)
def pop_count(x): return x._un("popcount", INT)
def count_leading_zeros(x): return x._un("clz", INT)
def count_trailing_zeros(x): return x._un("ctz", INT)
def quot(a, b): return a._bin("quot", b)
def rem(a, b): return a._bin("rem", b)
def div(a, b): return a._bin("idiv", b)
def mod(a, b): return a._bin("mod", b)
def atan2(a, b): return a._bin("atan2", b)
def log_base(b, x):
    b = b if isinstance(b, Exp) else lift(b, x.ty)
    return b._bin("logbase", x)
def rotate_l(a, n): return _shift("rotl", a, n)
def rotate_r(a, n): return _shift("rotr", a, n)


def max_(a, b):
    a = a if isinstance(a, Exp) else lift(a, b.ty)
    return a._bin("max", b)


def min_(a, b):
    a = a if isinstance(a, Exp) else lift(a, b.ty)
    return a._bin("min", b)


def land(a, b): return Exp(BOOL, f"(prim land u8 {a.sx} {b.sx})", a.deps | b.deps)
def lor(a, b): return Exp(BOOL, f"(prim lor u8 {a.sx} {b.sx})", a.deps | b.deps)
def lnot(a): return Exp(BOOL, f"(prim lnot u8 {a.sx})", a.deps)


def and_(a, b):
    """``(&&)`` (Classes/Eq.hs:57-62): a conditional, so the second operand is evaluated only when the
    first holds (``land`` is the strict ``(&&!)``)."""
    return cond(a, b, Exp(BOOL, "(const u8 0)"))


def or_(a, b):
    """``(||)`` (Classes/Eq.hs:78-83): the second operand is evaluated only when the first fails."""
    return cond(a, Exp(BOOL, "(const u8 1)"), b)


def _conv(op, x, to):
    return Exp(to, f"(prim {op} {x.ty} {to} {x.sx})", x.deps)


def vec_unpack(x):
    """``unpackVec{2,3,4,..}'`` / VecUnpack (AST.hs:570-573): the vector's components as a tuple."""
    n, c = vec_parts(x.ty)
    return Exp(tuple([c] * n), f"(vecunpack {n} {c} {x.sx})", x.deps)


def vec_pack(*xs):
    """VecPack (AST.hs:566-569): n equally typed scalars (or one n-tuple) as a vector."""
    x = xs[0] if len(xs) == 1 and isinstance(xs[0], Exp) else tup(*xs)
    n, c = len(x.ty), x.ty[0]
    if any(t != c for t in x.ty):
        raise TypeError("vec_pack: components differ in type")
    return Exp(vec(n, c), f"(vecpack {n} {c} {x.sx})", x.deps)


def from_integral(x, to): return _conv("fromintegral", x, to)
def to_floating(x, to): return _conv("tofloating", x, to)
def truncate(x, to=INT): return _conv("truncate", x, to)
def round_(x, to=INT): return _conv("round", x, to)
def floor(x, to=INT): return _conv("floor", x, to)
def ceiling(x, to=INT): return _conv("ceiling", x, to)
def min_bound(t): return Exp(t, f"(minbound {t})")
def max_bound(t): return Exp(t, f"(maxbound {t})")
def pi(t): return Exp(t, f"(pi {t})")
def bitcast(x, to): return Exp(to, f"(coerce {x.ty} {to} {x.sx})", x.deps)
def undef(t): return Exp(t, f"(undef {ty_sx(t)})")


def Just_(ix):
    """``Just_ ix`` as the PrimMaybe encoding (tag, ix)  (AST.hs:201-202)."""
    ix = ix if isinstance(ix, Exp) else index(*ix)
    return tup(Exp(BOOL, "(const u8 1)"), ix)


def Nothing_(rank):
    return tup(Exp(BOOL, "(const u8 0)"), undef(shape_ty(rank)))


def shape_size(sh): return Exp(INT, f"(shapesize {sh.sx})", sh.deps)
def to_index(sh, ix): return Exp(INT, f"(toindex {sh.sx} {ix.sx})", sh.deps | ix.deps)
def from_index(sh, i):
    i = lift(i, INT)
    return Exp(sh.ty, f"(fromindex {sh.sx} {i.sx})", sh.deps | i.deps)


def _lam(params, body):
    ps = " ".join(f"({n} {ty_sx(t)})" for n, t in params)
    return f"(lam ({ps}) {body.sx})"


def _fun(f, *tys):
    """Reify a Python function over expressions as ``(lam ...)`` text."""
    names = [_fresh("v") for _ in tys]
    args = [Exp(t, f"(var {n})") for n, t in zip(names, tys)]
    body = f(*args)
    if not isinstance(body, Exp):
        body = tup(*body) if isinstance(body, tuple) else constant(body)
    return _lam(list(zip(names, tys)), body), body


# ----------------------------------------------------------------------------
# Arrays
# ----------------------------------------------------------------------------
class Node:
    """A manifest array (program input or an executed node)."""

    def __init__(self, kind, rank, elt, sx=None, deps=(), nouts=1, data=None):
        self.kind, self.rank, self.elt, self.sx = kind, rank, elt, sx
        self.deps = list(deps)
        self.nouts = nouts
        self.names = [_fresh("a") for _ in range(nouts)]
        self.data = data        # inputs: (shape, [leaf ndarrays]) or None for a parameter
        self.out_ranks = [rank]
        self.out_elts = [elt]


class Acc:
    """An array term: manifest (``node``) or delayed (``extent`` + ``fn``)."""

    def __init__(self, rank, elt, node=None, out=0, extent=None, fn=None):
        self.rank, self.elt, self.node, self.out = rank, elt, node, out
        self._extent, self._fn = extent, fn

    @property
    def manifest(self):
        return self.node is not None

    @property
    def name(self):
        return self.node.names[self.out]

    # shape / indexing -----------------------------------------------------
    @property
    def shape(self):
        if self.manifest:
            return Exp(shape_ty(self.rank), f"(shape {self.name})", {self.node})
        return self._extent

    def size(self):
        return shape_size(self.shape)

    def __getitem__(self, ix):
        """``arr ! ix``"""
        if not isinstance(ix, Exp):
            ix = index(*ix) if isinstance(ix, tuple) else index(ix)
        if self.manifest:
            return Exp(self.elt, f"(index {self.name} {ix.sx})", ix.deps | {self.node})
        return self._fn(ix)

    def linear(self, i):
        """``arr !! i``"""
        i = lift(i, INT)
        if self.manifest:
            return Exp(self.elt, f"(lindex {self.name} {i.sx})", i.deps | {self.node})
        return self._fn(from_index(self.shape, i))

    def operand(self):
        """Text of this array as a consumer's operand, plus its dependencies."""
        if self.manifest:
            return f"(manifest {self.name})", {self.node}
        lam, body = _fun(self._fn, shape_ty(self.rank))
        return f"(delayed {self._extent.sx} {lam})", body.deps | self._extent.deps


def use(a, elt=None):
    """``use``: embed host array(s).  A tuple/list of equal-shape ndarrays is an
    array of tuples in struct-of-arrays form (Array/Data.hs:95-98)."""
    if isinstance(a, Acc):
        return a
    if isinstance(a, (tuple, list)):
        leaves = [np.asarray(x, order="C") for x in a]          # (keeps a 0-d array a Scalar)
        if elt is None:
            elt = tuple(TY_OF_NP[x.dtype] for x in leaves)
    else:
        a = np.asarray(a, order="C")
        leaves = [a.view(np.uint8) if a.dtype == np.bool_ else a]
        elt = elt or TY_OF_NP[a.dtype]
    sh = tuple(int(d) for d in leaves[0].shape)
    if vec_parts(elt):
        # the ndarray's last axis holds the components: it is no dimension of the array of vectors
        n, c = vec_parts(elt)
        if isinstance(a, (tuple, list)) or not sh or sh[-1] != n or TY_OF_NP[leaves[0].dtype] != c:
            raise TypeError(f"use: an array of {elt} is one ndarray of {c} whose last axis has length {n}")
        node = Node("in", len(sh) - 1, elt, data=(sh, leaves))
        return Acc(len(sh) - 1, elt, node=node)
    node = Node("in", len(sh), elt, data=(sh, leaves))
    return Acc(len(sh), elt, node=node)


def param(rank, elt):
    """An array parameter of a program (bound at run time)."""
    return Acc(rank, elt, node=Node("in", rank, elt))


def _mk(kind, rank, elt, sx, deps, nouts=1, ranks=None, elts=None):
    node = Node(kind, rank, elt, sx=sx, deps=[d for d in deps], nouts=nouts)
    if ranks:
        node.out_ranks, node.out_elts = ranks, elts
    return node


def _shape_exp(sh, rank=None):
    if isinstance(sh, Exp):
        return sh
    if isinstance(sh, int):
        sh = (sh,)
    return index(*sh)


def intersect(a, b):
    """Shape.hs:81-91"""
    if a.sx == b.sx:
        return a
    return tup(*[min_(x, y) for x, y in zip(a, b)])


# producers (stay delayed) ----------------------------------------------------
def generate(sh, f, elt=None):
    sh = _shape_exp(sh)
    rank = len(sh.ty)
    if elt is None:
        probe = f(Exp(shape_ty(rank), "(var _probe)"))
        probe = probe if isinstance(probe, Exp) else (tup(*probe) if isinstance(probe, tuple) else constant(probe))
        elt = probe.ty

    def fn(ix):
        r = f(ix)
        return r if isinstance(r, Exp) else (tup(*r) if isinstance(r, tuple) else lift(r, elt))
    return Acc(rank, elt, extent=sh, fn=fn)


def fill(sh, v):
    v = v if isinstance(v, Exp) else constant(v)
    return generate(sh, lambda ix: v, v.ty)


def map_(f, a):
    a = use(a)
    return generate(a.shape, lambda ix: f(a[ix]))


def zipWith(f, a, b):
    a, b = use(a), use(b)
    return generate(intersect(a.shape, b.shape), lambda ix: f(a[ix], b[ix]))


def _zip_with_n(f, *xs):
    """zipWith3, zipWith4 (Prelude.hs:316-349): the extent is the intersection of all operands'."""
    xs = [use(x) for x in xs]
    sh = xs[0].shape
    for x in xs[1:]:
        sh = intersect(sh, x.shape)
    return generate(sh, lambda ix: f(*[x[ix] for x in xs]))


def zipWith3(f, a, b, c):
    return _zip_with_n(f, a, b, c)


def zipWith4(f, a, b, c, d):
    return _zip_with_n(f, a, b, c, d)


def zip_(a, b):
    return zipWith(lambda x, y: tup(x, y), a, b)


def backpermute(sh, p, a):
    a = use(a)

    def fn(ix):
        j = p(ix)
        return a[j if isinstance(j, Exp) else index(*j)]
    return generate(_shape_exp(sh), fn, a.elt)


def enumFromN(sh, x):
    sh = _shape_exp(sh)
    x = x if isinstance(x, Exp) else constant(x)
    return generate(sh, lambda ix: x + from_integral(to_index(sh, ix), x.ty) if x.ty != INT else x + to_index(sh, ix), x.ty)


def reshape(sh, a):
    a = compute(use(a))
    sh = _shape_exp(sh)
    node = _mk("reshape", len(sh.ty), a.elt, f"(reshape {sh.sx} {a.name})", sh.deps | {a.node})
    return Acc(len(sh.ty), a.elt, node=node)


def compute(a):
    """Force a delayed array to be materialised (``compute``, Prelude.hs:2177)."""
    a = use(a)
    if a.manifest:
        return a
    lam, body = _fun(a._fn, shape_ty(a.rank))
    sx = f"(generate {ty_sx(a.elt)} {a._extent.sx} {lam})"
    node = _mk("generate", a.rank, a.elt, sx, body.deps | a._extent.deps)
    return Acc(a.rank, a.elt, node=node)


def unit(e):
    e = e if isinstance(e, Exp) else constant(e)
    return generate(index0, lambda ix: e, e.ty)


def the(a):
    return use(a)[index0]


# consumers (manifest nodes) -------------------------------------------------
def _fold_like(kind, f, z, a, seg=None):
    a = use(a)
    lam, fb = _fun(f, a.elt, a.elt)
    op, deps = a.operand()
    deps = deps | fb.deps
    zs = ""
    if z is not None:
        z = lift(z, a.elt)
        zs = " " + z.sx
        deps = deps | z.deps
    extra = ""
    if seg is not None:
        sop, sdeps = seg.operand()
        extra = " " + sop
        deps = deps | sdeps
    return f"({kind} {ty_sx(a.elt)} {lam}{zs} {op}{extra})", deps, a


def fold(f, z, a):
    """``fold`` (Language.hs:523): reduce the innermost dimension."""
    sx, deps, a = _fold_like("fold", f, z, a)
    return Acc(a.rank - 1, a.elt, node=_mk("fold", a.rank - 1, a.elt, sx, deps))


def fold1(f, a):
    """``fold1`` (Language.hs:541)."""
    return fold(f, None, a)


def foldSeg_(f, z, a, offsets):
    """``foldSeg'`` (Language.hs:561): the descriptor holds segment OFFSETS."""
    offsets = use(offsets)
    sx, deps, a = _fold_like("foldseg", f, z, a, seg=offsets)
    return Acc(a.rank, a.elt, node=_mk("foldseg", a.rank, a.elt, sx, deps))


def fold1Seg_(f, a, offsets):
    return foldSeg_(f, None, a, offsets)


def foldSeg(f, z, a, lengths):
    """``foldSeg`` (Prelude.hs:710-717): lengths are turned into offsets with
    ``scanl (+) 0``."""
    lengths = use(lengths)
    return foldSeg_(f, z, a, scanl(lambda x, y: x + y, lift(0, lengths.elt), lengths))


def fold1Seg(f, a, lengths):
    """``fold1Seg`` (Prelude.hs:737-743)."""
    lengths = use(lengths)
    return fold1Seg_(f, a, scanl(lambda x, y: x + y, lift(0, lengths.elt), lengths))


def _scan(kind, f, z, a):
    sx, deps, a = _fold_like(kind, f, z, a)
    return Acc(a.rank, a.elt, node=_mk(kind, a.rank, a.elt, sx, deps))


def scanl(f, z, a): return _scan("scanl", f, z, a)      # Language.hs:607
def scanl1(f, a): return _scan("scanl", f, None, a)     # Language.hs:660
def scanr(f, z, a): return _scan("scanr", f, z, a)      # Language.hs:673
def scanr1(f, a): return _scan("scanr", f, None, a)     # Language.hs:690


def _scan_prime(kind, f, z, a):
    sx, deps, a = _fold_like(kind, f, z, a)
    node = _mk(kind, a.rank, a.elt, sx, deps, nouts=2, ranks=[a.rank, a.rank - 1], elts=[a.elt, a.elt])
    return Acc(a.rank, a.elt, node=node, out=0), Acc(a.rank - 1, a.elt, node=node, out=1)


def scanl_prime(f, z, a): return _scan_prime("scanl'", f, z, a)   # scanl', Language.hs:640
def scanr_prime(f, z, a): return _scan_prime("scanr'", f, z, a)   # scanr', Language.hs:683


def permute(f, defaults, p, a):
    """``permute`` (Language.hs:792): ``f new old``; ``p`` returns ``Just_ ix`` /
    ``Nothing_``.  The defaults are always manifest (Fusion.hs:213)."""
    a = use(a)
    defaults = compute(use(defaults))
    lam, fb = _fun(f, a.elt, a.elt)

    def pf(ix):
        r = p(ix)
        return r
    plam, pb = _fun(pf, shape_ty(a.rank))
    op, deps = a.operand()
    deps = deps | fb.deps | pb.deps | {defaults.node}
    sx = f"(permute {ty_sx(a.elt)} {lam} {defaults.name} {plam} {op})"
    return Acc(defaults.rank, a.elt, node=_mk("permute", defaults.rank, a.elt, sx, deps))


def scatter(to, defaults, xs):
    """``scatter`` (Prelude.hs:1755-1766): ``permute const``; the source is cut to
    ``shape to `intersect` shape xs``; targets are assumed unique."""
    to, xs = use(to), use(xs)
    src = backpermute(intersect(to.shape, xs.shape), lambda ix: ix, xs)
    return permute(lambda new, old: new, defaults, lambda ix: Just_(index(to[ix])), src)


def scatterIf(to, mask, pred, defaults, xs):
    """``scatterIf`` (Prelude.hs:1780-1793)."""
    to, mask, xs = use(to), use(mask), use(xs)
    src = backpermute(intersect(to.shape, xs.shape), lambda ix: ix, xs)
    return permute(lambda new, old: new, defaults,
                   lambda ix: cond(pred(mask[ix]), Just_(index(to[ix])), Nothing_(1)), src)


def gather(frm, xs):
    """``gather`` (Prelude.hs:1701-1706): ``backpermute (shape from) (\\ix -> I1 (from ! ix))``."""
    frm, xs = use(frm), use(xs)
    return backpermute(frm.shape, lambda ix: index(frm[ix]), xs)


class Boundary:
    def __init__(self, kind, value=None):
        self.kind, self.value = kind, value


clamp, mirror, wrap = Boundary("clamp"), Boundary("mirror"), Boundary("wrap")


def function(f):
    """``function`` boundary (Language.hs:1060-1070)."""
    return Boundary("function", f)


def constant_boundary(v):
    """``AST.Constant`` boundary (AST.hs:480-485)."""
    return Boundary("constant", v)


def _stencil_arg(extent, elt):
    """Nested-tuple type of a neighbourhood: outermost dimension outermost."""
    t = elt
    for e in reversed(extent):
        t = tuple([t] * e)
    return t


def _nest(e, depth):
    """Turn an expression of nested-tuple type into nested Python tuples."""
    if depth == 0:
        return e
    return tuple(_nest(e[i], depth - 1) for i in range(len(e.ty)))


def _boundary_sx(b, rank, elt):
    if b.kind in ("clamp", "mirror", "wrap"):
        return b.kind, frozenset()
    if b.kind == "constant":
        v = lift(b.value, elt)
        return f"(constant {v.sx})", v.deps
    lam, body = _fun(lambda ix: lift(b.value(ix), elt), shape_ty(rank))
    return f"(function {lam})", body.deps


def stencil(f, boundary, a, extent=None):
    """``stencil`` (Language.hs:956).  ``extent`` gives the neighbourhood size
    per dimension (3/5/7/9; default 3 everywhere); ``f`` receives nested Python
    tuples, outermost dimension outermost, offsets -r..+r."""
    a = use(a)
    extent = tuple(extent or [3] * a.rank)
    st = _stencil_arg(extent, a.elt)
    lam, fb = _fun(lambda s: f(_nest(s, a.rank)), st)
    bsx, bdeps = _boundary_sx(boundary, a.rank, a.elt)
    op, deps = a.operand()
    relt = fb.ty
    sx = f"(stencil {ty_sx(relt)} (stencilr {' '.join(str(e) for e in extent)}) {lam} {bsx} {op})"
    return Acc(a.rank, relt, node=_mk("stencil", a.rank, relt, sx, deps | fb.deps | bdeps))


def stencil2(f, b1, a1, b2, a2, extent1=None, extent2=None):
    """``stencil2`` (Language.hs:975); result extent is the intersection."""
    a1, a2 = use(a1), use(a2)
    e1 = tuple(extent1 or [3] * a1.rank)
    e2 = tuple(extent2 or [3] * a2.rank)
    lam, fb = _fun(lambda s, t: f(_nest(s, a1.rank), _nest(t, a2.rank)), _stencil_arg(e1, a1.elt), _stencil_arg(e2, a2.elt))
    s1, d1 = _boundary_sx(b1, a1.rank, a1.elt)
    s2, d2 = _boundary_sx(b2, a2.rank, a2.elt)
    o1, dd1 = a1.operand()
    o2, dd2 = a2.operand()
    relt = fb.ty
    sx = (f"(stencil2 {ty_sx(relt)} (stencilr {' '.join(str(e) for e in e1)}) (stencilr {' '.join(str(e) for e in e2)}) "
          f"{lam} {s1} {o1} {s2} {o2})")
    return Acc(a1.rank, relt, node=_mk("stencil2", a1.rank, relt, sx, fb.deps | d1 | d2 | dd1 | dd2))


# derived operations (Prelude.hs:826-884) --------------------------------------
def sum_(a): a = use(a); return fold(lambda x, y: x + y, lift(0, a.elt), a)
def product(a): a = use(a); return fold(lambda x, y: x * y, lift(1, a.elt), a)
def maximum(a): return fold1(max_, a)
def minimum(a): return fold1(min_, a)


# segmented scans (Prelude.hs:950-1420): built from the skeletons above -----------------
def _outer_inner(sh, rank):
    """(outer components, innermost extent) of a shape expression."""
    return [sh[d] for d in range(rank - 1)], sh[rank - 1]


def _null(a):
    return use(a).size().eq(0)


def _take_inner(n, a):
    """The first ``n`` elements along the innermost dimension (``take``, Prelude.hs:1531-1540)."""
    a = use(a)
    outer, sz = _outer_inner(a.shape, a.rank)
    return backpermute(index(*outer, min_(max_(lift(n, INT), 0), sz)), lambda ix: ix, a)


def _drop_inner(n, a):
    """All but the first ``n`` elements along the innermost dimension (``drop``, Prelude.hs:1556-1567)."""
    a = use(a)
    outer, sz = _outer_inner(a.shape, a.rank)
    n = max_(lift(n, INT), 0)
    return backpermute(index(*outer, max_(sz - n, 0)), lambda ix: index(*[ix[d] for d in range(a.rank - 1)], ix[a.rank - 1] + n), a)


def _init1(a):
    """``init`` of a vector (Prelude.hs:1582-1591)."""
    a = use(a)
    return backpermute(index(max_(a.shape[0] - 1, 0)), lambda ix: ix, a)


# ----------------------------------------------------------------------------
# More of the Prelude, each built from the operations above as the reference builds it
# (shape-polymorphic slices are written with None for `All`; lenses _1, _2, .. are the
# numbers 1, 2, .. counted from the innermost dimension)
# ----------------------------------------------------------------------------
All = None


def replicate(slix, a):
    """``replicate`` (Language.hs:265-271): ``slix`` lists every dimension of the result, outermost
    first: ``All`` where the argument's next dimension goes, an extent where the array is repeated."""
    a = use(a)
    kept = [d for d, s in enumerate(slix) if s is All]
    if len(kept) != a.rank:
        raise TypeError("replicate: the slice has as many Alls as the array has dimensions")
    ash = a.shape
    ext, k = [], 0
    for s in slix:
        if s is All:
            ext.append(ash[k])
            k += 1
        else:
            ext.append(lift(s, INT))
    return backpermute(index(*ext), lambda ix: index(*[ix[d] for d in kept]), a)


def slice(a, slix):  # noqa: A001
    """``slice`` (Language.hs:398-403): one entry per dimension of the array, ``All`` to keep it, an
    index to cut there."""
    a = use(a)
    if len(slix) != a.rank:
        raise TypeError("slice: one entry per dimension")
    kept = [d for d, s in enumerate(slix) if s is All]
    ash = a.shape

    def src(ix):
        k, out = 0, []
        for s in slix:
            if s is All:
                out.append(ix[k])
                k += 1
            else:
                out.append(lift(s, INT))
        return index(*out)
    return backpermute(index(*[ash[d] for d in kept]), src, a)


def imap(f, a):
    """``imap`` (Prelude.hs:177-181): map with the element's index."""
    a = use(a)
    return generate(a.shape, lambda ix: f(ix, a[ix]))


def indexed(a):
    """``indexed`` (Prelude.hs:172-173: ``imap T2``): each element paired with its index."""
    a = use(a)
    return generate(a.shape, lambda ix: tup(ix, a[ix]))


def flatten(a):
    """``flatten`` (Prelude.hs:1430-1432)."""
    a = use(a)
    return reshape(index(a.size()), a)


def foldAll(f, z, a):
    """``foldAll`` (Prelude.hs:664-670): ``fold f e (flatten arr)``."""
    return fold(f, z, flatten(a))


def fold1All(f, a):
    return fold1(f, flatten(a))


def all_(p, a):
    """``all`` (Prelude.hs:780-784, 807-810): ``and . map p``, ``and = fold (&&) True``."""
    return fold(and_, Exp(BOOL, "(const u8 1)"), map_(p, a))


def any_(p, a):
    """``any`` (Prelude.hs:799-803, 814-817): ``or . map p``."""
    return fold(or_, Exp(BOOL, "(const u8 0)"), map_(p, a))


def prescanl(f, e, a):
    """``prescanl f e = afst . scanl' f e`` (Prelude.hs:899-905)."""
    return scanl_prime(f, e, a)[0]


def postscanl(f, e, a):
    """``postscanl f e = map (e `f`) . scanl1 f`` (Prelude.hs:916-922)."""
    a = use(a)
    e = lift(e, a.elt)
    return map_(lambda x: f(e, x), scanl1(f, a))


def prescanr(f, e, a):
    return scanr_prime(f, e, a)[0]


def postscanr(f, e, a):
    a = use(a)
    e = lift(e, a.elt)
    return map_(lambda x: f(x, e), scanr1(f, a))


def enumFromStepN(sh, x, y):
    """``enumFromStepN`` (Prelude.hs:1478-1490): x, x+y, x+y+y, .. in row-major order, computed as
    ``fromIntegral i * y + x``."""
    sh = _shape_exp(sh)
    x = x if isinstance(x, Exp) else constant(x)
    y = lift(y, x.ty)
    return generate(sh, lambda ix: from_integral(to_index(sh, ix), x.ty) * y + x, x.ty)


def concatOn(dim, xs, ys):
    """``concatOn`` (Prelude.hs:1588-1610) along the ``dim``-th dimension from the inside: that extent is
    the sum, every other one the smaller of the two."""
    xs, ys = use(xs), use(ys)
    r = xs.rank
    d = r - dim
    shx, shy = xs.shape, ys.shape
    m = shx[d]
    ext = [(m + shy[k]) if k == d else min_(shx[k], shy[k]) for k in range(r)]

    def f(ix):
        i = ix[d]
        return cond(i < m, xs[ix], ys[index(*[(i - m) if k == d else ix[k] for k in range(r)])])
    return generate(index(*ext), f, xs.elt)


def append(xs, ys):
    """``(++)`` (Prelude.hs:1527-1531): ``concatOn _1``."""
    return concatOn(1, xs, ys)


def compact(keep, a):
    """``compact`` (Prelude.hs:1652-1690): the elements of ``a`` whose flag is set, as one vector, and how
    many each innermost row kept.  (The reference's shortcuts for empty and all-kept vectors give the
    same values and are left out.)"""
    keep, a = use(keep), use(a)
    target, ln = scanl_prime(lambda x, y: x + y, constant(0), map_(lambda k: from_integral(k, INT), keep))
    if a.rank == 1:
        prj = lambda ix: cond(keep[ix], Just_(index(target[ix])), Nothing_(1))  # noqa: E731
        return permute(lambda new, old: new, fill(index(the(ln)), undef(a.elt)), prj, a), ln
    offset, valid = scanl_prime(lambda x, y: x + y, constant(0), flatten(ln))
    sz = ln.shape

    def prj(ix):
        row = to_index(sz, index(*[ix[k] for k in range(a.rank - 1)]))
        return cond(keep[ix], Just_(index(offset[index(row)] + target[ix])), Nothing_(1))
    return permute(lambda new, old: new, fill(index(the(valid)), undef(a.elt)), prj, a), ln


def filter_(p, a):
    """``filter p arr = compact (map p arr) arr`` (Prelude.hs:1637-1641)."""
    a = use(a)
    return compact(compute(map_(p, a)), a)


def gatherIf(frm, mask, pred, defaults, xs):
    """``gatherIf`` (Prelude.hs:1726-1740): the gathered element where the mask passes, else the default."""
    frm, mask, defaults, xs = use(frm), use(mask), use(defaults), use(xs)
    g = gather(frm, xs)
    sh = intersect(intersect(frm.shape, mask.shape), defaults.shape)
    return generate(sh, lambda ix: cond(pred(mask[ix]), g[ix], defaults[ix]), xs.elt)


def reverseOn(dim, a):
    """``reverseOn`` (Prelude.hs:1842-1852)."""
    a = use(a)
    d = a.rank - dim
    sh = a.shape
    return backpermute(sh, lambda ix: index(*[(sh[k] - 1 - ix[k]) if k == d else ix[k] for k in range(a.rank)]), a)


def reverse(a):
    return reverseOn(1, a)


def transposeOn(d1, d2, a):
    """``transposeOn`` (Prelude.hs:1896-1912): swap two dimensions (counted from the inside)."""
    a = use(a)
    i, j = a.rank - d1, a.rank - d2
    sh = a.shape

    def swap(t):
        xs = [t[k] for k in range(a.rank)]
        xs[i], xs[j] = xs[j], xs[i]
        return index(*xs)
    return backpermute(swap(sh), swap, a)


def transpose(a):
    return transposeOn(1, 2, a)


def take(n, a):
    """``take`` (Prelude.hs:1933-1937)."""
    return _take_inner(n, a)


def drop(n, a):
    """``drop`` (Prelude.hs:1960-1964)."""
    return _drop_inner(n, a)


def init(a):
    """``init`` (Prelude.hs:1986-1989): all but the last element of every innermost row."""
    a = use(a)
    outer, sz = _outer_inner(a.shape, a.rank)
    return backpermute(index(*outer, max_(sz - 1, 0)), lambda ix: ix, a)


def tail(a):
    """``tail`` (Prelude.hs:2012-2015)."""
    return _drop_inner(1, a)


def expand(f, g, xs):
    """``expand`` (Prelude.hs:2519-2560): every element x becomes the ``f x`` elements ``g x 0 .. g x (f x - 1)``,
    all in one vector (flattening by expansion: head flags from the sizes' offsets, a segmented iota and a
    segmented copy of the source positions)."""
    xs = compute(use(xs))
    szs = compute(map_(f, xs))
    offset, ln = scanl_prime(lambda x, y: x + y, constant(0), szs)
    m = the(ln)
    n = m + 1
    put = lambda ix: Just_(index(offset[ix]))  # noqa: E731
    head_flags = permute(lambda new, old: new, fill(index(n), constant(0)), put, fill(szs.shape, constant(1)))
    plus = segmentedL(lambda x, y: x + y)
    idxs = map_(lambda p: p[1] - 1, scanl1(plus, zip_(head_flags, fill(index(m), constant(1)))))
    starts = permute(lambda new, old: new, fill(index(n), undef(INT)),
                     lambda ix: cond(szs[ix] > 0, put(ix), Nothing_(1)), enumFromN(xs.shape, constant(0)))
    iotas = map_(lambda p: p[1], scanl1(segmentedL(lambda x, y: x), zip_(head_flags, starts)))
    full = zipWith(g, gather(iotas, xs), idxs)
    empty = generate(index(0), lambda ix: undef(full.elt), full.elt)
    return acond(or_(xs.size().eq(0), m.eq(0)), empty, full)


def mkHeadFlags(seg):
    """Head flags of a segment descriptor for left scans: non-zero where a segment starts; a value
    above one stands for that many segments starting there (empty ones) (Prelude.hs:1364-1375)."""
    seg = use(seg)
    offset, ln = scanl_prime(lambda x, y: x + y, lift(0, seg.elt), seg)
    zeros = fill(index(from_integral(the(ln), INT) + 1), lift(0, seg.elt))
    ones = fill(index(offset.size()), lift(1, seg.elt))
    return _init1(permute(lambda x, y: x + y, zeros, lambda ix: Just_(index(from_integral(offset[ix], INT))), ones))


def mkTailFlags(seg):
    """Tail flags for right scans: the flag sits on the last place of each segment (Prelude.hs:1379-1390)."""
    seg = use(seg)
    offset, ln = scanr_prime(lambda x, y: x + y, lift(0, seg.elt), seg)
    zeros = fill(index(from_integral(the(ln), INT) + 1), lift(0, seg.elt))
    ones = fill(index(offset.size()), lift(1, seg.elt))
    return _init1(permute(lambda x, y: x + y, zeros, lambda ix: Just_(index(from_integral(the(ln) - 1 - offset[ix], INT))), ones))


def segmentedL(f):
    """Segmented version of ``f`` on (flag, value) pairs (Sengupta et al.; Prelude.hs:1395-1401)."""
    return lambda a, b: tup(a[0] | b[0], cond(b[0].ne(0), b[1], f(a[1], b[1])))


def segmentedR(f):
    """Prelude.hs:1403-1407"""
    g = segmentedL(lambda x, y: f(y, x))
    return lambda y, x: g(x, y)


def _with_flags(flags, arr):
    """``zip (replicate (indexTail (shape arr) :. All) flags) arr``"""
    arr, flags = use(arr), compute(use(flags))
    outer, sz = _outer_inner(arr.shape, arr.rank)
    return generate(index(*outer, min_(sz, flags.shape[0])), lambda ix: tup(flags[index(ix[arr.rank - 1])], arr[ix]))


def scanl1Seg(f, arr, seg):
    """Prelude.hs:1138-1148"""
    return map_(lambda t: t[1], scanl1(segmentedL(f), _with_flags(mkHeadFlags(seg), arr)))


def scanr1Seg(f, arr, seg):
    """Prelude.hs:1315-1325"""
    return map_(lambda t: t[1], scanr1(segmentedR(f), _with_flags(mkTailFlags(seg), arr)))


def scanlSeg(f, z, arr, seg):
    """Segmented exclusive scan: the seed is injected at the head of every segment, then a
    segmented inclusive scan runs over the longer array (Prelude.hs:979-1013)."""
    arr, seg = use(arr), use(seg)
    z = lift(z, arr.elt)
    outer, sz = _outer_inner(arr.shape, arr.rank)
    flags = compute(mkHeadFlags(seg))
    inc = compute(scanl1(lambda x, y: x + y, flags))
    full = index(*outer, sz + seg.shape[0])
    last = arr.rank - 1
    arr2 = permute(lambda new, old: new, fill(full, z),
                   lambda ix: Just_(index(*[ix[d] for d in range(last)], ix[last] + from_integral(inc[index(ix[last])], INT))),
                   _take_inner(flags.shape[0], arr))
    seg2 = map_(lambda v: v + 1, seg)
    return acond(lor(_null(arr), _null(flags)), fill(full, z), scanl1Seg(f, arr2, seg2))


def scanl_primeSeg(f, z, arr, seg):
    """``scanl'Seg`` (Prelude.hs:1052-1105): the segmented exclusive scan taken apart into the
    scan bodies and the per-segment totals."""
    arr, seg = use(arr), use(seg)
    z = lift(z, arr.elt)
    outer, sz = _outer_inner(arr.shape, arr.rank)
    last = arr.rank - 1
    arr2 = compute(scanlSeg(f, z, arr, seg))
    add = lambda x, y: x + y  # noqa: E731
    seg2 = map_(lambda v: v + 1, seg)
    tails = compute(zipWith(add, seg, scanl_prime(add, lift(0, seg.elt), seg2)[0]))
    sums = backpermute(index(*outer, seg.shape[0]), lambda ix: index(*[ix[d] for d in range(last)], from_integral(tails[index(ix[last])], INT)), arr2)
    offset = compute(scanl1(add, seg))
    inc = compute(scanl1(add, permute(add, fill(index(arr.size() + 1), lift(0, seg.elt)), lambda ix: Just_(index(from_integral(offset[ix], INT))),
                                      fill(seg.shape, lift(1, seg.elt)))))
    ln = offset[index(offset.shape[0] - 1)]
    body = backpermute(index(*outer, from_integral(ln, INT)),
                       lambda ix: index(*[ix[d] for d in range(last)], ix[last] + from_integral(inc[index(ix[last])], INT)), arr2)
    empty_sums = fill(index(*outer, seg.shape[0]), z)
    return acond(_null(arr), (compute(arr), empty_sums), (body, sums))


def scanrSeg(f, z, arr, seg):
    """Prelude.hs:1200-1226"""
    arr, seg = use(arr), use(seg)
    z = lift(z, arr.elt)
    outer, sz = _outer_inner(arr.shape, arr.rank)
    flags = compute(mkHeadFlags(seg))
    inc = compute(scanl1(lambda x, y: x + y, flags))
    full = index(*outer, sz + seg.shape[0])
    last = arr.rank - 1
    arr2 = permute(lambda new, old: new, fill(full, z),
                   lambda ix: Just_(index(*[ix[d] for d in range(last)], ix[last] + from_integral(inc.linear(ix[last]), INT) - 1)),
                   _drop_inner(sz - flags.shape[0], arr))
    seg2 = map_(lambda v: v + 1, seg)
    return acond(lor(_null(arr), _null(flags)), fill(full, z), scanr1Seg(f, arr2, seg2))


def scanr_primeSeg(f, z, arr, seg):
    """``scanr'Seg`` (Prelude.hs:1259-1290)"""
    arr, seg = use(arr), use(seg)
    z = lift(z, arr.elt)
    outer, sz = _outer_inner(arr.shape, arr.rank)
    last = arr.rank - 1
    add = lambda x, y: x + y  # noqa: E731
    arr2 = compute(scanrSeg(f, z, arr, seg))
    seg2 = map_(lambda v: v + 1, seg)
    heads = compute(scanl_prime(add, lift(0, seg.elt), seg2)[0])
    sums = backpermute(index(*outer, seg.shape[0]), lambda ix: index(*[ix[d] for d in range(last)], from_integral(heads[index(ix[last])], INT)), arr2)
    flags = compute(mkHeadFlags(seg))
    inc = compute(scanl1(add, flags))
    body = backpermute(index(*outer, flags.shape[0]),
                       lambda ix: index(*[ix[d] for d in range(last)], ix[last] + from_integral(inc[index(ix[last])], INT)), arr2)
    empty_sums = fill(index(*outer, seg.shape[0]), z)
    return acond(_null(arr), (compute(arr), empty_sums), (body, sums))


def prescanlSeg(f, z, arr, seg): return scanl_primeSeg(f, z, arr, seg)[0]      # Prelude.hs:1152-1162
def prescanrSeg(f, z, arr, seg): return scanr_primeSeg(f, z, arr, seg)[0]      # Prelude.hs:1329-1339


def postscanlSeg(f, z, arr, seg):
    """Prelude.hs:1166-1176"""
    z = lift(z, use(arr).elt)
    return map_(lambda v: f(z, v), scanl1Seg(f, arr, seg))


def postscanrSeg(f, z, arr, seg):
    """Prelude.hs:1343-1353"""
    z = lift(z, use(arr).elt)
    return map_(lambda v: f(v, z), scanr1Seg(f, arr, seg))


# ----------------------------------------------------------------------------
# Program assembly
# ----------------------------------------------------------------------------
class Program:
    """Program text plus the description of its inputs and outputs."""

    def __init__(self, text, inputs, outputs):
        self.text = text
        self.inputs = inputs          # list of Node (kind "in")
        self.outputs = outputs        # list of (rank, elt)


_NAME = re.compile(r"(?<![\w.+-])([av])(\d+)(?![\w.])")


def _canonical_names(text):
    """Rename array (a<k>) and scalar (v<k>) variables in order of first appearance.  Generated
    names come from a process-wide counter; the kernel cache is keyed on the generated source, so
    the same program built twice must yield the same text."""
    table = {}

    def sub(m):
        old = m.group(0)
        if old not in table:
            table[old] = m.group(1) + str(sum(1 for k in table if k[0] == m.group(1)))
        return table[old]
    return _NAME.sub(sub, text)


# ----------------------------------------------------------------------------
# Array-level control flow (evaluated on the host by every backend:
# Interpreter.hs:215-231).  The operands are array-level functions; their nodes
# are serialised inside the control node, except what does not depend on the
# function's parameters (hoisted in front of it, as the reference's let-floating
# does) and what several bodies share.
# ----------------------------------------------------------------------------
def _as_list(x):
    return list(x) if isinstance(x, (list, tuple)) else [x]


def _avars(like):
    return [Acc(a.rank, a.elt, node=Node("avar", a.rank, a.elt)) for a in like]


def _control(kind, outs_like, deps, bodies, pred=None, args=()):
    node = Node(kind, outs_like[0].rank, outs_like[0].elt, deps=deps, nouts=len(outs_like))
    node.out_ranks, node.out_elts = [a.rank for a in outs_like], [a.elt for a in outs_like]
    node.bodies, node.pred, node.args = bodies, pred, list(args)
    return [Acc(a.rank, a.elt, node=node, out=k) for k, a in enumerate(outs_like)]


def acond(p, t, e):
    """``acond`` (Language.hs:396; evaluated as Interpreter.hs:217-219): only the chosen branch runs."""
    p = p if isinstance(p, Exp) else lift(p, BOOL)
    single = not isinstance(t, (list, tuple))
    ts, es = [compute(use(x)) for x in _as_list(t)], [compute(use(x)) for x in _as_list(e)]
    if [(a.rank, a.elt) for a in ts] != [(a.rank, a.elt) for a in es]:
        raise TypeError("acond: the branches yield different arrays")
    out = _control("acond", ts, list(p.deps), [([], ts), ([], es)], pred=p)
    return out[0] if single else tuple(out)


def awhile(cond_f, step_f, init):
    """``awhile`` (Language.hs:409; Interpreter.hs:221-229): apply ``step_f`` while ``cond_f`` yields True
    (a ``Scalar Bool``, read at linear index 0).  The state is one array or a tuple of arrays."""
    single = not isinstance(init, (list, tuple))
    st = [compute(use(x)) for x in _as_list(init)]
    pc, ps = _avars(st), _avars(st)
    c = compute(use(cond_f(pc[0] if single else tuple(pc))))
    nxt = [compute(use(x)) for x in _as_list(step_f(ps[0] if single else tuple(ps)))]
    if (c.rank, c.elt) != (0, BOOL):
        raise TypeError("awhile: the condition must yield a Scalar Bool")
    if [(a.rank, a.elt) for a in nxt] != [(a.rank, a.elt) for a in st]:
        raise TypeError("awhile: the step changes the type of the state")
    out = _control("awhile", st, [a.node for a in st], [(pc, [c]), (ps, nxt)], args=st)
    return out[0] if single else tuple(out)


def apply(f, *args):
    """``Apply`` of an array-level function (AST.hs:268; Interpreter.hs:215)."""
    xs = [compute(use(x)) for x in args]
    ps = _avars(xs)
    r = f(*ps)
    single = not isinstance(r, (list, tuple))
    rs = [compute(use(x)) for x in _as_list(r)]
    out = _control("apply", rs, [a.node for a in xs], [(ps, rs)], args=xs)
    return out[0] if single else tuple(out)


def aforeign(name, fallback, *args):
    """``Aforeign`` (AST.hs; Interpreter.hs:217): a backend that has no foreign implementation under ``name``
    runs the pure Accelerate function given as the fallback, which is what the interpreter always does and
    what this backend does."""
    del name
    return apply(fallback, *args)


def atrace(message, shown, result):
    """``Atrace`` (Language.hs ``atrace``/``atraceArray``; Interpreter.hs:215, atraceOp :873-880): when the term is
    evaluated, the message and the arrays ``shown`` (one, several or none) go to standard error; the value is
    ``result`` (an array or a tuple of arrays), unchanged."""
    single = not isinstance(result, (list, tuple))
    sh = [compute(use(x)) for x in _as_list(shown)] if shown is not None else []
    rs = [compute(use(x)) for x in _as_list(result)]
    sx = "(atrace (hex %s) (show %s) (args %s))" % (message.encode().hex(), " ".join(a.name for a in sh), " ".join(a.name for a in rs))
    node = _mk("atrace", rs[0].rank, rs[0].elt, sx, [a.node for a in sh + rs], nouts=len(rs),
               ranks=[a.rank for a in rs], elts=[a.elt for a in rs])
    out = [Acc(a.rank, a.elt, node=node, out=k) for k, a in enumerate(rs)]
    return out[0] if single else tuple(out)


def pipe(f, g):
    """``f >-> g`` (Language.hs:365-372): two computations kept apart, the second applied to the first's result."""
    return lambda *xs: apply(g, *_as_list(apply(f, *xs)))


def _is_control(n):
    return n.kind in ("acond", "awhile", "apply")


def _reach(roots, stop=()):
    """Nodes reachable through ``deps`` (bodies of control nodes are not entered), dependencies first."""
    order, seen = [], set(id(s) for s in stop)

    def visit(n):
        if id(n) in seen:
            return
        seen.add(id(n))
        for d in n.deps:
            visit(d)
        order.append(n)
    for r in roots:
        visit(r)
    return order


def _all_inputs(roots):
    """Every program input below ``roots``, the bodies of control nodes included, in first-use order."""
    ins, seen = [], set()

    def visit(n):
        if id(n) in seen:
            return
        seen.add(id(n))
        for d in n.deps:
            visit(d)
        if _is_control(n):
            for _, res in n.bodies:
                for r in res:
                    visit(r.node)
        if n.kind == "in":
            ins.append(n)
    for r in roots:
        visit(r)
    return ins


def _depends_on(n, params, memo):
    """Whether node ``n`` needs one of the ``params`` (directly, or inside the body of a control node)."""
    if id(n) in memo:
        return memo[id(n)]
    memo[id(n)] = False
    r = any(n is q for q in params) or any(_depends_on(d, params, memo) for d in n.deps)
    if not r and _is_control(n):
        r = any(_depends_on(x.node, params, memo) for _, res in n.bodies for x in res)
    memo[id(n)] = r
    return r


class _Emitter:
    def __init__(self, embed):
        self.embed = embed

    def hex_use(self, n):
        sh, leaves = n.data
        body = " ".join("(hex " + np.ascontiguousarray(x).tobytes().hex() + ")" for x in leaves)
        return f"(use (array {n.rank} {ty_sx(n.elt)}) (shape{''.join(' ' + str(d) for d in sh[:n.rank])}) {body})"

    def level(self, roots, emitted, lines, indent):
        """Emit, into ``lines``, every node the ``roots`` need that is not in ``emitted`` yet."""
        skip = lambda n: id(n) in emitted or n.kind in ("in", "avar")  # noqa: E731
        hoisted = {}                                   # id(control node) -> nodes to emit in front of it
        while True:
            order = []
            seen = set()

            def visit(n):
                if id(n) in seen:
                    return
                seen.add(id(n))
                for d in list(n.deps) + hoisted.get(id(n), []):
                    visit(d)
                order.append(n)
            for r in roots:
                visit(r)
            here = set(id(n) for n in order)
            count, more = {}, False
            for c in order:
                if not _is_control(c) or skip(c):
                    continue
                for params, res in c.bodies:
                    memo = {}
                    for n in _reach([r.node for r in res]):
                        if skip(n) or id(n) in here:
                            continue
                        free = c.kind != "acond" and not _depends_on(n, [q.node for q in params], memo)
                        count[id(n)] = count.get(id(n), 0) + 1
                        if free or count[id(n)] > 1:
                            hoisted.setdefault(id(c), []).append(n)
                            more = True
            if not more:
                break
        pad = "  " * indent
        for n in order:
            if skip(n):
                continue
            lhs = n.names[0] if n.nouts == 1 else "(" + " ".join(n.names) + ")"
            if _is_control(n):
                inner = set(emitted)
                parts = []
                for params, res in n.bodies:
                    sub = []
                    self.level([r.node for r in res], inner | set(id(q.node) for q in params), sub, indent + 2)
                    head = "(branch" if n.kind == "acond" else "(afun (" + " ".join(f"({q.name} (array {q.rank} {ty_sx(q.elt)}))" for q in params) + ")"
                    parts.append("\n".join([pad + "    " + head] + sub + [pad + "      (out " + " ".join(r.name for r in res) + "))"]))
                args = "(args " + " ".join(a.name for a in n.args) + ")"
                if n.kind == "acond":
                    text = f"(acond {n.pred.sx}\n" + "\n".join(parts) + ")"
                else:
                    text = f"({n.kind}\n" + "\n".join(parts) + f"\n{pad}    {args})"
                lines.append(f"{pad}(let {lhs} {text})")
            else:
                lines.append(f"{pad}(let {lhs} {n.sx})")
            emitted.add(id(n))


def build_program(results, embed=False):
    """Serialise everything the results depend on, in dependency order.  With ``embed`` the host
    arrays given to ``use`` travel inside the program text as ``(use ...)`` nodes (the reference's
    ``Use``, Interpreter.hs:231) instead of being program inputs."""
    results = [compute(use(r)) for r in (results if isinstance(results, (list, tuple)) else [results])]
    roots = [r.node for r in results]
    ins = _all_inputs(roots)
    inputs = [n for n in ins if not (embed and n.data is not None)]
    lines = ["(program"]
    for n in inputs:
        lines.append(f"  (in {n.names[0]} (array {n.rank} {ty_sx(n.elt)}))")
    em = _Emitter(embed)
    if embed:
        for n in ins:
            if n.data is not None:
                lines.append(f"  (let {n.names[0]} {em.hex_use(n)})")
    em.level(roots, set(), lines, 1)
    lines.append("  (out " + " ".join(r.name for r in results) + "))")
    return Program(_canonical_names("\n".join(lines)), inputs, [(r.rank, r.elt) for r in results])
