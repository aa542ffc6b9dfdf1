"""Data-parallel execution over several GPUs: one process per GPU, arrays split
along the outermost dimension, at most one exchange step per skeleton.

  fold to a scalar   local fold1, all-gather of the partials, combine in rank
                     order (keeps non-commutative functions correct)
  per-row folds,     row blocks; no communication
  maps, foldSeg      (foldSeg: the split falls on a segment boundary)
  1-D scans          local fold1 -> all-gather of the totals -> exclusive scan of
                     the totals gives each rank its carry-in -> local seeded scan
  permute            private full-size target per rank (rank 0 starts from the
                     defaults, the others from the combination's identity),
                     then all-reduce
  stencil            row slabs with `radius` halo rows exchanged with the two
                     neighbours (send/recv) before every application

Collectives go through ``torch.distributed`` (NCCL over NVLink on GPUs; gloo on
CPU in the tests).  The local work is delegated to an *executor*: the GPU
executor below runs programs through the C-ABI library and exposes device
arrays to torch without copying.  Nothing here computes array results on the
CPU.
"""
from __future__ import annotations

import numpy as np
import torch
import torch.distributed as dist

from . import language as L


def closure_key(obj, depth=0):
    """A hashable description of what a builder function will build: its code and, recursively,
    everything it closes over (functions by code and closure, constants by value, other objects by
    identity).  Two lambdas written at the same place that capture different functions, shapes or
    constants get different keys; re-creating the same lambda with the same captures does not."""
    if depth > 6:
        return ("deep", id(obj))
    if isinstance(obj, (int, float, str, bytes, bool, type(None), np.generic)):
        return (type(obj).__name__, repr(obj))
    if isinstance(obj, (tuple, list)):
        return (type(obj).__name__,) + tuple(closure_key(x, depth + 1) for x in obj)
    if isinstance(obj, dict):
        return ("dict",) + tuple((repr(k), closure_key(v, depth + 1)) for k, v in sorted(obj.items(), key=lambda kv: repr(kv[0])))
    code = getattr(obj, "__code__", None)
    if code is not None:
        cells = tuple(closure_key(c.cell_contents, depth + 1) for c in (obj.__closure__ or ()))
        dflt = tuple(closure_key(d, depth + 1) for d in (obj.__defaults__ or ()))
        return ("fn", code.co_filename, code.co_firstlineno, _code_key(code), cells, dflt)
    func = getattr(obj, "__func__", None)
    if func is not None:                      # bound method
        return ("method", closure_key(func, depth + 1), id(getattr(obj, "__self__", None)))
    if hasattr(obj, "elt") and hasattr(obj, "shape"):     # an array: builders only look at its type and shape
        return ("array", repr(obj.elt), tuple(obj.shape))
    return (type(obj).__name__, id(obj))


def _code_key(code):
    """Instructions, names and constants of a code object (nested lambdas are constants of it)."""
    consts = tuple(_code_key(c) if hasattr(c, "co_code") else repr(c) for c in code.co_consts)
    return (code.co_code, code.co_names, consts)


class ProgramCache:
    """Built programs by call-site key, input signature and builder identity."""

    def __init__(self):
        self._progs = {}

    def get(self, key, build, inputs):
        sig = (key, tuple((a.elt if L.is_scalar(a.elt) else tuple(a.elt), len(a.shape)) for a in inputs), closure_key(build))
        ent = self._progs.get(sig)
        if ent is None:
            L.reset_names()
            params = [L.param(len(a.shape), a.elt) for a in inputs]
            res = build(*params)
            single = not isinstance(res, (list, tuple))
            prog = L.build_program(res)
            order = [next(i for i, q in enumerate(params) if q.node is n) for n in prog.inputs]
            # `build` is kept so that objects its key names by identity stay alive as long as the entry
            ent = self._progs[sig] = (prog, order, single, build)
        return ent[:3]


class GpuExecutor:
    """Runs terms on this rank's GPU; arrays are ``backend.DeviceArray``."""

    def __init__(self, ctx, group=None):
        """``group``: a ``backend.Group`` (the library's own NCCL communicator); without one the
        exchange steps go through ``torch.distributed`` on views of the device arrays."""
        from . import backend
        self.backend, self.ctx, self.group = backend, ctx, group
        self.stream = torch.cuda.ExternalStream(ctx.stream(), device=torch.device("cuda", ctx.device))
        self._progs = ProgramCache()

    @classmethod
    def with_group(cls, ctx, deadline_s=60.0):
        """Executor whose exchange steps run inside the C-ABI library: rank 0 creates the rendezvous
        id and the ranks of the default process group receive it over ``torch.distributed``."""
        from . import backend
        rank, world = dist.get_rank(), dist.get_world_size()
        box = [backend.Group.unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        return cls(ctx, backend.Group(ctx, box[0], rank, world, deadline_s))

    def program(self, key, build, inputs):
        """Text of the (cached) program ``build`` yields for these inputs."""
        return self._progs.get(key, build, inputs)[0].text

    def run_rows(self, text, inputs, out, row_lo, row_hi):
        self.ctx.run_rows(text, inputs, out, row_lo, row_hi)

    def run_rows2(self, text, inputs, out, row_lo, row_hi, row_lo2, row_hi2):
        self.ctx.run_rows2(text, inputs, out, row_lo, row_hi, row_lo2, row_hi2)

    def run(self, key, build, inputs):
        """``build(*params)`` -> term(s).  The built program is cached under the input signature
        and the builder's own identity (its code and everything it captures: ``closure_key``);
        ``key`` only keeps unrelated call sites apart."""
        prog, order, single = self._progs.get(key, build, inputs)
        outs = self.ctx.execute(prog.text, [inputs[k] for k in order], len(prog.outputs))
        for o, (_, elt) in zip(outs, prog.outputs):
            o.elt = elt
        return outs[0] if single else outs

    def from_host(self, a):
        return self.ctx.from_host(a)

    def to_host(self, a):
        return a.download()

    def tensor(self, a, leaf=0):
        """Zero-copy torch view of one leaf of a device array."""
        dt = np.dtype(L.NP_OF[a.leaf_types[leaf]])
        n = int(np.prod(a.shape)) if len(a.shape) else 1
        if n == 0:
            return torch.empty(a.shape, dtype=torch.from_numpy(np.empty(0, dt)).dtype, device=self.stream.device)

        class View:
            pass
        v = View()
        v.__cuda_array_interface__ = {"shape": tuple(a.shape) if len(a.shape) else (1,), "typestr": dt.str, "data": (a.devptr(leaf), False),
                                      "version": 3}
        t = torch.as_tensor(v, device=self.stream.device)
        t._keepalive = a
        return t

    def wrap(self, t, elt):
        """Device array over a torch tensor's memory (the tensor must stay alive)."""
        a = self.ctx.wrap(elt, tuple(t.shape), [t.data_ptr()])
        a._keepalive = t
        return a

    def empty(self, elt, shape):
        return self.ctx.array(elt, tuple(shape))

    def slice1d(self, a, lo, hi):
        """Elements [lo, hi) of a vector of scalars as a view (no copy)."""
        item = np.dtype(L.NP_OF[a.leaf_types[0]]).itemsize
        v = self.ctx.wrap(a.elt, (hi - lo,), [a.devptr(0) + lo * item])
        v._keepalive = a
        return v

    def rows_view(self, a, lo, hi):
        """Rows [lo, hi) of a rank-2 array as a view (rows are contiguous: no copy)."""
        cols = a.shape[1]
        ptrs = [a.devptr(k) + lo * cols * np.dtype(L.NP_OF[t]).itemsize for k, t in enumerate(a.leaf_types)]
        v = self.ctx.wrap(a.elt, (hi - lo, cols), ptrs)
        v._keepalive = a
        return v

    def collective(self):
        """Context in which torch collectives are ordered after this executor's kernels."""
        return torch.cuda.stream(self.stream)

    def sync(self):
        self.ctx.sync()


class HaloSlab:
    """A row slab kept resident with room for its neighbours' halo rows: ``ext`` has
    ``top + rows + bot`` rows, the slab's own rows start at ``top``.  Stencils over
    several GPUs take and return this layout without copying."""

    def __init__(self, ext, top, rows, bot):
        self.ext, self.top, self.rows, self.bot = ext, top, rows, bot
        self.shape = (rows, ext.shape[1])
        self.elt = ext.elt


class Sharded:
    """Sharded skeletons over an executor and a process group."""

    def __init__(self, executor, group=None):
        self.ex = executor
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1

    # -- helpers ------------------------------------------------------------------
    def _all_gather_scalars(self, arr):
        """Replicated vector of every rank's rank-0 (or 1-element) array."""
        outs = []
        for leaf in range(len(arr.leaf_types) if hasattr(arr, "leaf_types") else 1):
            t = self.ex.tensor(arr, leaf).reshape(1)
            g = torch.empty(self.world, dtype=t.dtype, device=t.device)
            with self.ex.collective():
                if self.world > 1:
                    dist.all_gather_into_tensor(g, t, group=self.group)
                else:
                    g.copy_(t)
            outs.append(g)
        return outs

    def _gathered_array(self, arr):
        """All ranks' scalars as one local array of shape (world,) (element type kept)."""
        if getattr(self.ex, "group", None) is not None:
            return self.ex.group.all_gather(arr)
        leaves = self._all_gather_scalars(arr)
        if len(leaves) == 1:
            return self.ex.wrap(leaves[0], arr.elt)
        # tuples: one wrapped leaf each, zipped by a program
        parts = [self.ex.wrap(t, ty) for t, ty in zip(leaves, L.flatten_ty(arr.elt))]
        return self.ex.run(("zipleaves", len(parts)), lambda *ps: L.generate(ps[0].shape, lambda ix: _retuple(arr.elt, [p[ix] for p in ps])), parts)

    # -- folds ------------------------------------------------------------------------
    def fold_all(self, f, z, shard, key="fold_all"):
        """``fold f z`` of a vector split across ranks; the result is replicated.
        Shards must be non-empty (fold1 of the local part)."""
        part = self.ex.run((key, "local"), lambda x: L.fold1(f, x), [shard])
        allp = self._gathered_array(part)
        if z is None:
            return self.ex.run((key, "final1"), lambda p: L.fold1(f, p), [allp])
        return self.ex.run((key, "final", repr(z)), lambda p: L.fold(f, z, p), [allp])

    def fold_rows(self, f, z, rows_block, key="fold_rows"):
        """Per-row fold of this rank's block of rows: no communication."""
        return self.ex.run((key, repr(z)), lambda x: L.fold(f, z, x), [rows_block])

    # -- scans ------------------------------------------------------------------------
    def scan1d(self, kind, f, z, shard, key="scan"):
        """1-D ``scanl``/``scanl1``/``scanl'``/``scanr``/``scanr1``/``scanr'`` of a vector
        split into contiguous chunks in rank order.  Returns this rank's part of the
        result (and, for the primed forms, the replicated total).

        scanl / scanr: rank r holds out[r*n .. (r+1)*n); the last rank additionally holds
        out[N] (its part has n+1 elements).
        """
        right = kind in ("scanr", "scanr1", "scanr'")
        seeded = kind in ("scanl", "scanr", "scanl'", "scanr'")
        primed = kind.endswith("'")
        r, G = self.rank, self.world
        total = self.ex.run((key, "total"), lambda x: L.fold1(f, x), [shard])
        totals = self._gathered_array(total)
        # carry-in: everything that comes logically before this chunk
        if not right:
            if seeded:
                carries = self.ex.run((key, "carryL", repr(z)), lambda t: L.scanl(f, z, t), [totals])       # G+1 entries
            else:
                carries = self.ex.run((key, "carryL1"), lambda t: L.scanl1(f, t), [totals])                 # carry of rank r = entry r-1
        else:
            if seeded:
                carries = self.ex.run((key, "carryR", repr(z)), lambda t: L.scanr(f, z, t), [totals])       # entry r+1 = carry of rank r
            else:
                carries = self.ex.run((key, "carryR1"), lambda t: L.scanr1(f, t), [totals])
        n = shard.shape[0]
        if not right:
            idx = r if seeded else r - 1
        else:
            idx = r + 1
        has_carry = seeded or (not right and r > 0) or (right and r < G - 1)
        if not has_carry:
            # first chunk of an unseeded scan
            return self.ex.run((key, "plain", kind), lambda x: (L.scanl1 if not right else L.scanr1)(f, x), [shard])
        pick = lambda c: c[L.index(idx)]  # noqa: E731
        op = L.scanr if right else L.scanl
        full = self.ex.run((key, "seeded", kind, idx), lambda x, c: op(f, pick(c), x), [shard, carries])    # n+1 values
        if primed:
            tot_idx = 0 if right else G
            tot = self.ex.run((key, "tot", tot_idx), lambda c: L.unit(c[L.index(tot_idx)]), [carries])
            part = self._slice(full, 1, n + 1) if right else self._slice(full, 0, n)
            return part, tot
        if seeded:
            # the chunk's n values; the rank holding the end of the vector also keeps the extra element
            # (scanl: out[N] = total; scanr: out[N] = seed)
            return full if r == G - 1 else self._slice(full, 0, n)
        # inclusive: drop the carry itself
        return self._slice(full, 0, n) if right else self._slice(full, 1, n + 1)

    def _slice(self, arr, lo, hi):
        if hasattr(self.ex, "slice1d"):
            return self.ex.slice1d(arr, lo, hi)          # a view, no copy
        return self.ex.run(("slice", lo, hi), lambda x: L.backpermute(L.index(hi - lo), lambda ix: L.index(ix[0] + lo), x), [arr])

    # -- permute ----------------------------------------------------------------------
    def permute(self, op, defaults, index_fn, inputs, build_source, key="permute"):
        """``permute (op)`` with ``op`` in {"add", "min", "max"}: every rank combines its
        source shard into a private full-size target (rank 0 from the defaults, the others
        from the identity), then the targets are all-reduced.  ``index_fn(ix, *inputs)`` and
        ``build_source(*inputs)`` are given the rank's input shards."""
        f = {"add": lambda a, b: a + b, "min": L.min_, "max": L.max_}[op]
        elt = defaults.elt
        if not L.is_scalar(elt):
            raise ValueError("sharded permute reduces one scalar leaf; tuple element types are not supported")
        if self.rank == 0:
            start = defaults
        else:
            ident = {"add": lambda t: L.lift(0, t), "min": lambda t: L.max_bound(t) if not L.is_float(t) else L.lift(float("inf"), t),
                     "max": lambda t: L.min_bound(t) if not L.is_float(t) else L.lift(float("-inf"), t)}[op](elt)
            start = self.ex.run((key, "ident", op), lambda d: L.fill(d.shape, ident), [defaults])
        out = self.ex.run((key, op), lambda d, *xs: L.permute(f, d, lambda ix: index_fn(ix, *xs), build_source(*xs)), [start] + list(inputs))
        if self.world > 1:
            if getattr(self.ex, "group", None) is not None:
                self.ex.group.all_reduce(out, op)
                return out
            t = self.ex.tensor(out)
            with self.ex.collective():
                dist.all_reduce(t, op={"add": dist.ReduceOp.SUM, "min": dist.ReduceOp.MIN, "max": dist.ReduceOp.MAX}[op], group=self.group)
        return out

    # -- stencils -----------------------------------------------------------------------
    def _neighbours(self, boundary):
        r, G = self.rank, self.world
        wrap = boundary.kind == "wrap" and G > 1
        up = (r - 1) % G if (r > 0 or wrap) else None
        down = (r + 1) % G if (r < G - 1 or wrap) else None
        return up, down

    def halo_slab(self, slab, boundary, radius=1, key="halo"):
        """Copy a plain row slab into the resident layout with halo rows (done once, when the
        array is distributed)."""
        if isinstance(slab, HaloSlab):
            return slab
        up, down = self._neighbours(boundary)
        rows, cols = slab.shape
        top, bot = (radius if up is not None else 0), (radius if down is not None else 0)
        if top == 0 and bot == 0:
            return HaloSlab(slab, 0, rows, 0)
        ext = self.ex.run((key, "extend", top, bot), lambda x: L.generate(L.index(rows + top + bot, cols),
                          lambda ix: L.cond(L.land(ix[0] >= top, ix[0] < top + rows), x[L.index(L.min_(L.max_(ix[0] - top, 0), rows - 1), ix[1])],
                                            L.lift(0, slab.elt)), slab.elt), [slab])
        return HaloSlab(ext, top, rows, bot)

    def stencil_iterate(self, f, boundary, slab, iterations, radius=1, key="stencil"):
        """Apply a rank-2 stencil ``iterations`` times to an array split into row slabs.
        Interior ranks keep ``radius`` halo rows on either side of their slab; the halos are
        refreshed from the neighbours before each application (wrap boundaries also connect
        the first and last rank).  ``slab`` is a plain slab (copied into the halo layout
        first) or a ``HaloSlab``.  Returns this rank's slab of the result, a view of the last
        application's output."""
        if self.world == 1 and not isinstance(slab, HaloSlab):
            cur = slab
            for _ in range(iterations):
                cur = self.ex.run((key, "it"), lambda x: L.stencil(f, boundary, x), [cur])
            return cur
        h = self.halo_slab(slab, boundary, radius, key)
        up, down = self._neighbours(boundary)
        ext = h.ext
        cols = ext.shape[1]
        g = getattr(self.ex, "group", None)
        if g is not None and iterations > 0 and h.rows >= 4 * radius and (h.top or h.bot):
            # Exchange and kernels overlap: the rows that need no halo rows are computed while the
            # halo rows of the current grid are still in flight (second stream), the `radius` rows at
            # either edge of the slab after they have arrived; the edges of the new grid then travel
            # while the next application's interior runs.  Two grids in the halo layout alternate.
            text = self.ex.program((key, "it"), lambda x: L.stencil(f, boundary, x), [ext])
            spare = [self.ex.empty(ext.elt, ext.shape) for _ in range(min(iterations, 2))]      # the caller's grid is only read
            lo, hi = h.top, h.top + h.rows
            ilo, ihi = lo + (radius if h.top else 0), hi - (radius if h.bot else 0)
            g.halo_exchange(ext, h.top, h.rows, h.bot, radius, up, down, overlap=True)
            src = ext
            for k in range(iterations):
                dst = spare[k % 2]
                self.ex.run_rows(text, [src], dst, ilo, ihi)
                g.halo_wait()
                if ilo > lo and ihi < hi:
                    self.ex.run_rows2(text, [src], dst, lo, ilo, ihi, hi)      # both edges in one launch
                elif ilo > lo:
                    self.ex.run_rows(text, [src], dst, lo, ilo)
                elif ihi < hi:
                    self.ex.run_rows(text, [src], dst, ihi, hi)
                if k + 1 < iterations:
                    g.halo_exchange(dst, h.top, h.rows, h.bot, radius, up, down, overlap=True)
                src = dst
            return self.ex.rows_view(src, h.top, h.top + h.rows)
        for _ in range(iterations):
            self._exchange_halos(ext, h.rows, cols, h.top, h.bot, up, down, radius)
            ext = self.ex.run((key, "it"), lambda x: L.stencil(f, boundary, x), [ext])
        return self.ex.rows_view(ext, h.top, h.top + h.rows)

    def stencil2(self, f, b1, slab1, b2, slab2, radius=1, key="stencil2"):
        """One application of a rank-2 ``stencil2`` to two arrays split into the same row slabs
        (plain slabs or ``HaloSlab``s)."""
        if self.world == 1 and not isinstance(slab1, HaloSlab) and not isinstance(slab2, HaloSlab):
            return self.ex.run((key, "single"), lambda x, y: L.stencil2(f, b1, x, b2, y), [slab1, slab2])
        hs = [self.halo_slab(slab1, b1, radius, key), self.halo_slab(slab2, b2, radius, key)]
        if (hs[0].top, hs[0].rows, hs[0].bot) != (hs[1].top, hs[1].rows, hs[1].bot):
            raise ValueError("stencil2 over slabs needs the same halo layout for both arrays")
        for h, b in zip(hs, (b1, b2)):
            up, down = self._neighbours(b)
            self._exchange_halos(h.ext, h.rows, h.ext.shape[1], h.top, h.bot, up, down, radius)
        out = self.ex.run((key, "apply"), lambda x, y: L.stencil2(f, b1, x, b2, y), [hs[0].ext, hs[1].ext])
        return self.ex.rows_view(out, hs[0].top, hs[0].top + hs[0].rows)

    def _exchange_halos(self, ext, rows, cols, top, bot, up, down, radius):
        if getattr(self.ex, "group", None) is not None:
            if up is not None or down is not None:
                self.ex.group.halo_exchange(ext, top, rows, bot, radius, up, down, overlap=False)
            return
        t = self.ex.tensor(ext)
        ops = []
        # sends first (up, down), then receives (from down, from up): with two ranks and a wrap
        # boundary both neighbours are the same peer, and point-to-point messages between one
        # pair are matched in posting order
        if up is not None:
            ops.append(dist.P2POp(dist.isend, t[top:top + radius], up, self.group))
        if down is not None:
            ops.append(dist.P2POp(dist.isend, t[top + rows - radius:top + rows], down, self.group))
        if down is not None:
            ops.append(dist.P2POp(dist.irecv, t[top + rows:top + rows + bot], down, self.group))
        if up is not None:
            ops.append(dist.P2POp(dist.irecv, t[0:top], up, self.group))
        if ops:
            with self.ex.collective():
                for w in dist.batch_isend_irecv(ops):
                    w.wait()


def _retuple(elt, leaves):
    it = iter(leaves)

    def go(t):
        if L.is_scalar(t):
            return next(it)
        return L.tup(*[go(c) for c in t])
    return go(elt)


def split_segments(offsets, parts):
    """Boundaries (segment indices) that split a segmented vector into ``parts`` chunks
    of nearly equal element counts; each boundary falls on a segment boundary."""
    offsets = np.asarray(offsets)
    n = int(offsets[-1])
    cuts = [0]
    for k in range(1, parts):
        cuts.append(int(np.searchsorted(offsets, k * n // parts, side="left")))
    cuts.append(len(offsets) - 1)
    return cuts
