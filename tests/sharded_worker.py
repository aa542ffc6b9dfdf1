"""Worker for the CPU multi-process tests of accelerate_b200.sharded: gloo ranks
whose local executor is the CPU oracle (test infrastructure), checked against
the oracle run on the undivided arrays."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import accelerate_b200 as A  # noqa: E402
from accelerate_b200 import language as L  # noqa: E402
from accelerate_b200.sharded import Sharded, split_segments  # noqa: E402
from oracle import oracle  # noqa: E402

add = lambda a, b: a + b  # noqa: E731


class HostArray:
    def __init__(self, leaves, elt):
        self.leaves = [np.require(x, requirements='C') for x in leaves]
        self.elt = elt
        self.shape = tuple(self.leaves[0].shape)
        self.leaf_types = L.flatten_ty(elt)


class OracleExecutor:
    """Same interface as sharded.GpuExecutor, on host arrays."""

    def run(self, key, build, inputs):
        res = build(*[A.use(tuple(a.leaves) if not L.is_scalar(a.elt) else a.leaves[0], a.elt) for a in inputs])
        single = not isinstance(res, (list, tuple))
        prog = L.build_program(res)
        outs = oracle.run_text(prog.text, [n.data for n in prog.inputs])
        arrs = [HostArray(leaves, elt) for (_, leaves), (_, elt) in zip(outs, prog.outputs)]
        return arrs[0] if single else arrs

    def from_host(self, a):
        return HostArray([a], L.TY_OF_NP[a.dtype])

    def to_host(self, a):
        return a.leaves[0] if L.is_scalar(a.elt) else tuple(a.leaves)

    def tensor(self, a, leaf=0):
        return torch.from_numpy(a.leaves[leaf])

    def wrap(self, t, elt):
        return HostArray([t.numpy()], elt)

    def slice1d(self, a, lo, hi):
        return HostArray([x[lo:hi] for x in a.leaves], a.elt)

    def rows_view(self, a, lo, hi):
        return HostArray([x[lo:hi] for x in a.leaves], a.elt)

    def collective(self):
        import contextlib
        return contextlib.nullcontext()

    def sync(self):
        pass


def _mss(a, b):
    return A.tup(A.max_(a[0], A.max_(b[0], a[2] + b[1])), A.max_(a[1], a[3] + b[1]), A.max_(b[2], a[2] + b[3]), a[3] + b[3])


def main(rank, world, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    if GPU:
        from accelerate_b200 import backend
        from accelerate_b200.sharded import GpuExecutor
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        # "gpu": the exchange steps run inside the C-ABI library (its own NCCL communicator);
        # "gpu-torch": through torch.distributed on views of the device arrays
        ex = GpuExecutor.with_group(backend.Context(rank), deadline_s=120.0) if sys.argv[4] == "gpu" else GpuExecutor(backend.Context(rank))
    else:
        dist.init_process_group("gloo", rank=rank, world_size=world)
        ex = OracleExecutor()
    sh = Sharded(ex)
    rng = np.random.default_rng(5)
    n = 1000
    x = rng.integers(-50, 50, size=n * world).astype(np.int64)
    mine = ex.from_host(x[rank * n:(rank + 1) * n])
    fails = []

    def check(name, got, want):
        got = np.asarray(got)
        if got.shape != np.asarray(want).shape or not np.array_equal(got, want):
            fails.append(name)

    # fold to a scalar, commutative and not
    check("fold", ex.to_host(sh.fold_all(add, 7, mine)), oracle.run(A.fold(add, 7, x)))
    g = lambda v: A.tup(A.max_(v, 0), A.max_(v, 0), A.max_(v, 0), v)  # noqa: E731
    tup_in = ex.run("g", lambda a: A.compute(A.map(g, a)), [mine])
    got = ex.to_host(sh.fold_all(_mss, None, tup_in, key="mss"))
    want = oracle.run(A.fold1(_mss, A.map(g, x)))
    for a, b in zip(got, want):
        check("fold-noncomm", a, b)
    # scans: every variant; parts concatenated in rank order must equal the undivided scan
    for kind, ref in [("scanl", A.scanl(add, 3, x)), ("scanl1", A.scanl1(add, x)), ("scanr", A.scanr(add, 3, x)), ("scanr1", A.scanr1(add, x))]:
        part = ex.to_host(sh.scan1d(kind, add, 3 if kind in ("scanl", "scanr") else None, mine, key=kind))
        parts = [None] * world
        dist.all_gather_object(parts, part)
        check(kind, np.concatenate(parts), oracle.run(ref))
    for kind, ref in [("scanl'", A.scanl_prime(add, 3, x)), ("scanr'", A.scanr_prime(add, 3, x))]:
        part, tot = sh.scan1d(kind, add, 3, mine, key=kind)
        parts = [None] * world
        dist.all_gather_object(parts, ex.to_host(part))
        rp, rt = oracle.run(list(ref))
        check(kind, np.concatenate(parts), rp)
        check(kind + "-total", ex.to_host(tot), rt)
    # permute (+) into a replicated histogram
    keys = rng.integers(0, 37, size=n * world).astype(np.int64)
    kmine = ex.from_host(keys[rank * n:(rank + 1) * n])
    defaults = ex.from_host(np.arange(37, dtype=np.int64))
    got = ex.to_host(sh.permute("add", defaults, lambda ix, k, v: A.Just_(A.index(k[ix])), [kmine, mine], lambda k, v: v))
    ku = A.use(keys)
    check("permute", got, oracle.run(A.permute(add, np.arange(37, dtype=np.int64), lambda ix: A.Just_(A.index(ku[ix])), x)))
    # stencil over row slabs with halo exchange, clamp and wrap
    rows = 6
    grid = rng.integers(0, 100, size=(rows * world, 9)).astype(np.int64)
    slab = ex.from_host(grid[rank * rows:(rank + 1) * rows])
    jac = lambda s: s[0][1] + s[2][1] + s[1][0] + s[1][2] - 3 * s[1][1]  # noqa: E731
    for bnd, name in [(A.clamp, "clamp"), (A.wrap, "wrap"), (A.mirror, "mirror")]:
        out = ex.to_host(sh.stencil_iterate(jac, bnd, slab, 3, key="st" + name))
        parts = [None] * world
        dist.all_gather_object(parts, out)
        ref = A.use(grid)
        for _ in range(3):
            ref = A.stencil(jac, bnd, ref)
        check("stencil-" + name, np.concatenate(parts), oracle.run(ref))
    # stencil2 over slabs
    grid2 = rng.integers(0, 100, size=(rows * world, 9)).astype(np.int64)
    slab2 = ex.from_host(grid2[rank * rows:(rank + 1) * rows])
    f2 = lambda s, t: s[0][1] + t[2][1] + s[1][0] * t[1][2] - s[1][1]  # noqa: E731
    out = ex.to_host(sh.stencil2(f2, A.mirror, slab, A.mirror, slab2))
    parts = [None] * world
    dist.all_gather_object(parts, out)
    check("stencil2", np.concatenate(parts), oracle.run(A.stencil2(f2, A.mirror, grid, A.mirror, grid2)))
    # the same from the resident halo layout (slabs distributed once with room for halo rows)
    h1, h2 = sh.halo_slab(slab, A.mirror), sh.halo_slab(slab2, A.mirror)
    out = ex.to_host(sh.stencil2(f2, A.mirror, h1, A.mirror, h2))
    parts = [None] * world
    dist.all_gather_object(parts, out)
    check("stencil2-halo-layout", np.concatenate(parts), oracle.run(A.stencil2(f2, A.mirror, grid, A.mirror, grid2)))
    out = ex.to_host(sh.stencil_iterate(jac, A.clamp, sh.halo_slab(slab, A.clamp), 2, key="sthalo"))
    parts = [None] * world
    dist.all_gather_object(parts, out)
    check("stencil-halo-layout", np.concatenate(parts), oracle.run(A.stencil(jac, A.clamp, A.stencil(jac, A.clamp, A.use(grid)))))
    # segment split falls on segment boundaries
    off = np.concatenate([[0], np.cumsum(rng.integers(0, 9, size=50))])
    cuts = split_segments(off, world)
    if cuts[0] != 0 or cuts[-1] != 50 or any(b < a for a, b in zip(cuts, cuts[1:])):
        fails.append("split_segments")
    res = [None] * world
    dist.all_gather_object(res, fails)
    dist.destroy_process_group()
    if rank == 0:
        bad = [f for r in res for f in r]
        print("SHARDED_OK" if not bad else "SHARDED_FAIL " + ",".join(bad))
    sys.exit(0)


GPU = len(sys.argv) > 4 and sys.argv[4].startswith("gpu")

if __name__ == "__main__":
    main(int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3]))
