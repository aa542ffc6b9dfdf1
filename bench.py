#!/usr/bin/env python
"""Benchmark of the hot path: every skeleton of the benchmark specification's
configs[1-4] on synthetic inputs of the stated shapes and distributions.

One *step* is one pass over the suite: fold1Seg(+) i32 2^28, fold max
65536x4096 f32, scanl1(+) i32 2^30, scanl'(+) f32 2^28, scanr1 max i64 2^28,
permute(+) histogram 2^30 Zipf(1.1) keys -> 2^16 bins, permute(+) f32 2^30
(dst = key mod 2^20, ~10 % dropped), 100 Jacobi iterations on 16384^2 f32 and
one stencil2 on two such arrays.  `value` counts elements (points x iterations
for Jacobi) per second with inputs resident in HBM; `e2e` is the same suite
through the public API with pinned HOST buffers (H2D and D2H inside the timed
region).  Every input is larger than the 126 MB L2, so no flush is needed
between iterations.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--scale S] [--impl reference]

`--scale S` divides every size by 2^S (for quick checks; the reported config
says so).  `--impl reference` times the CPU restatement of the reference
interpreter (the reference itself is Haskell and cannot be built here) on a
bounded sample of the same suite.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
os.environ.setdefault("ACCELERATE_B200_CACHE_DIR", os.path.join(ROOT, ".kernel_cache"))

import accelerate_b200 as A  # noqa: E402

add = lambda a, b: a + b  # noqa: E731
GAUSS = [[1, 2, 1], [2, 4, 2], [1, 2, 1]]


def jacobi(s):
    return 0.25 * (s[0][1] + s[2][1] + s[1][0] + s[1][2])


def gauss2(s, t):
    acc = A.constant(np.float32(0))
    for i in range(3):
        for j in range(3):
            acc = acc + np.float32(GAUSS[i][j] / 16.0) * (s[i][j] + t[i][j])
    return acc


# ---------------------------------------------------------------------------------
# synthetic inputs (seeded; large arrays repeat a seeded 2^24-element block so that
# host-side generation stays within seconds)
# ---------------------------------------------------------------------------------
BLOCK = 1 << 24


def tiled(gen, n, dtype):
    if n <= BLOCK:
        return gen(n).astype(dtype)
    b = gen(BLOCK).astype(dtype)
    return np.tile(b, (n + BLOCK - 1) // BLOCK)[:n]


def zipf_keys(rng, n, bins, s=1.1, shuffle=False):
    """Zipf(s) over ranks 1..bins by inverse CDF on a 2^24-entry quantile table; bin = rank-1, or,
    with ``shuffle``, a fixed (seeded) permutation of the bins applied to rank-1, so that the
    frequent keys are scattered over the whole target instead of sitting at its start."""
    p = 1.0 / np.arange(1, bins + 1, dtype=np.float64) ** s
    cdf = np.cumsum(p / p.sum())
    table = np.searchsorted(cdf, (np.arange(1 << 24) + 0.5) / (1 << 24)).astype(np.int32)
    table = np.minimum(table, bins - 1)
    if shuffle:
        table = np.random.default_rng(7).permutation(bins).astype(np.int32)[table]
    return tiled(lambda m: table[rng.integers(0, 1 << 24, size=m)], n, np.int32)


def make_grid(seed2, rank, side, side_c):
    """Rank `rank`'s (side x side_c) slab of the stencil input with seed `seed2`."""
    g = np.random.default_rng(seed2 + 1000 * rank)
    return tiled(lambda m: g.random(size=m, dtype=np.float32), side * side_c, np.float32).reshape(side, side_c)


class Workload:
    def __init__(self, name, config, inputs, build, elements, alg_bytes, kernel, launches, in_value=True):
        self.name, self.config, self.inputs, self.build = name, config, inputs, build
        self.elements, self.alg_bytes, self.kernel, self.launches = elements, alg_bytes, kernel, launches
        self.in_value = in_value      # False: reported beside the suite, not part of `value`


def suite(scale=0, seed=42, rank=0):
    """The nine workloads.  `inputs` are thunks producing host arrays."""
    rng = np.random.default_rng(seed + 1000 * rank)
    sh = lambda e: max(e - scale, 8)  # noqa: E731
    n28, n30 = 1 << sh(28), 1 << sh(30)
    rows, cols = 1 << sh(16) if scale == 0 else max(1 << (16 - scale // 2 - scale % 2), 16), 1 << (12 if scale == 0 else max(12 - scale // 2, 6))
    side = 1 << (14 - (scale + 1) // 2) if scale else 16384
    side_c = 1 << (14 - scale // 2) if scale else 16384
    bins16 = 1 << 16 if scale == 0 else max(1 << (16 - scale // 2), 64)
    bins20 = 1 << 20 if scale == 0 else max(1 << (20 - scale // 2), 64)
    iters = 100
    W = []

    def seg_lengths():
        ls, tot = [], 0
        while tot < n28:
            c = rng.integers(1, 2049, size=max(1024, n28 // 1024 + 1024))
            ls.append(c)
            tot += int(c.sum())
        l = np.concatenate(ls)
        cs = np.cumsum(l)
        k = int(np.searchsorted(cs, n28))
        l = l[:k + 1].copy()
        l[k] -= cs[k] - n28
        return l[l > 0].astype(np.int32)

    W.append(Workload("fold1seg_add_i32", "configs[1]", [lambda: tiled(lambda m: rng.integers(-1000, 1000, size=m), n28, np.int32), seg_lengths],
                      lambda v, l: A.fold1Seg(add, v, l), n28, 4 * n28, "acc_foldseg", 3))
    W.append(Workload("fold_max_rows_f32", "configs[1]", [lambda: tiled(lambda m: rng.standard_normal(size=m, dtype=np.float32), rows * cols, np.float32).reshape(rows, cols)],
                      lambda m: A.fold1(A.max_, m), rows * cols, 4 * rows * cols, "acc_fold_rows", 1))
    W.append(Workload("scanl1_add_i32", "configs[2]", [lambda: tiled(lambda m: rng.integers(0, 100, size=m), n30, np.int32)],
                      lambda x: A.scanl1(add, x), n30, 8 * n30, "acc_scan", 1))
    W.append(Workload("scanl_prime_add_f32", "configs[2]", [lambda: tiled(lambda m: rng.random(size=m, dtype=np.float32), n28, np.float32)],
                      lambda x: list(A.scanl_prime(add, 0.0, x)), n28, 8 * n28, "acc_scan", 1))
    W.append(Workload("scanr1_max_i64", "configs[2]", [lambda: tiled(lambda m: rng.integers(np.iinfo(np.int64).min, np.iinfo(np.int64).max, size=m, dtype=np.int64), n28, np.int64)],
                      lambda x: A.scanr1(A.max_, x), n28, 16 * n28, "acc_scan", 1))
    W.append(Workload("permute_hist_i32", "configs[3]", [lambda: zipf_keys(rng, n30, bins16)],
                      lambda k: A.permute(add, A.fill(bins16, A.constant(np.int32(0))), lambda ix: A.Just_(A.index(A.from_integral(k[ix], "i64"))),
                                          A.fill(k.shape, A.constant(np.int32(1)))), n30, 4 * n30, "acc_permute", 2))

    def signed_keys():
        k = tiled(lambda m: rng.integers(0, 1 << 31, size=m), n30, np.int32)
        drop = tiled(lambda m: rng.random(size=m) < 0.1, n30, np.bool_)
        k[drop] = -k[drop] - 1          # a negative key means "ignore" (~10 %)
        return k
    W.append(Workload("permute_add_f32", "configs[3]", [signed_keys, lambda: tiled(lambda m: rng.random(size=m, dtype=np.float32), n30, np.float32)],
                      lambda k, v: A.permute(add, A.fill(bins20, A.constant(np.float32(0))),
                                             lambda ix: A.cond(k[ix] < 0, A.Nothing_(1), A.Just_(A.index(A.from_integral(k[ix], "i64") % bins20))), v),
                      n30, 8 * n30, "acc_permute", 2))

    def grid(seed2):
        return lambda: make_grid(seed2, rank, side, side_c)

    def jac(m):
        for _ in range(iters):
            m = A.stencil(jacobi, A.clamp, m)
        return m
    W.append(Workload("jacobi5_clamp_x100_f32", "configs[4]", [grid(seed)], jac, side * side_c * iters, 8 * side * side_c * iters, "acc_stencil2d", iters))
    W.append(Workload("stencil2_gauss_mirror_f32", "configs[4]", [grid(seed), grid(seed + 1)],
                      lambda a, b: A.stencil2(gauss2, A.mirror, a, A.mirror, b), side * side_c, 12 * side * side_c, "acc_stencil2d", 1))
    # the same histogram with the bins shuffled (reported beside the suite; `value` keeps the rank-1 layout)
    hist_build = W[5].build
    W.append(Workload("permute_hist_i32_shuffled", "configs[3]", [lambda: zipf_keys(np.random.default_rng(seed + 77 + 1000 * rank), n30, bins16, shuffle=True)],
                      hist_build, n30, 4 * n30, "acc_permute", 2, in_value=False))
    for w in W:
        w.bins = bins16 if w.name.startswith("permute_hist_i32") else bins20
        w.iters, w.side, w.scale, w.seed = iters, (side, side_c), scale, seed
    return W


class Bound:
    """A workload bound to a context: program text, resident inputs."""

    def __init__(self, ctx, w, host):
        from accelerate_b200 import language as L
        self.w, self.ctx, self.host = w, ctx, host
        L.reset_names()
        params = [L.param(h.ndim, L.TY_OF_NP[h.dtype]) for h in host]
        res = w.build(*params)
        self.prog = L.build_program(res)
        self.order = [next(i for i, q in enumerate(params) if q.node is n) for n in self.prog.inputs]
        self.dev = None

    def upload(self):
        self.dev = [self.ctx.from_host(self.host[k]) for k in self.order]

    def run(self):
        return self.ctx.execute(self.prog.text, self.dev, len(self.prog.outputs))

    def run_e2e(self, out_bufs):
        dev = [self.ctx.from_host(self.host[k]) for k in self.order]
        outs = self.ctx.execute(self.prog.text, dev, len(self.prog.outputs))
        res = []
        for k, o in enumerate(outs):
            buf = out_bufs[k] if out_bufs is not None else None
            # results go back on the copy-out stream while the next workload's inputs come in
            res.append(o.download_async([buf]) if buf is not None else o.download())
        return res


def strong_part(w, host, world):
    """The first 1/world of a rank's inputs: this rank's part when the config size is split over the ranks."""
    if w.name == "fold1seg_add_i32":
        vals, lens = host
        c = np.cumsum(lens, dtype=np.int64)
        k = max(1, int(np.searchsorted(c, vals.size // world, side="right")))
        return [vals[:int(c[k - 1])], lens[:k]]
    return [h[:max(1, h.shape[0] // world)] for h in host]


class ShardedBound:
    """A workload on one rank of a multi-GPU run: this rank's shard is resident; each run does
    the local kernels plus the skeleton's one exchange step (accelerate_b200.sharded)."""

    def __init__(self, sh, w, host):
        self.sh, self.w, self.host = sh, w, host
        self.dev = None
        self.aux = {}

    def upload(self):
        ex = self.sh.ex
        self.dev = [ex.from_host(h) for h in self.host]
        name = self.w.name
        if name.startswith("permute_hist_i32"):
            self.aux["defaults"] = ex.from_host(np.zeros(self.w.bins, np.int32))
        if name == "permute_add_f32":
            self.aux["defaults"] = ex.from_host(np.zeros(self.w.bins, np.float32))
        # stencil inputs are resident as row slabs with room for the neighbours' halo rows
        if name == "jacobi5_clamp_x100_f32":
            self.dev = [self.sh.halo_slab(self.dev[0], A.clamp, key="c4a")]
        if name == "stencil2_gauss_mirror_f32":
            self.dev = [self.sh.halo_slab(x, A.mirror, key="c4b") for x in self.dev]

    def run_e2e(self, out_bufs):
        """Host shard in, this rank's part of the result back to the host."""
        for d in (self.dev or []):
            if hasattr(d, "free"):
                d.free()
        self.upload()
        r = self.run()
        outs = list(r) if isinstance(r, (list, tuple)) else [r]
        res = []
        for k, o in enumerate(outs):
            buf = out_bufs[k] if out_bufs is not None and k < len(out_bufs) else None
            res.append(o.download_async([buf]) if buf is not None else o.download())
        self.dev = None
        return res

    def run(self):
        sh, d, name = self.sh, self.dev, self.w.name
        ex = sh.ex
        if name == "fold1seg_add_i32":
            return ex.run("c1a", lambda v, l: A.fold1Seg(add, v, l), d)            # segments never straddle ranks
        if name == "fold_max_rows_f32":
            return ex.run("c1b", lambda m: A.fold1(A.max_, m), d)                  # row blocks
        if name == "scanl1_add_i32":
            return sh.scan1d("scanl1", add, None, d[0], key="c2a")
        if name == "scanl_prime_add_f32":
            return sh.scan1d("scanl'", add, 0.0, d[0], key="c2b")
        if name == "scanr1_max_i64":
            return sh.scan1d("scanr1", A.max_, None, d[0], key="c2c")
        if name.startswith("permute_hist_i32"):
            return sh.permute("add", self.aux["defaults"], lambda ix, k: A.Just_(A.index(A.from_integral(k[ix], "i64"))), d,
                              lambda k: A.fill(k.shape, A.constant(np.int32(1))), key="c3a")
        if name == "permute_add_f32":
            bins = self.w.bins
            return sh.permute("add", self.aux["defaults"],
                              lambda ix, k, v: A.cond(k[ix] < 0, A.Nothing_(1), A.Just_(A.index(A.from_integral(k[ix], "i64") % bins))), d,
                              lambda k, v: v, key="c3b")
        if name == "jacobi5_clamp_x100_f32":
            return sh.stencil_iterate(jacobi, A.clamp, d[0], 100, key="c4a")
        if name == "stencil2_gauss_mirror_f32":
            return sh.stencil2(gauss2, A.mirror, d[0], A.mirror, d[1], key="c4b")
        raise KeyError(name)


# ---------------------------------------------------------------------------------
# parity of what was timed: every rank checks its part of every result against NumPy
# (integers bit-exact; Float sums within 1e-5 * sqrt(n) relative; stencils bit-exact on
# blocks that include the array's corners and the rows either side of every slab edge)
# ---------------------------------------------------------------------------------
def _gather(x, rank, world, dist, dtype):
    """Every rank's scalar `x` as a NumPy vector."""
    if world == 1:
        return np.array([x], dtype)
    import torch
    t = torch.zeros(world, dtype=torch.float64 if np.dtype(dtype).kind == "f" else torch.int64, device="cuda")
    t[rank] = float(x) if np.dtype(dtype).kind == "f" else int(x)
    dist.all_reduce(t)
    return t.cpu().numpy().astype(dtype)


def _allreduce_np(a, world, dist):
    if world == 1:
        return a
    import torch
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    dist.all_reduce(t)
    return t.cpu().numpy()


def _stencil_blocks(w, rank, world, got, apply_np, mode, seeds, iters, radius=1):
    """Compare blocks of this rank's result slab with NumPy.  The expected block is computed from the
    input window `iters * radius` wider on every side (taken from the neighbouring ranks' slabs where
    it crosses a slab edge): after `iters` applications everything further than that from a window
    edge that is not an edge of the whole array is exact."""
    side, side_c = w.side
    grids = {}

    def rows(seed2, lo, hi):
        parts = []
        for r in range(lo // side, (hi - 1) // side + 1):
            if (seed2, r) not in grids:
                grids[(seed2, r)] = make_grid(seed2, r, side, side_c)
            parts.append(grids[(seed2, r)][max(lo - r * side, 0):min(hi - r * side, side)])
        return np.concatenate(parts, axis=0)

    H, B, halo = world * side, min(64, side // 2), iters * radius
    base = rank * side
    blocks = [(base, 0), (base + side - B, side_c - B), (base + side // 2, side_c // 2 - B // 2)]
    for (r0, c0) in blocks:
        lo, hi = max(r0 - halo, 0), min(r0 + B + halo, H)
        cl, ch = max(c0 - halo, 0), min(c0 + B + halo, side_c)
        wins = [rows(sd, lo, hi)[:, cl:ch].copy() for sd in seeds]
        for _ in range(iters):
            wins = [apply_np(*[np.pad(x, radius, mode=mode) for x in wins])] + wins[1:]
        want = wins[0][r0 - lo:r0 - lo + B, c0 - cl:c0 - cl + B]
        have = got[r0 - base:r0 - base + B, c0:c0 + B]
        if not np.array_equal(want, have):
            return False
    return True


def _jacobi_np(p):
    return np.float32(0.25) * (((p[:-2, 1:-1] + p[2:, 1:-1]) + p[1:-1, :-2]) + p[1:-1, 2:])


def _gauss2_np(p, q):
    acc = np.zeros((p.shape[0] - 2, p.shape[1] - 2), np.float32)
    for i in range(3):
        for j in range(3):
            acc = acc + np.float32(GAUSS[i][j] / 16.0) * (p[i:p.shape[0] - 2 + i, j:p.shape[1] - 2 + j] + q[i:q.shape[0] - 2 + i, j:q.shape[1] - 2 + j])
    return acc


def verify(w, host, outs, rank, world, dist):
    """True if this rank's part of workload `w`'s result (`outs`: host arrays) is right."""
    name = w.name
    if name == "fold1seg_add_i32":
        vals, lens = host
        offs = np.concatenate([[0], np.cumsum(lens, dtype=np.int64)[:-1]])
        return np.array_equal(outs[0], np.add.reduceat(vals.astype(np.int64), offs).astype(np.int32))
    if name == "fold_max_rows_f32":
        return np.array_equal(outs[0], host[0].max(axis=1))
    if name == "scanl1_add_i32":
        x = host[0]
        tot = _gather(int(x.sum(dtype=np.int64)), rank, world, dist, np.int64)
        carry = np.uint32(int(tot[:rank].sum()) & 0xffffffff)
        want = (np.cumsum(x.view(np.uint32), dtype=np.uint32) + carry).view(np.int32)
        return np.array_equal(outs[0], want)
    if name == "scanl_prime_add_f32":
        x = host[0]
        tot = _gather(float(x.sum(dtype=np.float64)), rank, world, dist, np.float64)
        c = np.cumsum(x, dtype=np.float64)
        want = c - x + tot[:rank].sum()
        tol = min(1e-5 * np.sqrt(float(x.size) * world), 1e-4)      # the specification's bound, capped: a tree scan is far inside it
        ok = bool(np.all(np.abs(outs[0] - want) <= tol * np.maximum(np.abs(want), 1.0)))
        return ok and abs(float(outs[1]) - tot.sum()) <= tol * tot.sum()
    if name == "scanr1_max_i64":
        x = host[0]
        mx = _gather(int(x.max()), rank, world, dist, np.int64)
        want = np.maximum.accumulate(x[::-1])[::-1]
        if rank + 1 < world:
            want = np.maximum(want, mx[rank + 1:].max())
        return np.array_equal(outs[0], want)
    if name.startswith("permute_hist_i32"):
        k = host[0]
        want = np.zeros(w.bins, np.int64)
        for a in range(0, k.size, 1 << 26):
            want += np.bincount(k[a:a + (1 << 26)], minlength=w.bins)
        return np.array_equal(outs[0], _allreduce_np(want, world, dist).astype(np.int32))
    if name == "permute_add_f32":
        k, v = host
        want = np.zeros(w.bins, np.float64)
        for a in range(0, k.size, 1 << 26):
            kk, vv = k[a:a + (1 << 26)], v[a:a + (1 << 26)]
            keep = kk >= 0
            want += np.bincount(kk[keep] % w.bins, weights=vv[keep].astype(np.float64), minlength=w.bins)
        want = _allreduce_np(want, world, dist)
        tol = 1e-5 * np.sqrt(max(float(k.size) * world / w.bins, 1.0))
        return bool(np.all(np.abs(outs[0] - want) <= tol * np.maximum(np.abs(want), 1.0)))
    if name == "jacobi5_clamp_x100_f32":
        return _stencil_blocks(w, rank, world, outs[0], _jacobi_np, "edge", [w.seed], w.iters)
    if name == "stencil2_gauss_mirror_f32":
        return _stencil_blocks(w, rank, world, outs[0], _gauss2_np, "reflect", [w.seed, w.seed + 1], 1)
    raise KeyError(name)


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled while the timed region runs."""

    def __init__(self, index):
        self.rows, self.proc, self.index = [], None, index

    def start(self):
        q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.index)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def mark(self):
        """The timed region starts here (the sampler itself is started before the warm-up, so
        that nvidia-smi is already delivering samples when a short timed region begins)."""
        self.first = len(self.rows)

    def stop(self):
        if self.proc:
            self.proc.terminate()
        first = getattr(self, "first", 0)
        rows, window = self.rows[first:], "timed region"
        if len(rows) < 2:
            # the region was shorter than two sampling periods: add the samples just before it,
            # taken while the warm-up ran the same kernels
            rows, window = self.rows[max(0, first - 5):], "timed region and the end of the warm-up"
        sm = [float(r[0]) for r in rows if r and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for k, n in enumerate(names) if any(len(r) > 3 + k and r[3 + k].lower().startswith("active") for r in rows)]
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons, "samples": len(sm),
                "window": window}


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return json.load(open(p)).get("hbm_gbs", 6650.0), "measured"
    return 6650.0, "fallback"


NOMINAL_HBM_GBS = 8000.0       # the nominal HBM3e figure the benchmark specification quotes


def _cpu_one(args):
    """One workload on the CPU oracle (runs in a worker process); returns (name, elements, seconds)."""
    k, shrink = args
    from oracle import oracle
    ws = [w for w in suite(scale=shrink) if w.in_value]
    # the shared generator is consumed in suite order: draw the earlier workloads' inputs too
    for w in ws[:k]:
        for f in w.inputs:
            f()
    w = ws[k]
    host = [f() for f in w.inputs]
    build, elements = w.build, w.elements
    if w.name.startswith("jacobi"):
        build = lambda m: A.stencil(jacobi, A.clamp, A.stencil(jacobi, A.clamp, m))  # noqa: E731  (2 of the 100 iterations)
        elements = w.elements // 50
    term = build(*[A.use(h) for h in host])
    t0 = time.perf_counter()
    oracle.run(term)
    return w.name, elements, time.perf_counter() - t0


def cpu_baseline(shrink=8, workers=1):
    """The oracle (CPU restatement of the reference interpreter) on a bounded sample of every
    workload: every size / 2^shrink, two of the 100 Jacobi iterations.  The interpreter is
    sequential; with `workers` > 1 the workloads of the suite run side by side, one per host
    thread, and the step takes as long as the slowest of them."""
    from oracle import oracle
    oracle.build()
    n = len([w for w in suite(scale=shrink) if w.in_value])
    jobs = [(k, shrink) for k in range(n)]
    if workers > 1:
        import multiprocessing as mp
        with mp.get_context("fork").Pool(min(workers, n)) as pool:
            res = pool.map(_cpu_one, jobs, chunksize=1)
        step_s = max(r[2] for r in res)
        cores = min(workers, n)
    else:
        res = [_cpu_one(j) for j in jobs]
        step_s = sum(r[2] for r in res)
        cores = 1
    total_e = sum(r[1] for r in res)
    return {"value": total_e / step_s, "unit": "elements/s", "cores": cores, "kind": "port",
            "sample": f"every workload at 1/{1 << shrink} of its size (Jacobi: 2 iterations), {sum(r[2] for r in res):.1f} s of CPU work"
                      + (f" spread over {cores} host threads (one workload each)" if cores > 1 else ""),
            "per_skeleton": {r[0]: r[1] / r[2] for r in res}, "step_s": step_s}


def reference_arm(args):
    """The reference's CPU path: the oracle port (the Haskell interpreter cannot be built here), every
    workload of the suite on its own host thread.  Runs the warm-up and the steps it is asked for."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    t0 = time.perf_counter()
    workers = min(9, os.cpu_count() or 1)
    shrink = 9
    for _ in range(args.warmup):
        cb = cpu_baseline(shrink, workers)
    vals, step_ms = [], []
    for _ in range(max(1, args.steps)):
        cb = cpu_baseline(shrink, workers)
        step_ms.append(cb["step_s"] * 1e3)
        vals.append(cb["value"])
    v = float(np.mean(vals))
    cb["value"] = v
    line = {"impl": "reference", "metric": "elements/s over the configs[1-4] skeleton suite", "value": v, "unit": "elements/s",
            "n_gpus": args.gpus, "steps": max(1, args.steps), "warmup": args.warmup, "ms_per_step": float(np.mean(step_ms)), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "i32/i64/f32", "data": "synthetic",
            "config": {"workload": "configs[1-4] skeleton suite", "sample": cb["sample"],
                       "note": "CPU restatement of Data.Array.Accelerate.Interpreter (oracle/); the Haskell reference cannot be built here"},
            "cpu_baseline": {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": v, "unit": "elements/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "wall_s": time.perf_counter() - t0}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--scale", type=int, default=0)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-verify", action="store_true")
    ap.add_argument("--no-strong", action="store_true", help="N > 1: skip the strong-scaling pass")
    ap.add_argument("--only", default="")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    import torch
    from accelerate_b200 import backend
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ctx = backend.Context(local)
    stream = torch.cuda.ExternalStream(ctx.stream(), device=torch.device("cuda", local))
    ws_all = suite(args.scale, rank=rank)
    if args.only:
        ws_all = [w for w in ws_all if any(s in w.name for s in args.only.split(","))]
    t_gen = time.perf_counter()
    bound_all = []
    sharded = None
    if world > 1:
        from accelerate_b200.sharded import GpuExecutor, Sharded
        sharded = Sharded(GpuExecutor.with_group(ctx))     # exchange steps inside the C-ABI library (NCCL)
    for w in ws_all:
        b = ShardedBound(sharded, w, [f() for f in w.inputs]) if sharded else Bound(ctx, w, [f() for f in w.inputs])
        b.upload()
        bound_all.append(b)
    ctx.sync()
    t_gen = time.perf_counter() - t_gen
    bound = [b for b in bound_all if b.w.in_value]
    if bound:
        # A step starts with its longest workload: the timed region opens on an idle GPU (barrier), and the host's
        # latency of the first launches would otherwise be charged to a workload of 0.2 ms.
        k0 = int(np.argmax([b.w.alg_bytes for b in bound]))
        bound = [bound[k0]] + bound[:k0] + bound[k0 + 1:]
    ws = [b.w for b in bound]
    extra = [b for b in bound_all if not b.w.in_value]

    def barrier():
        ctx.sync()
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        ctx.sync()

    # warm-up (compiles kernels on first use)
    sampler = ClockSampler(local)
    sampler.start()
    for _ in range(max(args.warmup, 1)):
        for b in bound_all:
            b.run()
    barrier()
    l0 = ctx.stats()["launches"]
    ev = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in bound] for _ in range(args.steps)]
    e_start, e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    sampler.mark()
    e_start.record(stream)
    for s in range(args.steps):
        for k, b in enumerate(bound):
            ev[s][k][0].record(stream)
            b.run()
            ev[s][k][1].record(stream)
    e_end.record(stream)
    barrier()
    clocks = sampler.stop()
    launches = ctx.stats()["launches"] - l0
    total_ms = e_start.elapsed_time(e_end) if bound else 0.0
    if dist is not None:
        t = torch.tensor([total_ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    per_ms = [float(np.mean([ev[s][k][0].elapsed_time(ev[s][k][1]) for s in range(args.steps)])) for k in range(len(bound))]
    per_ms_min = [float(np.min([ev[s][k][0].elapsed_time(ev[s][k][1]) for s in range(args.steps)])) for k in range(len(bound))]
    per_steps = [[round(float(ev[s][k][0].elapsed_time(ev[s][k][1])), 4) for s in range(args.steps)] for k in range(len(bound))]
    # workloads reported beside the suite (not part of `value`): timed the same way, after it
    ex_ms, ex_min = [], []
    for b in extra:
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
        barrier()
        for s in range(args.steps):
            evs[s][0].record(stream)
            b.run()
            evs[s][1].record(stream)
        barrier()
        ts = [a.elapsed_time(z) for a, z in evs]
        if dist is not None:
            t = torch.tensor(ts, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ts = [float(x) for x in t.tolist()]
        ex_ms.append(float(np.mean(ts)))
        ex_min.append(float(np.min(ts)))
        per_steps.append([round(float(t), 4) for t in ts])
    # The same workloads once more, each run `steps` + 1 times in a row (the first run left out).  In the suite a
    # workload also pays for what its predecessor left behind (the write-back of up to 126 MB of dirty L2 lines
    # after a kernel that writes a grid); run after itself it pays for its own output, which is the figure to hold
    # against its own roofline.  `value` is not affected.
    rep_ms = {}
    for b in bound:
        n_rep = max(args.steps, 2) + 1
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n_rep)]
        barrier()
        for a_, z_ in evs:
            a_.record(stream)
            b.run()
            z_.record(stream)
        barrier()
        ts = [a_.elapsed_time(z_) for a_, z_ in evs][1:]
        if dist is not None:
            t = torch.tensor(ts, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ts = [float(x) for x in t.tolist()]
        rep_ms[b.w.name] = float(np.mean(ts))
    elements_step = sum(w.elements for w in ws) * world
    value = elements_step * args.steps / (total_ms * 1e-3) if bound else 0.0
    peak, peak_kind = measured_peaks()
    per = {}
    for (w, ms, ms_min), steps_ms in zip(list(zip(ws, per_ms, per_ms_min)) + list(zip([b.w for b in extra], ex_ms, ex_min)), per_steps):
        gbs = w.alg_bytes / (ms * 1e-3) / 1e9
        per[w.name] = {"ms": round(ms, 4), "ms_fastest_step": round(ms_min, 4), "ms_steps": steps_ms[:32], "elements_per_s": w.elements / (ms * 1e-3), "achieved_gbs": round(gbs, 1),
                       "frac_of_hbm_peak": round(gbs / peak, 4), "frac_of_nominal_8tbs": round(gbs / NOMINAL_HBM_GBS, 4), "config": w.config,
                       "in_value": w.in_value}
        if w.name in rep_ms:
            per[w.name]["ms_run_after_itself"] = round(rep_ms[w.name], 4)
            per[w.name]["frac_of_hbm_peak_run_after_itself"] = round(w.alg_bytes / (rep_ms[w.name] * 1e-3) / 1e9 / peak, 4)
    roofline = None
    if bound:
        # dominant kernel: the one with the largest share of the step
        dom = int(np.argmax(per_ms))
        wd = ws[dom]
        many = wd.launches > 3        # the Jacobi workload is 100 launches of the same kernel
        launch_ms = per_ms[dom] / wd.launches if many else per_ms[dom]
        achieved = wd.alg_bytes / (wd.launches if many else 1) / (launch_ms * 1e-3) / 1e9
        # DRAM bytes per launch of the Jacobi kernel, scaled from an ncu capture of the 8192^2 case
        # (493.4 MB per launch there; traffic grows with the number of points: x4 at 16384^2)
        jac_full = wd.name.startswith("jacobi") and args.scale == 0
        roofline = {"bound": "hbm", "kernel": wd.kernel, "workload": wd.name, "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                    "frac": round(achieved / peak, 4), "peak_kind": f"of {peak_kind}", "frac_of_nominal_8tbs": round(achieved / NOMINAL_HBM_GBS, 4),
                    "traffic": 492.4e6 * 4 if jac_full else None, "traffic_from": "ncu capture of the 8192^2 case x4 (scaled, not measured at this size)" if jac_full else None,
                    "launch_ms": round(launch_ms, 4)}

    # parity of what was just timed: one more run of every workload, checked against NumPy on every rank
    parity_ok, parity_failed = None, []
    if not args.no_verify:
        for b in bound_all:
            r = b.run()
            outs = [o.download() for o in (list(r) if isinstance(r, (list, tuple)) else [r])]
            ctx.sync()
            good = bool(verify(b.w, b.host, outs, rank, world, dist))
            if dist is not None:
                t = torch.tensor([0 if good else 1], device="cuda")
                dist.all_reduce(t)
                good = int(t.item()) == 0
            if not good:
                parity_failed.append(b.w.name)
            del outs, r
        parity_ok = not parity_failed

    # strong scaling beside the weak-scaling `value`: every workload once more with the CONFIG size split over the
    # ranks (each rank takes the first 1/N of its resident shard as its part), timed the same way
    strong = None
    if sharded is not None and not args.no_strong:
        strong = {}
        for b in bound:
            hs = strong_part(b.w, b.host, world)
            sb = ShardedBound(sharded, b.w, hs)
            sb.upload()
            for _ in range(2):
                sb.run()
            evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(max(args.steps, 3))]
            barrier()
            for a_, z_ in evs:
                a_.record(stream)
                sb.run()
                z_.record(stream)
            barrier()
            t = torch.tensor([a_.elapsed_time(z_) for a_, z_ in evs], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.mean().item())
            part = sum(int(h.size) for h in hs) / max(1, sum(int(h.size) for h in b.host))
            strong[b.w.name] = {"ms": round(ms, 4), "elements_per_s": b.w.elements * part * world / (ms * 1e-3),
                                "fraction_of_config_size_per_rank": round(part, 6)}
            for d in (sb.dev or []):
                if hasattr(d, "free"):
                    d.free()
            del sb
        ctx.sync()

    # end to end: pinned host buffers in, results back to pinned host buffers
    e2e = None
    if not args.no_e2e and bound:
        for b in extra:
            for d in (b.dev or []):
                if hasattr(d, "free"):
                    d.free()
            b.dev = None
        h2d = d2h = 0
        pinned_in, outs_buf = [], []
        for b in bound:
            hs = []
            for h in b.host:
                t = torch.empty(h.shape, dtype=torch.from_numpy(np.empty(0, h.dtype)).dtype, pin_memory=True)
                t.numpy()[...] = h
                hs.append(t)
            pinned_in.append(hs)
        for b, hs in zip(bound, pinned_in):
            b.host_saved, b.host = b.host, [t.numpy() for t in hs]
            for d in b.dev:
                if hasattr(d, "free"):
                    d.free()
            b.dev = None
        ctx.sync()
        # one untimed pass to size the output buffers
        shapes = []
        for b in bound:
            r = b.run_e2e(None)
            bufs = []
            for x in r:
                t = torch.empty(x.shape, dtype=torch.from_numpy(np.empty(0, x.dtype)).dtype, pin_memory=True)
                bufs.append(t)
            shapes.append(bufs)
        barrier()
        n_e2e = max(1, min(args.steps, 2))
        s0 = ctx.stats()
        t0 = time.perf_counter()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(n_e2e):
            for b, bufs in zip(bound, shapes):
                b.run_e2e([t.numpy() for t in bufs])
        ctx.sync()            # the last results have arrived in host memory
        e1.record(stream)
        barrier()
        wall = time.perf_counter() - t0
        s1 = ctx.stats()
        ms = max(e0.elapsed_time(e1), 0.0)
        if dist is not None:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        h2d = (s1["h2d_bytes"] - s0["h2d_bytes"]) // n_e2e * world      # every rank copies a shard of the same size
        d2h = (s1["d2h_bytes"] - s0["d2h_bytes"]) // n_e2e * world
        e2e = {"value": elements_step * n_e2e / (ms * 1e-3), "unit": "elements/s", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
               "ms_per_step": ms / n_e2e, "wall_ms_per_step": wall * 1e3 / n_e2e, "steps": n_e2e}

    # configs[0] (dotp) beside the suite: the reference's own CPU-sized case, and the same fused
    # zipWith+fold at a size where bandwidth rather than launch latency decides (not part of `value`)
    c0 = None
    if world == 1 and not args.only and args.scale == 0:
        c0 = {}
        g = np.random.default_rng(42)
        for n in (1 << 20, 1 << 28):
            hx = tiled(lambda m: g.uniform(-1, 1, m), n, np.float32)
            hy = tiled(lambda m: g.uniform(-1, 1, m), n, np.float32)
            w0 = Workload("dotp", "configs[0]", [], lambda x, y: A.fold(add, 0.0, A.zipWith(lambda a, b: a * b, x, y)), n, 8 * n, "acc_fold_all", 1)
            b0 = Bound(ctx, w0, [hx, hy])
            b0.upload()
            for _ in range(3):
                b0.run()
            reps = 20
            ea, eb = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            barrier()
            ea.record(stream)
            for _ in range(reps):
                b0.run()
            eb.record(stream)
            barrier()
            ms = ea.elapsed_time(eb) / reps
            gbs = 8 * n / (ms * 1e-3) / 1e9
            c0[f"dotp_f32_2^{n.bit_length() - 1}"] = {"ms": round(ms, 4), "elements_per_s": n / (ms * 1e-3), "achieved_gbs": round(gbs, 1),
                                                   "frac_of_hbm_peak": round(gbs / peak, 4), "frac_of_nominal_8tbs": round(gbs / NOMINAL_HBM_GBS, 4),
                                                   "note": "8 MiB of input: L2-resident and launch-latency bound" if n == 1 << 20 else "2 GiB of input"}
            for d in b0.dev:
                d.free()

    cb = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cb = cpu_baseline()
        cb = {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")}

    if rank == 0:
        line = {"metric": "elements/s over the configs[1-4] skeleton suite",
                "value": value, "unit": "elements/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "i32/i64/f32", "data": "synthetic (seeded 2^24-element blocks tiled to size)",
                "config": {"workload": "configs[1-4] skeleton suite" + (f" / 2^{args.scale}" if args.scale else ""),
                           "l2": "every input is larger than L2 (126 MB); no flush", "order": [w.name for w in ws], "per_gpu_elements_per_step": sum(w.elements for w in ws),
                           "histogram_bins": "value uses bin = Zipf rank - 1; per_skeleton.permute_hist_i32_shuffled is the same histogram with the bins shuffled",
                           "parallelism": f"dp{world}", "setup_s": round(t_gen, 1)},
                "roofline": roofline, "per_skeleton": per, "gpu_launches": int(launches), "clocks": clocks,
                "parity_ok": parity_ok, "parity_failed": parity_failed, "strong_scaling": strong, "e2e": e2e, "cpu_baseline": cb,
                "config0_dotp": c0}
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()
    ctx.close()


if __name__ == "__main__":
    main()
