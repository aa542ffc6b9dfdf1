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


def zipf_keys(rng, n, bins, s=1.1):
    """Zipf(s) over ranks 1..bins by inverse CDF on a 2^24-entry quantile table; bin = rank-1."""
    p = 1.0 / np.arange(1, bins + 1, dtype=np.float64) ** s
    cdf = np.cumsum(p / p.sum())
    table = np.searchsorted(cdf, (np.arange(1 << 24) + 0.5) / (1 << 24)).astype(np.int32)
    table = np.minimum(table, bins - 1)
    return tiled(lambda m: table[rng.integers(0, 1 << 24, size=m)], n, np.int32)


class Workload:
    def __init__(self, name, config, inputs, build, elements, alg_bytes, kernel, launches):
        self.name, self.config, self.inputs, self.build = name, config, inputs, build
        self.elements, self.alg_bytes, self.kernel, self.launches = elements, alg_bytes, kernel, launches


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
        g = np.random.default_rng(seed2 + 1000 * rank)
        return lambda: tiled(lambda m: g.random(size=m, dtype=np.float32), side * side_c, np.float32).reshape(side, side_c)

    def jac(m):
        for _ in range(iters):
            m = A.stencil(jacobi, A.clamp, m)
        return m
    W.append(Workload("jacobi5_clamp_x100_f32", "configs[4]", [grid(seed)], jac, side * side_c * iters, 8 * side * side_c * iters, "acc_stencil2d", iters))
    W.append(Workload("stencil2_gauss_mirror_f32", "configs[4]", [grid(seed), grid(seed + 1)],
                      lambda a, b: A.stencil2(gauss2, A.mirror, a, A.mirror, b), side * side_c, 12 * side * side_c, "acc_stencil2d", 1))
    for w in W:
        w.bins = bins16 if w.name == "permute_hist_i32" else bins20
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
        if name == "permute_hist_i32":
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
        if name == "permute_hist_i32":
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


def cpu_baseline(scale_hint=0, budget_s=20.0):
    """The oracle (CPU restatement of the reference interpreter, 1 thread) on a
    bounded sample of every workload."""
    from oracle import oracle
    shrink = 8    # every size / 2^8: 2^20..2^22 elements per skeleton; two of the 100 Jacobi iterations
    ws = suite(scale=shrink)
    total_e, total_t, per = 0, 0.0, {}
    for w in ws:
        host = [f() for f in w.inputs]
        build = w.build
        elements = w.elements
        if w.name.startswith("jacobi"):
            build = lambda m: A.stencil(jacobi, A.clamp, A.stencil(jacobi, A.clamp, m))  # noqa: E731  (2 of the 100 iterations)
            elements = w.elements // 50
        term = build(*[A.use(h) for h in host])
        t0 = time.perf_counter()
        oracle.run(term)
        dt = time.perf_counter() - t0
        per[w.name] = elements / dt
        total_e += elements
        total_t += dt
        if total_t > budget_s * 3:
            break
    return {"value": total_e / total_t, "unit": "elements/s", "cores": 1, "kind": "port",
            "sample": f"every workload at 1/{1 << shrink} of its size (Jacobi: 2 iterations), {total_t:.1f} s of CPU work",
            "per_skeleton": per}


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    t0 = time.perf_counter()
    vals = []
    cb = None
    step_ms = []
    for _ in range(max(1, min(args.steps, 2))):
        t1 = time.perf_counter()
        cb = cpu_baseline()
        step_ms.append((time.perf_counter() - t1) * 1e3)
        vals.append(cb["value"])
    v = float(np.mean(vals))
    cb["value"] = v
    line = {"impl": "reference", "metric": "elements/s over the configs[1-4] skeleton suite", "value": v, "unit": "elements/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": float(np.mean(step_ms)), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "i32/i64/f32", "data": "synthetic",
            "config": {"workload": "configs[1-4] skeleton suite", "sample": cb["sample"],
                       "note": "CPU restatement of Data.Array.Accelerate.Interpreter (oracle/), 1 thread like the interpreter; the Haskell reference cannot be built here"},
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
    ws = suite(args.scale, rank=rank)
    if args.only:
        ws = [w for w in ws if any(s in w.name for s in args.only.split(","))]
    t_gen = time.perf_counter()
    bound = []
    sharded = None
    if world > 1:
        from accelerate_b200.sharded import GpuExecutor, Sharded
        sharded = Sharded(GpuExecutor(ctx))
    for w in ws:
        b = ShardedBound(sharded, w, [f() for f in w.inputs]) if sharded else Bound(ctx, w, [f() for f in w.inputs])
        b.upload()
        bound.append(b)
    ctx.sync()
    t_gen = time.perf_counter() - t_gen

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
        for b in bound:
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
    total_ms = e_start.elapsed_time(e_end)
    if dist is not None:
        t = torch.tensor([total_ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    per_ms = [float(np.mean([ev[s][k][0].elapsed_time(ev[s][k][1]) for s in range(args.steps)])) for k in range(len(bound))]
    per_ms_min = [float(np.min([ev[s][k][0].elapsed_time(ev[s][k][1]) for s in range(args.steps)])) for k in range(len(bound))]
    elements_step = sum(w.elements for w in ws) * world
    value = elements_step * args.steps / (total_ms * 1e-3)
    peak, peak_kind = measured_peaks()
    per = {}
    for w, ms, ms_min in zip(ws, per_ms, per_ms_min):
        gbs = w.alg_bytes / (ms * 1e-3) / 1e9
        per[w.name] = {"ms": round(ms, 4), "ms_fastest_step": round(ms_min, 4), "elements_per_s": w.elements / (ms * 1e-3), "achieved_gbs": round(gbs, 1),
                       "frac_of_hbm_peak": round(gbs / peak, 4), "config": w.config}
    # dominant kernel: the one with the largest share of the step
    dom = int(np.argmax(per_ms))
    wd = ws[dom]
    many = wd.launches > 3        # the Jacobi workload is 100 launches of the same kernel
    launch_ms = per_ms[dom] / wd.launches if many else per_ms[dom]
    achieved = wd.alg_bytes / (wd.launches if many else 1) / (launch_ms * 1e-3) / 1e9
    # DRAM bytes per launch of the Jacobi kernel from the ncu capture summarised in
    # profiles/acc_stencil2d_jacobi5_clamp.md (8192^2 case: 493.4 MB; traffic grows with the points: x4 at 16384^2)
    traffic = 493.4e6 * 4 if (wd.name.startswith("jacobi") and args.scale == 0) else None
    roofline = {"bound": "hbm", "kernel": wd.kernel, "workload": wd.name, "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                "frac": round(achieved / peak, 4), "peak_kind": f"of {peak_kind}", "traffic": traffic,
                "launch_ms": round(launch_ms, 4)}

    # end to end: pinned host buffers in, results back to pinned host buffers
    e2e = None
    if not args.no_e2e:
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
                                                   "frac_of_hbm_peak": round(gbs / peak, 4),
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
                           "l2": "every input is larger than L2 (126 MB); no flush", "per_gpu_elements_per_step": sum(w.elements for w in ws),
                           "parallelism": f"dp{world}", "setup_s": round(t_gen, 1)},
                "roofline": roofline, "per_skeleton": per, "gpu_launches": int(launches), "clocks": clocks, "e2e": e2e, "cpu_baseline": cb,
                "config0_dotp": c0}
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()
    ctx.close()


if __name__ == "__main__":
    main()
