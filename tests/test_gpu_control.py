"""GPU parity for the nodes the reference evaluates on the host (Interpreter.hs:215-231): Use
(arrays embedded in the program text), Acond, Awhile, Apply.  Same programs as the oracle tests
(tests/control_cases.py), through the C ABI; expected values from NumPy, and the oracle beside."""
import numpy as np
import pytest

import accelerate_b200 as A
from accelerate_b200 import backend
from oracle import oracle
from tests import control_cases as C
from tests import golden_cases as G
from tests.util import similar

pytestmark = pytest.mark.gpu
CASES = C.cases()
GOLDEN = G.cases()


@pytest.mark.parametrize("embed", [False, True], ids=["inputs", "embedded-use"])
@pytest.mark.parametrize("key", sorted(CASES))
def test_gpu_control_flow(key, embed, gpu_ctx):
    term, want = CASES[key]
    got = backend.run(term, gpu_ctx, embed=embed)
    ref = oracle.run(term)
    if isinstance(term, list):
        for g, w, r in zip(got, want, ref):
            similar(g, w)
            similar(g, r)
    else:
        similar(got, want)
        similar(got, ref)


@pytest.mark.parametrize("key", sorted(GOLDEN))
def test_gpu_reference_vectors_with_embedded_use(key, gpu_ctx):
    # the haddock examples and regression tests in their original `run (... (use xs))` form
    got = backend.run(GOLDEN[key], gpu_ctx, embed=True)
    tol = dict(rtol=5e-3, atol=5e-5) if key.startswith("issue114") else {}
    similar(got, G.expected(key, got), **tol)


def test_gpu_awhile_jacobi_100_iterations_in_one_program(gpu_ctx):
    # "iterated 100 times" as one program: the loop runs in the library, one scalar read-back per trip
    grid = np.random.default_rng(9).random(size=(256, 384), dtype=np.float32)
    t = A.awhile(lambda s: A.unit(A.the(s[1]) < 100),
                 lambda s: (A.stencil(C.jacobi, A.clamp, s[0]), A.unit(A.the(s[1]) + 1)),
                 (grid, A.unit(A.constant(np.int64(0)))))
    out, count = backend.run(list(t), gpu_ctx)
    assert int(count) == 100
    assert np.array_equal(out, C.jacobi_np(grid, 100))
    unrolled = A.use(grid)
    for _ in range(100):
        unrolled = A.stencil(C.jacobi, A.clamp, unrolled)
    assert np.array_equal(out, backend.run(unrolled, gpu_ctx))


def test_gpu_kernel_cache_hits_across_sizes(gpu_ctx):
    # shapes are kernel parameters: the same program on arrays of another size compiles nothing new
    # (Analysis/Hash.hs:67-99, hashing with perfect=False ignores what does not reach the kernel)
    f = backend.runN(lambda a: A.fold(lambda x, y: x + y, 0, A.map(lambda v: v * 3 + 1, a)), gpu_ctx)
    f(np.arange(100, dtype=np.int64))
    s0 = gpu_ctx.stats()
    for n in (7, 5000, 100000):
        x = np.arange(n, dtype=np.int64)
        assert int(f(x)) == int((x * 3 + 1).sum())
    s1 = gpu_ctx.stats()
    assert s1["compiled"] == s0["compiled"] and s1["disk_hits"] == s0["disk_hits"]
    assert s1["mem_hits"] > s0["mem_hits"]


def test_gpu_memory_table_uploads_a_host_array_once(gpu_ctx):
    # the reference's memory table (Array/Remote/Table.hs:89-100): arrays are keyed by their unique id, so
    # a host array that several runs use travels to the device once
    from accelerate_b200 import language as L
    x = np.arange(1 << 16, dtype=np.int32)
    L.reset_names()
    prog = A.build_program(A.map(lambda v: v + 1, L.param(1, "i32")))
    key = 0xABCDEF01
    s0 = gpu_ctx.stats()["h2d_bytes"]
    for _ in range(3):
        d = gpu_ctx.intern(key, x)
        out, = gpu_ctx.execute(prog.text, [d], 1)
        assert np.array_equal(out.download(), x + 1)
        d.free()                                     # the id goes, the table keeps the device copy
        out.free()
    assert gpu_ctx.stats()["h2d_bytes"] - s0 == x.nbytes
    with pytest.raises(backend.B200Error) as e:
        gpu_ctx.intern(key, x[:100])
    assert e.value.code == 7
    gpu_ctx.forget(key)
    d = gpu_ctx.intern(key, x)
    out, = gpu_ctx.execute(prog.text, [d], 1)
    assert np.array_equal(out.download(), x + 1)
    assert gpu_ctx.stats()["h2d_bytes"] - s0 == 2 * x.nbytes
    gpu_ctx.forget(key)


def test_gpu_freed_buffers_are_reused_by_size(gpu_ctx):
    # the reference's nursery (Array/Remote/Nursery.hs:55-108; Table.hs:176-205): a freed device buffer is kept
    # and handed to the next allocation of the same (chunk-rounded) size; `purge` gives everything back
    gpu_ctx.sync()
    gpu_ctx.purge()
    n = 300_001                                       # 1 200 004 bytes: not a multiple of the chunk
    a = gpu_ctx.from_host(np.arange(n, dtype=np.int32))
    p = a.devptr()
    m0 = gpu_ctx.memory_stats()
    assert m0["live_bytes"] >= 4 * n
    a.free()
    m1 = gpu_ctx.memory_stats()
    assert m1["nursery_blocks"] == m0["nursery_blocks"] + 1 and m1["nursery_bytes"] - m0["nursery_bytes"] >= 4 * n
    b = gpu_ctx.from_host(np.arange(n - 1, dtype=np.int32) * 3)        # rounds up to the same size
    assert b.devptr() == p
    m2 = gpu_ctx.memory_stats()
    assert m2["nursery_hits"] == m1["nursery_hits"] + 1 and m2["nursery_blocks"] == m0["nursery_blocks"]
    assert np.array_equal(b.download(), np.arange(n - 1, dtype=np.int32) * 3)
    c = gpu_ctx.from_host(np.zeros(17, dtype=np.int64))                # another size: no hit
    assert gpu_ctx.memory_stats()["nursery_hits"] == m2["nursery_hits"]
    b.free(); c.free()
    gpu_ctx.purge()
    m3 = gpu_ctx.memory_stats()
    assert m3["nursery_blocks"] == 0 and m3["nursery_bytes"] == 0
    # results of a program come out of the nursery too
    x = np.arange(1 << 12, dtype=np.float32)
    h0 = gpu_ctx.memory_stats()["nursery_hits"]
    for _ in range(3):
        out = backend.run(A.map(lambda v: v * 2, x), gpu_ctx)
        assert np.array_equal(out, x * 2)
    assert gpu_ctx.memory_stats()["nursery_hits"] > h0


def test_gpu_permute_updates_unshared_defaults_in_place(gpu_ctx):
    # Language.hs:764-765: defaults that are used only by the permutation are updated in place; defaults that
    # are an input, are used again, or are read by the permutation's own source are copied first
    add = lambda a, b: a + b  # noqa: E731
    k = (np.arange(5000, dtype=np.int64) * 7) % 64
    ones = np.ones(5000, dtype=np.int32)
    want = np.bincount(k, minlength=64).astype(np.int32)
    ix = lambda i: A.Just_(A.index(A.use(k)[i]))  # noqa: E731
    m0 = gpu_ctx.memory_stats()["inplace_permutes"]
    got = backend.run(A.permute(add, A.fill(64, A.constant(np.int32(0))), ix, ones), gpu_ctx)
    assert np.array_equal(got, want)
    assert gpu_ctx.memory_stats()["inplace_permutes"] == m0 + 1
    base = np.arange(64, dtype=np.int32)
    got = backend.run(A.permute(add, base, ix, ones), gpu_ctx)                 # an input: not touched
    assert np.array_equal(got, want + base) and np.array_equal(base, np.arange(64, dtype=np.int32))
    assert gpu_ctx.memory_stats()["inplace_permutes"] == m0 + 1
    d = A.scanl1(add, base)                                                     # a temporary used twice
    h = A.permute(add, d, ix, ones)
    got = backend.run(A.zipWith(add, h, d), gpu_ctx)
    assert np.array_equal(got, want + 2 * np.cumsum(base, dtype=np.int32))
    assert gpu_ctx.memory_stats()["inplace_permutes"] == m0 + 1
    d2 = A.scanl1(add, base)                                                    # a temporary that the permutation's index and source read
    got = backend.run(A.permute(add, d2, lambda i: A.Just_(A.index(A.from_integral(d2[i] % 64, "i64"))), A.map(lambda v: v * 3, d2)), gpu_ctx)
    c = np.cumsum(base, dtype=np.int32)
    w = c.copy()
    np.add.at(w, c % 64, 3 * c)
    assert np.array_equal(got, w)
    assert gpu_ctx.memory_stats()["inplace_permutes"] == m0 + 1


def test_gpu_atrace_and_aforeign(gpu_ctx, capfd):
    # the same lines on standard error as the oracle writes; the traced term's value is handed on
    x = np.arange(6, dtype=np.int32).reshape(2, 3)
    y = np.array([1.5, 2.25], dtype=np.float32)
    t = A.atrace("after map", [A.map(lambda v: v + 1, x), A.zip(y, y)], A.map(lambda v: v * 2, x))
    capfd.readouterr()
    got = backend.run(t, gpu_ctx)
    err = capfd.readouterr().err
    assert np.array_equal(got, x * 2)
    assert err == "after map: Matrix (Z :. 2 :. 3) [1,2,3,4,5,6], Vector (Z :. 2) [(1.5,1.5),(2.25,2.25)]\n"
    got = backend.run(A.map(lambda v: v + 1, A.atrace("no arrays", None, x)), gpu_ctx)
    assert np.array_equal(got, x + 1) and capfd.readouterr().err == "no arrays\n"
    t = A.aforeign("vendor.scale", lambda a: A.map(lambda v: v * 3.0, a), y)
    assert np.array_equal(backend.run(t, gpu_ctx), y * 3)


def test_gpu_stencil_row_windows_one_and_two_ranges(gpu_ctx):
    # b200_program_run_rows / _rows2: rows of a one-stencil program's result written into an existing array
    # (what the multi-GPU stencil uses for the rows that do and do not need fresh halo rows)
    from accelerate_b200 import language as L
    g = np.random.default_rng(3)
    m = g.uniform(0, 1, (70, 300)).astype(np.float32)
    jac = lambda s: 0.25 * (s[0][1] + s[2][1] + s[1][0] + s[1][2])  # noqa: E731
    L.reset_names()
    text = A.build_program(A.stencil(jac, A.clamp, L.param(2, "f32"))).text
    a = gpu_ctx.from_host(m)
    full, = gpu_ctx.execute(text, [a], 1)
    want = full.download()
    out = gpu_ctx.from_host(np.zeros_like(m))
    gpu_ctx.run_rows(text, [a], out, 10, 40)
    got = out.download()
    assert np.array_equal(got[10:40], want[10:40]) and not got[:10].any() and not got[40:].any()
    out2 = gpu_ctx.from_host(np.zeros_like(m))
    gpu_ctx.run_rows2(text, [a], out2, 0, 3, 37, 70)
    got = out2.download()
    assert np.array_equal(got[:3], want[:3]) and np.array_equal(got[37:], want[37:]) and not got[3:37].any()
    gpu_ctx.run_rows2(text, [a], out2, 3, 36, 36, 37)                  # the rest, in two ranges of very different size
    assert np.array_equal(out2.download(), want)
    with pytest.raises(backend.B200Error) as e:
        gpu_ctx.run_rows2(text, [a], out2, 10, 20, 15, 30)             # overlapping ranges
    assert e.value.code == 7
    with pytest.raises(backend.B200Error):
        gpu_ctx.run_rows2(text, [a], out2, 0, 3, 60, 71)               # outside the array
