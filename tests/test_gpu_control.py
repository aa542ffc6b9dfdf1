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
