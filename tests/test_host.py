"""Host-side checks that need no GPU: the C-ABI library loads and exports what
include/accelerate_b200.h declares, program text is parsed and type-checked with
the documented status codes, every skeleton compiles for sm_100a through NVRTC,
and nothing falls back to the CPU when no GPU is present."""
import ctypes
import os
import re

import numpy as np
import pytest

import accelerate_b200 as A
from accelerate_b200 import backend

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
add = lambda a, b: a + b  # noqa: E731


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "accelerate_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(lib_built):
    lib = ctypes.CDLL(lib_built)
    names = declared_symbols()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in the header but not exported"


def test_no_gpu_means_a_loud_error_not_a_fallback(lib_built):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(backend.B200Error) as e:
        backend.Context(0)
    assert e.value.code == 4 and "no CPU fallback" in str(e.value)
    with pytest.raises(backend.B200Error):
        backend.run(A.fold(add, 0, np.arange(4)))


def _check(text):
    return backend.compile_check(text)


def test_ring_scan_alignment_rule(lib_built):
    """The ring scan kernel copies whole tiles with cp.async.bulk (16-byte aligned sources): rows whose
    pitch in bytes is not a multiple of 16 must take the register kernel whenever the pitch enters a
    tile's address (several rows, or a right-to-left scan)."""
    lib = ctypes.CDLL(lib_built)
    f = lib.b200_scan_ring_aligned
    f.argtypes = [ctypes.c_int, ctypes.c_int64, ctypes.c_int64, ctypes.c_int]
    assert f(4, 1 << 20, 1, 0) == 1 and f(4, 1 << 20, 1, 1) == 1
    assert f(4, 8196, 300, 0) == 1            # 4-byte elements, n % 4 == 0: always aligned
    assert f(2, 8196, 1, 0) == 1              # one row, left to right: tiles start at multiples of the tile
    assert f(2, 8196, 1, 1) == 0              # right to left: tiles start at n - k*tile -> 8 mod 16
    assert f(2, 8196, 300, 0) == 0            # rows start at row * 16392 bytes
    assert f(2, 8200, 300, 1) == 1
    assert f(1, 8196, 2, 0) == 0 and f(1, 8208, 2, 1) == 1
    assert f(8, 4098, 2, 0) == 1 and f(8, 4097, 2, 0) == 0


def test_parse_and_type_errors_have_codes(lib_built):
    with pytest.raises(backend.B200Error) as e:
        _check("(program (in a (array 1 i32)) (out a")
    assert e.value.code == 1
    with pytest.raises(backend.B200Error) as e:
        _check("(program (in a (array 1 i32)) (let b (fold i32 (lam ((x i32) (y i32)) (prim add f32 (var x) (var y))) (manifest a))) (out b))")
    assert e.value.code == 2
    with pytest.raises(backend.B200Error) as e:
        _check("(program (in a (array 1 i32)) (let b (frobnicate a)) (out b))")
    assert e.value.code == 1
    with pytest.raises(backend.B200Error) as e:
        _check("(program (in a (array 1 i32)) (out nosuch))")
    assert e.value.code == 2


def test_skeletons_compile_for_sm100a(lib_built):
    xf, xi = np.zeros(8, np.float32), np.zeros(8, np.int32)
    m = np.zeros((4, 8), np.float32)
    k = A.use(xi)
    terms = [
        A.fold(add, 0.0, A.zipWith(lambda a, b: a * b, xf, xf)),
        A.fold1Seg(add, xi, np.array([3, 5], np.int32)),
        list(A.scanr_prime(add, 0, xi)),
        A.permute(add, A.fill(4, A.constant(np.int32(0))), lambda ix: A.Just_(A.index(A.from_integral(k[ix], "i64"))), xi),
        A.stencil(lambda s: s[0][1] + s[2][1] + s[1][0] + s[1][2], A.mirror, m),
    ]
    for t in terms:
        log = _check(A.build_program(t).text)
        assert "ok " in log


def test_generated_source_uses_the_vector_path_and_exact_semantics(lib_built):
    prog = A.build_program(A.fold(add, 0.0, A.zipWith(lambda a, b: a * b, np.zeros(8, np.float32), np.zeros(8, np.float32))))
    src = backend.kernel_source(prog.text, 0)
    assert "acc_ld4" in src and "acc_fold_all" in src and "D0_get4" in src
    assert "fmaf" not in src                      # no contraction in generated code
    prog = A.build_program(A.map(lambda v: (v // 3) + (v % 3) + (v << 40), np.zeros(8, np.int32)))
    src = backend.kernel_source(prog.text, 0)
    assert "acc_div<i32>" in src and "acc_mod<i32>" in src and "acc_shl<i32>" in src


def test_program_text_is_deterministic_and_ordered():
    def build():
        A.reset_names()
        x = A.param(1, "i32")
        s = A.scanl1(add, x)
        return A.build_program(A.fold(add, 0, A.zipWith(add, s, x))).text
    t1, t2 = build(), build()
    assert t1 == t2
    assert t1.index("scanl") < t1.index("(fold")


def test_oracle_raises_the_references_errors():
    from oracle import oracle
    with pytest.raises(oracle.OracleError, match="empty array"):
        oracle.run(A.fold1(add, np.zeros(0, np.int32)))                       # Interpreter.hs:386
    with pytest.raises(oracle.OracleError, match="empty segment"):
        oracle.run(A.fold1Seg(add, np.zeros(4, np.int32), np.array([2, 0, 2], np.int32)))   # Interpreter.hs:423
    with pytest.raises(oracle.OracleError, match="out of bounds"):
        oracle.run(A.backpermute(A.index(3), lambda ix: A.index(ix[0] + 5), np.zeros(4, np.int32)))


HASKELL_DIALECT = '''(program
  (in a0 (array 1 f32))
  (in a1 (array 1 f32))
  (let a2 (fold f32 (lam ((p0 f32) (p2 f32)) (let x0 (var p0) (let x1 (var p2) (prim add f32 (snoc (snoc (tup) (var x0)) (var x1)))))) (const f32 0x0p+0)
     (delayed (snoc (tup) (prim min i64 (snoc (snoc (tup) (last (shape a0))) (last (shape a1)))))
              (lam ((p0 (tup i64))) (let x0 (last (var p0)) (prim mul f32 (snoc (snoc (tup) (index a0 (snoc (tup) (var x0)))) (index a1 (snoc (tup) (var x0))))))))))
  (out a2))'''


def test_program_text_as_the_haskell_module_writes_it(lib_built):
    """haskell/src/Data/Array/Accelerate/B200.hs writes tuples as snoc lists ((tup), snoc, init,
    last) and passes binary primitives one pair: dotp in that dialect runs on the oracle,
    compiles, and still takes the vectorised path."""
    from oracle import oracle
    x = np.arange(8, dtype=np.float32)
    (_, (res,)), = oracle.run_text(HASKELL_DIALECT, [((8,), [x]), ((8,), [x])])
    assert float(res) == 140.0
    assert "ok fold" in backend.compile_check(HASKELL_DIALECT)
    assert "acc_ld4(p.a0_l0" in backend.kernel_source(HASKELL_DIALECT, 0)


HASKELL_DIALECT_SIMD = '''(program
  (in a0 (array 1 (vec 2 f16)))
  (let a1 (generate (vec 2 f16) (shape a0)
     (lam ((p0 (tup i64))) (let x0 (vecunpack 2 f16 (index a0 (var p0)))
        (vecpack 2 f16 (snoc (snoc (tup) (last (var x0))) (prim add f16 (snoc (snoc (tup) (last (init (var x0)))) (const f16 0x1p-1)))))))))
  (out a1))'''


def test_simd_and_half_as_the_haskell_module_writes_them(lib_built):
    """Vec n t as (vec n t) with VecPack/VecUnpack over snoc-list tuples, Half as f16 with hexadecimal
    literals: (x, y) -> (y, x + 0.5) over an array the caller hands over as its (n, 2) payload."""
    from oracle import oracle
    x = np.arange(10, dtype=np.float16).reshape(5, 2)
    (shape, (res,)), = oracle.run_text(backend.program_lowered(HASKELL_DIALECT_SIMD), [((5, 2), [x])])
    assert shape == (5, 2) and np.array_equal(res, np.stack([x[:, 1], x[:, 0] + np.float16(0.5)], axis=-1))
    assert "ok elementwise" in backend.compile_check(HASKELL_DIALECT_SIMD)


def test_sharded_program_cache_tells_builders_apart():
    """The executor of the sharded skeletons caches built programs.  Builders are closures: the same
    call site with another function, shape or constant must not get the first call's program."""
    from accelerate_b200 import language as L
    from accelerate_b200.sharded import ProgramCache

    class Arr:
        def __init__(self, elt, shape):
            self.elt, self.shape = elt, shape
    cache = ProgramCache()
    x = Arr("i32", (10,))

    def fold_all(f):
        return cache.get(("fold_all", "local"), lambda a: L.fold1(f, a), [x])[0].text
    t_add, t_max = fold_all(add), fold_all(L.max_)
    assert "add" in t_add and "max" in t_max and t_add != t_max
    assert fold_all(lambda a, b: a + b) == t_add                          # same code, same captures: one entry
    n_before = len(cache._progs)
    fold_all(add)
    assert len(cache._progs) == n_before

    def extend(rows):
        return cache.get("halo", lambda a: L.generate(L.index(rows + 2, 4), lambda ix: a[L.index(L.min_(ix[0], rows - 1), ix[1])], "i32"),
                         [Arr("i32", (rows, 4))])[0].text
    assert extend(6) != extend(8)                                          # the extent is baked into the program
    assert cache.get("k", lambda a: L.map_(lambda v: v + 1, a), [x])[0].text != cache.get("k", lambda a: L.map_(lambda v: v + 2, a), [x])[0].text


def test_kernel_cache_disk_hit_force_recompile_and_damaged_files(lib_built, tmp_path, monkeypatch):
    """The on-disk kernel cache: a second compilation of the same source is served from the cache,
    ACCELERATE_B200_FORCE_RECOMP bypasses it, and a cache file that is cut short or is not a cubin
    is recompiled and replaced instead of being loaded."""
    monkeypatch.setenv("ACCELERATE_B200_CACHE_DIR", str(tmp_path))
    text = A.build_program(A.map(lambda v: v * 7 + 3, np.zeros(8, np.int32))).text
    log = _check(text)
    assert log.count("compiled") == 1 and "disk cache" not in log
    files = sorted(tmp_path.glob("*.cubin"))
    assert len(files) == 1 and not list(tmp_path.glob("*.tmp*"))
    good = files[0].read_bytes()
    assert good[:4] == b"\x7fELF"
    assert "from the disk cache" in _check(text)
    monkeypatch.setenv("ACCELERATE_B200_FORCE_RECOMP", "1")
    assert "compiled" in _check(text)
    monkeypatch.delenv("ACCELERATE_B200_FORCE_RECOMP")
    for damaged in (good[:len(good) // 2], b"not a cubin at all " * 40, b""):
        files[0].write_bytes(damaged)
        assert "compiled" in _check(text)
        assert files[0].read_bytes()[:4] == b"\x7fELF" and len(files[0].read_bytes()) == len(good)
    # another scalar body is another kernel; another array SIZE is not (shapes are kernel parameters)
    assert "compiled" in _check(A.build_program(A.map(lambda v: v * 7 + 4, np.zeros(8, np.int32))).text)
    assert "from the disk cache" in _check(A.build_program(A.map(lambda v: v * 7 + 3, np.zeros(100000, np.int32))).text)


def test_bench_strong_scaling_parts_are_consistent():
    # bench.py splits the config size over the ranks for its strong-scaling figures: the first 1/N of every input,
    # and for fold1Seg whole segments whose lengths add up to the values that are kept
    import importlib.util
    spec = importlib.util.spec_from_file_location("bench_mod", os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    ws = {w.name: w for w in bench.suite(scale=14)}
    for world in (2, 3, 8):
        w = ws["fold1seg_add_i32"]
        vals, lens = [f() for f in w.inputs]
        v2, l2 = bench.strong_part(w, [vals, lens], world)
        assert int(l2.sum()) == v2.size and 0 < v2.size <= vals.size // world + 2048 and np.array_equal(v2, vals[:v2.size])
        w = ws["fold_max_rows_f32"]
        m, = [f() for f in w.inputs]
        p, = bench.strong_part(w, [m], world)
        assert p.shape == (max(1, m.shape[0] // world), m.shape[1])
