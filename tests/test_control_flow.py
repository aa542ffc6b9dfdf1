"""Array-level control flow and embedded arrays (Acond, Awhile, Apply, Use: the nodes the reference
evaluates on the host, Interpreter.hs:215-231) on the CPU oracle, against NumPy; and the
program-text checks of the C-ABI library for the same forms (no GPU needed)."""
import numpy as np
import pytest

import accelerate_b200 as A
from accelerate_b200 import backend
from oracle import oracle
from tests import control_cases as C
from tests import golden_cases as G
from tests.util import similar

CASES = C.cases()


@pytest.mark.parametrize("key", sorted(CASES))
def test_oracle_control_flow(key):
    term, want = CASES[key]
    got = oracle.run(term)
    if isinstance(term, list):
        for g, w in zip(got, want):
            similar(g, w)
    else:
        similar(got, want)


@pytest.mark.parametrize("key", sorted(CASES))
def test_control_flow_programs_type_check_and_compile(key, lib_built):
    term, _ = CASES[key]
    for embed in (False, True):
        assert "ok " in backend.compile_check(A.build_program(term, embed=embed).text) or key == "apply_radixsort_empty"


def test_embedded_use_gives_the_same_results_as_inputs():
    # the haddock examples in their original `run (... (use xs))` form: arrays inside the program text
    from accelerate_b200 import language as L
    for key, term in sorted(G.cases().items()):
        prog = L.build_program(term, embed=True)
        assert not prog.inputs and "(in " not in prog.text
        outs = oracle.run_text(prog.text, [])
        got = [leaves[0] if L.is_scalar(elt) else tuple(leaves) for (_, leaves), (_, elt) in zip(outs, prog.outputs)]
        got = got if isinstance(term, (list, tuple)) else got[0]
        tol = dict(rtol=5e-3, atol=5e-5) if key.startswith("issue114") else {}
        similar(got, G.expected(key, got), **tol)


def test_control_flow_type_errors(lib_built):
    bad_branches = """(program (in a0 (array 1 i32))
      (let a1 (acond (const u8 1) (branch (out a0))
                                  (branch (let a2 (fold i32 (lam ((v0 i32) (v1 i32)) (prim add i32 (var v0) (var v1))) (manifest a0))) (out a2))))
      (out a1))"""
    with pytest.raises(backend.B200Error) as e:
        backend.compile_check(bad_branches)
    assert e.value.code == 2 and "branches" in str(e.value)
    bad_cond = """(program (in a0 (array 1 i32))
      (let a1 (awhile (afun ((a2 (array 1 i32))) (out a2)) (afun ((a3 (array 1 i32))) (out a3)) (args a0)))
      (out a1))"""
    with pytest.raises(backend.B200Error) as e:
        backend.compile_check(bad_cond)
    assert e.value.code == 2 and "Scalar Bool" in str(e.value)
    short_payload = "(program (let a0 (use (array 1 i32) (shape 3) (hex 0100000002000000))) (out a0))"
    with pytest.raises(backend.B200Error) as e:
        backend.compile_check(short_payload)
    assert e.value.code == 2 and "payload" in str(e.value)
    twice = "(program (in a0 (array 1 i32)) (let a0 (reshape (shape a0) a0)) (out a0))"
    with pytest.raises(backend.B200Error) as e:
        backend.compile_check(twice)
    assert e.value.code == 1


def test_atrace_prints_message_and_arrays_and_hands_the_result_on(capfd):
    # Atrace (Interpreter.hs:215, atraceOp :873-880): message, ": " and the arrays when there are any, on stderr
    x = np.arange(6, dtype=np.int32).reshape(2, 3)
    y = np.array([1.5, 2.25], dtype=np.float32)
    t = A.atrace("after map", [A.map(lambda v: v + 1, x), A.zip(y, y)], A.map(lambda v: v * 2, x))
    capfd.readouterr()
    got = oracle.run(t)
    err = capfd.readouterr().err
    assert np.array_equal(got, x * 2)
    assert err == "after map: Matrix (Z :. 2 :. 3) [1,2,3,4,5,6], Vector (Z :. 2) [(1.5,1.5),(2.25,2.25)]\n"
    got = oracle.run(A.map(lambda v: v + 1, A.atrace("no arrays", None, x)))
    assert np.array_equal(got, x + 1) and capfd.readouterr().err == "no arrays\n"
    s = A.atrace("scalar", A.fold(lambda a, b: a + b, 0, A.use(np.arange(5, dtype=np.int64))), (x, y))
    a, b = oracle.run(list(s))
    assert np.array_equal(a, x) and np.array_equal(b, y) and capfd.readouterr().err == "scalar: Scalar Z [10]\n"


def test_aforeign_runs_the_pure_fallback():
    # Aforeign (Interpreter.hs:217): without a foreign implementation the fallback function is applied
    x = np.arange(7, dtype=np.float32)
    t = A.aforeign("vendor.scale", lambda a: A.map(lambda v: v * 3.0, a), x)
    assert np.array_equal(oracle.run(t), x * 3)


def test_atrace_and_aforeign_programs_compile(lib_built):
    from accelerate_b200 import backend
    x = np.arange(6, dtype=np.int32).reshape(2, 3)
    for t in (A.atrace("m", [A.map(lambda v: v + 1, x)], A.map(lambda v: v * 2, x)), A.aforeign("f", lambda a: A.map(lambda v: v * 3, a), x)):
        assert "ok" in backend.compile_check(A.build_program(t).text)
    with pytest.raises(backend.B200Error):
        backend.compile_check("(program (in a0 (array 1 i32)) (let a1 (atrace (hex 6d) (show a9) (args a0))) (out a1))")
