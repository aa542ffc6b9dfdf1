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
