"""SIMD vector element types on the oracle (through the program text the library rewrites), against
NumPy; the kernels of the same programs are compiled here and run in tests/test_gpu_simd.py."""
import numpy as np
import pytest

import accelerate_b200 as A
from accelerate_b200 import backend
from oracle import oracle
from tests import simd_cases

CASES = simd_cases.cases()


@pytest.mark.parametrize("key", sorted(CASES))
def test_simd_on_the_oracle(key):
    term, want = CASES[key]
    got = oracle.run(term)
    assert got.dtype == want.dtype and got.shape == want.shape
    assert np.array_equal(got, want, equal_nan=got.dtype.kind == "f")


def test_vectors_cross_the_boundary_as_one_more_dimension():
    x = simd_cases.data("f32", (5, 3), 1)
    xs = A.use(x, elt=A.vec(3, "f32"))
    assert (xs.rank, xs.elt) == (1, "(vec 3 f32)")
    prog = A.build_program(A.map(lambda v: A.vec_pack(*A.vec_unpack(v)), xs))
    assert "(in a0 (array 1 (vec 3 f32)))" in prog.text
    low = backend.program_lowered(prog.text)
    assert "(in a0_aos (array 2 f32))" in low and "(out a1_aos)" in low and "(vec 3 f32)" in low
    # a program without vectors gains nothing
    plain = A.build_program(A.map(lambda v: v + 1, np.arange(4, dtype=np.int32))).text
    assert backend.program_lowered(plain).split() == plain.split()
    # embedded arrays are regrouped the same way
    emb = A.build_program(A.map(lambda v: A.vec_unpack(v)[0], xs), embed=True).text
    assert "(use (array 1 (vec 3 f32)) (shape 5)" in emb
    assert "(use (array 2 f32) (shape 5 3)" in backend.program_lowered(emb)


def test_simd_type_errors():
    x = simd_cases.data("f32", (5, 3), 1)
    with pytest.raises(TypeError):
        A.use(x, elt=A.vec(4, "f32"))                         # the last axis is not 4 long
    with pytest.raises(TypeError):
        A.vec(5, "f32")
    xs = A.use(x, elt=A.vec(3, "f32"))
    with pytest.raises(backend.B200Error):                    # arithmetic is not defined on vectors (AST.hs: PrimFun takes single types)
        backend.compile_check(A.build_program(A.map(lambda v: v + v, xs)).text)
    with pytest.raises(backend.B200Error):                    # a vector inside a tuple cannot leave the program
        backend.compile_check(A.build_program(A.map(lambda v: A.tup(v, A.constant(1)), xs)).text)
    with pytest.raises(backend.B200Error):
        backend.compile_check("(program (in a0 (array 1 f32)) (let a1 (generate (vec 2 f32) (shape a0) (lam ((v0 (tup i64))) "
                              "(vecpack 2 f32 (tup (index a0 (var v0)) (const i32 1)))))) (out a1))")


@pytest.mark.parametrize("key", ["extract_v3_f16_2", "inject_v4_u8", "fold_sum_v3_i32", "scanl1_sum_v3_i32", "complex_square_v2_f64"])
def test_simd_programs_compile(key):
    assert "ok" in backend.compile_check(A.build_program(CASES[key][0]).text)


def test_vectors_through_control_nodes_and_as_scalars():
    x = simd_cases.data("f32", (4, 3), 2)
    xs = A.use(x, elt=A.vec(3, "f32"))
    rot = lambda v: A.vec_pack(*[A.vec_unpack(v)[(k + 1) % 3] for k in range(3)])  # noqa: E731
    assert np.array_equal(oracle.run(A.compute(xs)), x)                              # in and straight out again
    st = A.awhile(lambda s: A.map(lambda c: c < 2, s[1]), lambda s: (A.map(rot, s[0]), A.map(lambda c: c + 1, s[1])),
                  (xs, A.unit(A.constant(0))))
    assert np.array_equal(oracle.run(st[0]), np.roll(x, -2, axis=1))
    assert "ok" in backend.compile_check(A.build_program(st[0]).text)
    pick = A.acond(A.the(A.unit(A.constant(1))).eq(1), A.map(rot, xs), xs)
    assert np.array_equal(oracle.run(pick), np.roll(x, -1, axis=1))
    one = A.use(np.array([1, 2], np.int32), elt=A.vec(2, "i32"))                     # a Scalar of a vector
    assert one.rank == 0 and int(oracle.run(A.map(lambda v: A.vec_unpack(v)[0] + A.vec_unpack(v)[1], one))) == 3
