"""Pins the CPU oracle to the reference: every known-answer vector the
reference's own tests and haddock examples hold for the hot path."""
import numpy as np
import pytest

from oracle import oracle
from tests import golden_cases as G
from tests.util import similar

CASES = G.cases()
EXTRA = G.extra_cases()


@pytest.mark.parametrize("key", sorted(CASES))
def test_oracle_matches_reference_vector(key):
    got = oracle.run(CASES[key])
    want = G.expected(key, got)
    tol = dict(rtol=5e-3, atol=5e-5) if key.startswith("issue114") else {}     # Test/Similar.hs:90-91
    similar(got, want, **tol)


@pytest.mark.parametrize("key", sorted(EXTRA))
def test_oracle_matches_reference_closed_form(key):
    term, want = EXTRA[key]
    got = oracle.run(term)
    tol = dict(rtol=5e-3, atol=5e-5) if key.startswith("issue114") else {}
    similar(got, want, **tol)


PRELUDE = G.prelude_cases()


@pytest.mark.parametrize("key", sorted(PRELUDE))
def test_oracle_matches_reference_prelude_example(key):
    got = oracle.run(PRELUDE[key])
    if isinstance(got, tuple):          # nested tuples (an index paired with a value) are their leaves in order
        got = tuple(got)
    similar(got, G.expected(key, got))


@pytest.mark.parametrize("key", ["replicate_two", "slice_sl1_cube", "indexed_mat", "all_even", "enumFromStepN_mat", "concatOn_2",
                                 "filter_odd_mat_0", "gatherIf", "transposeOn_box_13", "postscanl_vec", "primes_100"])
def test_prelude_examples_compile_for_the_gpu(key):
    # (these programs are run on the oracle only; their kernels are the skeletons the GPU suite exercises)
    import accelerate_b200 as A
    from accelerate_b200 import backend
    assert "ok" in backend.compile_check(A.build_program(PRELUDE[key]).text)


ISSUES = G.issue_cases()


@pytest.mark.parametrize("key", sorted(ISSUES))
def test_oracle_matches_reference_regression_test(key):
    term, want = ISSUES[key]
    tol = dict(rtol=5e-3, atol=5e-5) if key.startswith("issue409") else {}     # Test/Similar.hs:90-93
    similar(oracle.run(term), want, **tol)


@pytest.mark.parametrize("key", ["issue102", "issue119_2", "issue119_10_ps", "issue168_C", "issue184_B", "issue287_C", "issue436_B_0"])
def test_regression_tests_compile_for_the_gpu(key):
    import accelerate_b200 as A
    from accelerate_b200 import backend
    assert "ok" in backend.compile_check(A.build_program(ISSUES[key][0]).text)


def test_every_extracted_vector_is_used():
    assert set(G.VECTORS) == set(CASES) | set(PRELUDE) | {"issue102_ref1"}
