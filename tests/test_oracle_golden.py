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


def test_every_extracted_vector_is_used():
    assert set(G.VECTORS) == set(CASES)
