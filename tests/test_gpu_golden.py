"""The reference's known-answer vectors through the GPU backend (C ABI)."""
import pytest

from accelerate_b200 import backend
from tests import golden_cases as G
from tests.util import similar

pytestmark = pytest.mark.gpu
CASES = G.cases()
EXTRA = G.extra_cases()


@pytest.mark.parametrize("key", sorted(CASES))
def test_gpu_matches_reference_vector(key, gpu_ctx):
    got = backend.run(CASES[key], gpu_ctx)
    tol = dict(rtol=5e-3, atol=5e-5) if key.startswith("issue114") else {}
    similar(got, G.expected(key, got), **tol)


@pytest.mark.parametrize("key", sorted(EXTRA))
def test_gpu_matches_reference_closed_form(key, gpu_ctx):
    term, want = EXTRA[key]
    tol = dict(rtol=5e-3, atol=5e-5) if key.startswith("issue114") else {}
    similar(backend.run(term, gpu_ctx), want, **tol)
