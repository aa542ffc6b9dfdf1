"""GPU parity for SIMD vector element types (Test/NoFib/Prelude/SIMD.hs): the same programs as
tests/test_simd.py through the C ABI, with the arrays as inputs and embedded as `Use` nodes; expected
values from NumPy and the oracle."""
import numpy as np
import pytest

from accelerate_b200 import backend
from oracle import oracle
from tests import simd_cases

pytestmark = pytest.mark.gpu
CASES = simd_cases.cases()


@pytest.mark.parametrize("key", sorted(CASES))
def test_gpu_simd(key, gpu_ctx):
    term, want = CASES[key]
    got = backend.run(term, gpu_ctx, embed=key.startswith("inject"))
    assert got.dtype == want.dtype and got.shape == want.shape
    assert np.array_equal(got, want, equal_nan=got.dtype.kind == "f")
    assert np.array_equal(got, oracle.run(term), equal_nan=got.dtype.kind == "f")
