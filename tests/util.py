"""Helpers shared by the parity tests: run a term on the GPU backend and on the
CPU oracle, and compare with the reference suite's notion of similarity
(Test/Similar.hs:35-37, 89-93, 181-190: exact for integers, absolute/relative
tolerance for floating point)."""
import numpy as np

import accelerate_b200 as A
from accelerate_b200 import backend
from oracle import oracle


def leaves(x):
    return list(x) if isinstance(x, tuple) else [x]


def similar(got, want, rtol=0.0, atol=0.0):
    """Bit-exact for integers; |a-b| <= atol or relative <= rtol for floats."""
    for g, w in zip(leaves(got), leaves(want)):
        assert g.shape == w.shape, (g.shape, w.shape)
        assert g.dtype == w.dtype, (g.dtype, w.dtype)
        if np.issubdtype(g.dtype, np.floating):
            if rtol == 0.0 and atol == 0.0:
                ok = (g == w) | (np.isnan(g) & np.isnan(w))
            else:
                d = np.abs(g.astype(np.float64) - w.astype(np.float64))
                denom = np.maximum(np.abs(g.astype(np.float64)), np.abs(w.astype(np.float64)))
                ok = (d <= atol) | (d <= rtol * denom) | (np.isnan(g) & np.isnan(w))
            if not np.all(ok):
                bad = np.argwhere(~ok)[:5]
                raise AssertionError(f"float mismatch at {bad.tolist()}: got {g[~ok][:5]}, want {w[~ok][:5]}")
        else:
            if not np.array_equal(g, w):
                bad = np.argwhere(g != w)[:5]
                raise AssertionError(f"integer mismatch at {bad.tolist()}: got {g[g != w][:5]}, want {w[g != w][:5]}")


def check(acc, rtol=0.0, atol=0.0, embed=False):
    """Evaluate on GPU and oracle; compare; return the GPU result."""
    multi = isinstance(acc, (list, tuple))
    got = backend.run(list(acc) if multi else acc, embed=embed)
    want = oracle.run(list(acc) if multi else acc)
    if multi:
        for g, w in zip(got, want):
            similar(g, w, rtol, atol)
    else:
        similar(got, want, rtol, atol)
    return got
