"""The allocation-free prefix sum, b200_scanl1_add_i32_noalloc.

Some users of the library must not allocate device memory and cannot let the
library do it either (a host runtime whose collector owns every device byte, a
caller on a path where cudaMalloc's device-wide synchronisation is ruled out).
For them the library offers one entry point whose scratch memory is a fixed
array inside the library image.  This test drives it through the C ABI on two
calls in a row — the second on a shorter, different input, so stale descriptors
left by the first call would be noticed — and requires bit-identical results to
the regular entry point (b200_program_run of `scanl1 (+)`), as for every integer
result in this suite.  It also checks that an over-long input is refused.

This file sorts last on purpose: a run that stops at the first failure has then
already executed every other test.
"""
import ctypes

import numpy as np
import pytest

import accelerate_b200 as A
from accelerate_b200 import backend

pytestmark = pytest.mark.gpu


def _noalloc_scan(ctx, host):
    lib = backend.lib()
    lib.b200_scanl1_add_i32_noalloc.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p]
    lib.b200_scanl1_add_i32_noalloc.restype = ctypes.c_int
    src = ctx.from_host(host)                       # input and output belong to the caller
    dst = ctx.array("i32", host.shape)
    rc = lib.b200_scanl1_add_i32_noalloc(src.devptr(0), dst.devptr(0), host.size, ctx.stream())
    assert rc == 0, backend.lib().b200_last_error().decode()
    return dst.download()


def _regular_scan(ctx, host):
    return backend.run(A.scanl1(lambda a, b: a + b, host), ctx)


def test_noalloc_scan_matches_regular_entry_point_twice(gpu_ctx):
    rng = np.random.default_rng(7)
    first = rng.integers(0, 100, size=3 * 4096 * 37 + 123).astype(np.int32)
    second = rng.integers(-2_000_000_000, 2_000_000_000, size=4096 * 5 + 1).astype(np.int32)   # wraps, shorter
    for host in (first, second):
        got = _noalloc_scan(gpu_ctx, host)
        want = _regular_scan(gpu_ctx, host)
        assert got.dtype == want.dtype and got.shape == want.shape
        assert np.array_equal(got, want)
        assert np.array_equal(got, np.cumsum(host, dtype=np.int32))


def test_noalloc_scan_rejects_oversize_and_accepts_empty(gpu_ctx):
    lib = backend.lib()
    lib.b200_scanl1_add_i32_noalloc.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p]
    lib.b200_scanl1_add_i32_noalloc.restype = ctypes.c_int
    buf = gpu_ctx.array("i32", (16,))
    too_many = (1 << 28) + 1
    rc = lib.b200_scanl1_add_i32_noalloc(buf.devptr(0), buf.devptr(0), too_many, gpu_ctx.stream())
    assert rc == 7                                                   # B200_ERR_ARG
    assert b"B200_NOALLOC_SCAN_MAX_ELEMS" in lib.b200_last_error()
    assert lib.b200_scanl1_add_i32_noalloc(None, None, 0, gpu_ctx.stream()) == 0


def test_noalloc_scan_at_the_size_limit_and_on_unaligned_pointers(gpu_ctx):
    """The largest input the fixed scratch array can describe (exactly B200_NOALLOC_SCAN_MAX_ELEMS), and
    an input/output pair that is only 4-byte aligned, which takes the scalar instead of the 128-bit path."""
    lib = backend.lib()
    lib.b200_scanl1_add_i32_noalloc.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p]
    lib.b200_scanl1_add_i32_noalloc.restype = ctypes.c_int
    n = 1 << 28
    block = np.random.default_rng(11).integers(0, 100, size=1 << 22).astype(np.int32)
    host = np.tile(block, n >> 22)
    got = _noalloc_scan(gpu_ctx, host)
    assert np.array_equal(got, np.cumsum(host, dtype=np.int32))
    del got, host
    # 4 bytes past a 16-byte boundary on both sides
    m = 3 * 4096 + 77
    host = np.random.default_rng(12).integers(-1000, 1000, size=m + 1).astype(np.int32)
    src = gpu_ctx.from_host(host)
    dst = gpu_ctx.array("i32", (m + 1,))
    rc = lib.b200_scanl1_add_i32_noalloc(src.devptr(0) + 4, dst.devptr(0) + 4, m, gpu_ctx.stream())
    assert rc == 0, lib.b200_last_error().decode()
    assert np.array_equal(dst.download()[1:], np.cumsum(host[1:], dtype=np.int32))
