"""TEST INFRASTRUCTURE ONLY — Python handle on the CPU oracle (``interp.cpp``).

The oracle is a sequential restatement of the reference interpreter
(``src/Data/Array/Accelerate/Interpreter.hs``).  It may be used by the
test-suite, the smoke check and the benchmark's CPU-baseline leg, and by
nothing in the product path.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "interp.cpp")
_LIB = os.path.join(_HERE, "_build", "liboracle.so")
_NP = {"i8": np.int8, "i16": np.int16, "i32": np.int32, "i64": np.int64, "u8": np.uint8, "u16": np.uint16,
       "u32": np.uint32, "u64": np.uint64, "f32": np.float32, "f64": np.float64, "f16": np.float16}
_lib = None


def build(force=False):
    """Compile the oracle (g++, no fast-math, no FMA contraction)."""
    if not force and os.path.exists(_LIB) and os.path.getmtime(_LIB) >= os.path.getmtime(_SRC):
        return _LIB
    os.makedirs(os.path.dirname(_LIB), exist_ok=True)
    subprocess.check_call(["g++", "-O2", "-std=c++17", "-ffp-contract=off", "-fPIC", "-shared", _SRC, "-o", _LIB])
    return _LIB


def _load():
    global _lib
    if _lib is None:
        lib = ctypes.CDLL(build())
        lib.orc_parse.restype = ctypes.c_void_p
        lib.orc_parse.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_int]
        lib.orc_free.argtypes = [ctypes.c_void_p]
        lib.orc_set_input.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_int64),
                                      ctypes.c_int, ctypes.POINTER(ctypes.c_void_p)]
        lib.orc_run.argtypes = [ctypes.c_void_p]
        lib.orc_error.restype = ctypes.c_char_p
        lib.orc_error.argtypes = [ctypes.c_void_p]
        for n in ("orc_num_inputs", "orc_num_outputs"):
            getattr(lib, n).argtypes = [ctypes.c_void_p]
        for n in ("orc_out_rank", "orc_out_nleaves"):
            getattr(lib, n).argtypes = [ctypes.c_void_p, ctypes.c_int]
        lib.orc_out_shape.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(ctypes.c_int64)]
        lib.orc_out_leaf_type.restype = ctypes.c_char_p
        lib.orc_out_leaf_type.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int]
        lib.orc_out_leaf_copy.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
        _lib = lib
    return _lib


class OracleError(RuntimeError):
    """The oracle's counterpart of the reference's ``error`` calls (Error.hs)."""


def run_text(text, inputs):
    """Evaluate program ``text``.  ``inputs`` is a list of ``(shape, [leaves])``;
    returns a list of ``(shape, [leaf ndarrays])``."""
    lib = _load()
    err = ctypes.create_string_buffer(1024)
    h = lib.orc_parse(text.encode(), err, 1024)
    if not h:
        raise OracleError("parse: " + err.value.decode())
    try:
        keep = []
        for k, (shape, leaves) in enumerate(inputs):
            leaves = [np.ascontiguousarray(x) for x in leaves]
            keep.append(leaves)
            sh = (ctypes.c_int64 * max(1, len(shape)))(*shape)
            ptrs = (ctypes.c_void_p * len(leaves))(*[x.ctypes.data for x in leaves])
            if lib.orc_set_input(h, k, len(shape), sh, len(leaves), ptrs):
                raise OracleError(lib.orc_error(h).decode())
        if lib.orc_run(h):
            raise OracleError(lib.orc_error(h).decode())
        outs = []
        for k in range(lib.orc_num_outputs(h)):
            rank = lib.orc_out_rank(h, k)
            sh = (ctypes.c_int64 * max(1, rank))()
            lib.orc_out_shape(h, k, sh)
            shape = tuple(int(sh[i]) for i in range(rank))
            leaves = []
            for l in range(lib.orc_out_nleaves(h, k)):
                dt = _NP[lib.orc_out_leaf_type(h, k, l).decode()]
                a = np.empty(shape, dtype=dt)
                lib.orc_out_leaf_copy(h, k, l, a.ctypes.data)
                leaves.append(a)
            outs.append((shape, leaves))
        return outs
    finally:
        lib.orc_free(h)


def run(results):
    """Evaluate array term(s) built with ``accelerate_b200.language`` whose
    inputs were embedded with ``use``.  Returns ndarray (scalar elements) or a
    tuple of ndarrays (tuple elements) per result."""
    from accelerate_b200 import language as L
    single = not isinstance(results, (list, tuple))
    prog = L.build_program(results)
    text = prog.text
    if "(vec " in text:
        # Arrays of SIMD vectors cross a program's boundary as arrays of their components with one more
        # dimension; the library rewrites the text accordingly and the oracle evaluates what it wrote.
        from accelerate_b200 import backend
        text = backend.program_lowered(text)
    outs = run_text(text, [n.data for n in prog.inputs])
    res = [leaves[0] if L.is_scalar(elt) else tuple(leaves) for (_, leaves), (_, elt) in zip(outs, prog.outputs)]
    return res[0] if single else res
