"""ctypes binding of libadder_b200.so (the C ABI declared in include/adder_b200.h).

There is no fallback: if the library is missing it is built with nvcc, and if that fails the
import raises.  Nothing here computes on the CPU.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_size_t, c_void_p, POINTER
from pathlib import Path

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "libadder_b200.so"

ADDER_OK = 0
FLAG_FAST_CLAMP = 1
FLAG_ACCUMULATE = 2

_GEOM = [c_int] * 8  # n, ci, h, w, co, k, stride, pad

# name -> (restype, argtypes); must list every symbol of include/adder_b200.h
SIGNATURES = {
    "adder_b200_status_string": (c_char_p, [c_int]),
    "adder_b200_version": (c_int, []),
    "adder_b200_launch_count": (ctypes.c_ulonglong, []),
    "adder_b200_output_size": (c_int, [c_int, c_int, c_int, c_int, c_int, POINTER(c_int), POINTER(c_int)]),
    "adder_b200_forward": (c_int, [c_void_p, c_void_p, c_void_p, *_GEOM, c_void_p]),
    "adder_b200_backward_input": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, *_GEOM, c_int, c_void_p]),
    "adder_b200_backward_weight_workspace_bytes": (c_size_t, [*_GEOM]),
    "adder_b200_backward_weight": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p,
                                           c_size_t, *_GEOM, c_int, c_void_p]),
    "adder_b200_static_scratch_bytes": (c_size_t, []),
    "adder_b200_backward_weight_static": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, *_GEOM,
                                                  c_void_p]),
    "adder_b200_backward": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_size_t,
                                    *_GEOM, c_int, c_void_p]),
    "adder_b200_conv_col": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "adder_b200_col_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "adder_b200_conv_weight_col": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p,
                                           c_size_t, c_void_p]),
    "adder_b200_conv_input_col": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "adder_b200_backward_col": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                        c_void_p, c_size_t, c_void_p]),
    "adder_b200_batchnorm_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "adder_b200_batchnorm_forward": (c_int, [c_void_p] * 10 + [c_float, c_float, c_int, c_void_p, c_size_t,
                                             c_int, c_int, c_int, c_void_p]),
    "adder_b200_batchnorm_backward": (c_int, [c_void_p] * 10 + [c_int, c_void_p, c_size_t, c_int, c_int, c_int,
                                              c_void_p]),
    "adder_b200_set_tile_hint": (c_int, [c_int] * 7),
    "adder_b200_set_micro_tile": (c_int, [c_int, c_int, c_int]),
    "adder_b200_describe_plan": (c_int, [c_int, *_GEOM, c_int, c_char_p, c_size_t]),
}

_lib = None


def load() -> ctypes.CDLL:
    """Load (building first if necessary) the shared library and attach the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        from . import build as _build
        _build.build()
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)   # AttributeError here means header and library disagree
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(status: int, what: str) -> None:
    """Raise for a non-zero status: ValueError for caller mistakes, RuntimeError otherwise."""
    if status == ADDER_OK:
        return
    msg = load().adder_b200_status_string(status).decode()
    exc = ValueError if status in (1, 2, 3, 4, 5, 8) else RuntimeError
    raise exc(f"{what}: {msg} (status {status})")


def describe_plan(op: int, n, ci, h, w, co, k, stride, pad, flags: int = 0) -> str:
    """Tile plan of one kernel family for a layer, as text (launches nothing)."""
    buf = ctypes.create_string_buffer(512)
    check(load().adder_b200_describe_plan(op, n, ci, h, w, co, k, stride, pad, flags, buf, 512), "describe_plan")
    return buf.value.decode()
