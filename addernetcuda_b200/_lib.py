"""ctypes binding of libadder_b200.so (the C ABI declared in include/adder_b200.h).

There is no fallback: if the library is missing it is built with nvcc, and if that fails the
import raises.  Nothing here computes on the CPU.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_longlong, c_size_t, c_uint, c_ulonglong, c_void_p, POINTER
from pathlib import Path

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "libadder_b200.so"
TUNING_LIB_PATH = _PKG / "libadder_b200_tuning.so"

ADDER_OK = 0
FLAG_FAST_CLAMP = 1
FLAG_ACCUMULATE = 2
# status codes of include/adder_b200.h
(OK, ERR_NULL_POINTER, ERR_BAD_SHAPE, ERR_UNSUPPORTED, ERR_ALIGNMENT, ERR_WORKSPACE, ERR_CUDA, ERR_INTERNAL,
 ERR_TOO_LARGE, ERR_TIMEOUT) = range(10)

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
    "adder_b200_forward_stat_slices": (c_int, [*_GEOM]),
    "adder_b200_forward_with_stats": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, *_GEOM, c_void_p]),
    "adder_b200_batchnorm_forward_from_stats": (c_int, [c_void_p, c_void_p, c_int] + [c_void_p] * 9 +
                                                [c_float, c_float, c_int, c_int, c_int, c_int, c_void_p]),
    "adder_b200_batchnorm_backward": (c_int, [c_void_p] * 10 + [c_int, c_void_p, c_size_t, c_int, c_int, c_int,
                                              c_void_p]),
    "adder_b200_affine_forward": (c_int, [c_void_p] * 5 + [c_int, c_int, c_int, c_int, c_void_p]),
    "adder_b200_device_status": (c_int, [POINTER(c_int), c_int]),
    "adder_b200_peer_area_bytes": (c_size_t, [c_longlong, c_int]),
    "adder_b200_ipc_export": (c_int, [c_void_p, c_void_p, POINTER(c_ulonglong)]),
    "adder_b200_ipc_open": (c_int, [c_void_p, c_ulonglong, POINTER(c_void_p)]),
    "adder_b200_ipc_close": (c_int, [c_void_p, c_ulonglong]),
    "adder_b200_peer_comm_create": (c_int, [POINTER(c_void_p), c_int, c_int, c_int, c_void_p, c_void_p, c_longlong,
                                            c_int, c_int]),
    "adder_b200_peer_allreduce": (c_int, [c_void_p, c_void_p]),
    "adder_b200_peer_comm_status": (c_int, [c_void_p, POINTER(c_int), POINTER(c_uint), c_int]),
    "adder_b200_peer_comm_destroy": (c_int, [c_void_p]),
    "adder_b200_describe_plan": (c_int, [c_int, *_GEOM, c_int, c_char_p, c_size_t]),
}
# exported by libadder_b200_tuning.so only (the header's ADDER_B200_TUNING section)
TUNING_SIGNATURES = {
    "adder_b200_set_tile_hint": (c_int, [c_int] * 7),
    "adder_b200_set_micro_tile": (c_int, [c_int, c_int, c_int]),
    "adder_b200_set_variant": (c_int, [c_int, c_int]),
}

_product = None
_tuning = None
_active = None


def _open(path: Path, signatures) -> ctypes.CDLL:
    if not path.exists():
        from . import build as _build
        _build.build()
    lib = ctypes.CDLL(str(path))
    for name, (res, args) in signatures.items():
        fn = getattr(lib, name)   # AttributeError here means header and library disagree
        fn.restype = res
        fn.argtypes = args
    return lib


def load() -> ctypes.CDLL:
    """The library every op of this package calls: the product library, unless a `tuning()` block is
    active.  Loaded (and built first if necessary) on first use."""
    global _product, _active
    if _active is not None:
        return _active
    if _product is None:
        _product = _open(LIB_PATH, SIGNATURES)
    _active = _product
    return _active


class tuning:
    """`with tuning() as lib:` routes every op of this package through libadder_b200_tuning.so, whose
    extra entry points (`lib.adder_b200_set_tile_hint`, `_set_micro_tile`, `_set_variant`) override the
    tile planners.  On exit all overrides are cleared and the product library is active again."""

    def __enter__(self) -> ctypes.CDLL:
        global _tuning, _active
        if _tuning is None:
            _tuning = _open(TUNING_LIB_PATH, {**SIGNATURES, **TUNING_SIGNATURES})
        self._previous = _active
        _active = _tuning
        return _tuning

    def __exit__(self, *exc) -> None:
        global _active
        for op in range(3):
            _tuning.adder_b200_set_tile_hint(op, 0, 0, 0, 0, 0, 0)
            _tuning.adder_b200_set_micro_tile(op, 0, 0)
            _tuning.adder_b200_set_variant(op, 0)
        _active = self._previous


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


def device_status(reset: bool = True) -> int:
    """0 unless a kernel's bounded wait for the copy engine ran out on the current device."""
    v = c_int(0)
    check(load().adder_b200_device_status(ctypes.byref(v), int(reset)), "adder_b200_device_status")
    return v.value
