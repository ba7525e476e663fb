"""ctypes binding of the C ABI declared in include/deepshift_b200.h.

There is no CPU fallback: if the CUDA library cannot be found or built, importing the
symbols raises, and every wrapper raises ``RuntimeError`` on a non-zero status.
"""
import ctypes
import os

from . import _build

_lib = None

c_i32p = ctypes.POINTER(ctypes.c_int32)


class Fuse(ctypes.Structure):
    """Mirror of ``ds_fuse_t``."""
    _fields_ = [
        ("in_kind", ctypes.c_int), ("out_kind", ctypes.c_int),
        ("act_integer_bits", ctypes.c_int), ("act_fraction_bits", ctypes.c_int),
        ("relu", ctypes.c_int), ("requant", ctypes.c_int),
        ("residual", ctypes.c_void_p), ("act_bits", ctypes.c_int),
        ("round_f32", ctypes.c_int), ("reserved", ctypes.c_int * 3),
        ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_longlong),
        ("prepared", ctypes.c_void_p), ("prepared_bytes", ctypes.c_longlong),
    ]


class Staged(ctypes.Structure):
    """Mirror of ``ds_staged_t``."""
    _fields_ = [("data", ctypes.c_void_p), ("B", ctypes.c_int), ("H", ctypes.c_int), ("W", ctypes.c_int),
                ("C", ctypes.c_int), ("halo", ctypes.c_int)]


class StagedOut(ctypes.Structure):
    """Mirror of ``ds_staged_out_t``."""
    _fields_ = [
        ("codes", ctypes.c_void_p), ("f32", ctypes.c_void_p), ("nchw", ctypes.c_void_p),
        ("nchw_is_f32", ctypes.c_int), ("staged", ctypes.POINTER(Staged)), ("residual", ctypes.c_void_p),
        ("relu", ctypes.c_int), ("round_f32", ctypes.c_int), ("act_integer_bits", ctypes.c_int),
        ("act_fraction_bits", ctypes.c_int), ("in_act_bits", ctypes.c_int), ("reserved", ctypes.c_int * 3),
    ]


IN_I32, IN_F32_CONV, IN_F32_LINEAR, IN_I32_CLAMP = 0, 1, 2, 3
OUT_I32, OUT_F32 = 0, 1

_VP, _I, _LL = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
_SIGNATURES = {
    "ds_linear_i32": [_VP, _VP, _VP, _VP, _I, _I, _I, _I, _I, _I, _VP],
    "ds_conv2d_i32": [_VP, _VP, _VP, _VP] + [_I] * 14 + [_VP],
    "ds_linear_ex": [_VP, _VP, _VP, _VP, _I, _I, _I, _I, _I, ctypes.POINTER(Fuse), _VP],
    "ds_conv2d_ex": [_VP, _VP, _VP, _VP] + [_I] * 13 + [ctypes.POINTER(Fuse), _VP],
    "ds_conv2d_noalloc": [_VP, _VP, _VP, _VP] + [_I] * 13 + [ctypes.POINTER(Fuse), _VP],
    "ds_conv2d_prepare": [_VP] + [_I] * 13 + [ctypes.POINTER(Fuse), ctypes.POINTER(ctypes.c_longlong), _VP],
    "ds_compress": [_VP, _VP, _VP, _I, _I, _I, _I, _VP],
    "ds_quantize_f32": [_VP, _VP, _LL, _I, _I, _I, _VP],
    "ds_maxpool2d_i32": [_VP, _VP, _I, _I, _I, _I, _I, _I, _I, _VP],
    "ds_add_relu_f32": [_VP, _VP, _LL, _I, _VP],
    "ds_maxpool2d_f32": [_VP, _VP, _I, _I, _I, _I, _I, _I, _I, _VP],
    "ds_avgpool_fix_i32": [_VP, _VP, _I, _I, _I, _I, _I, _VP],
    "ds_pipe_peak": [_I, _I, ctypes.POINTER(ctypes.c_double), _VP],
    "ds_last_kernel_error": [ctypes.POINTER(ctypes.c_int)],
    "ds_bounds_status": [ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)],
    "ds_bounds_debug_shrink_x": [_LL],
    "ds_unopt_linear_f32": [_VP, _VP, _VP, _VP, _I, _I, _I, _VP],
    "ds_unopt_conv2d_f32": [_VP, _VP, _VP, _VP] + [_I] * 11 + [_VP],
    "ds_staged_fill": [ctypes.POINTER(Staged), _VP],
    "ds_stage_nchw": [_VP, _I, _I, _I, ctypes.POINTER(Staged), _VP],
    "ds_staged_prepare": [_VP, _I, _I, _I, _I, _I, _I, _VP, _LL, ctypes.POINTER(ctypes.c_longlong), _VP],
    "ds_staged_conv2d": [ctypes.POINTER(Staged), _VP, _LL, _VP] + [_I] * 7 + [ctypes.POINTER(StagedOut), _VP, _LL, _VP],
    "ds_maxpool_nhwc": [_VP] + [_I] * 7 + [_VP, ctypes.POINTER(Staged), _I, _I, _VP],
    "ds_avgpool_fix_nhwc": [_VP, _VP, _I, _I, _I, _I, _I, _VP],
}


def lib():
    """Loads (building first if the sources changed and nvcc is present) the CUDA library."""
    global _lib
    if _lib is None:
        # DEEPSHIFT_B200_CHECKED=1 selects the bounds-checking flavour of the library
        # (DEEPSHIFT_B200_TIMING=1 the cycle-counting one, a diagnostic)
        checked = os.environ.get("DEEPSHIFT_B200_CHECKED", "") not in ("", "0")
        timing = not checked and os.environ.get("DEEPSHIFT_B200_TIMING", "") not in ("", "0")
        path = _build.CHECKED_LIB_PATH if checked else (_build.TIMING_LIB_PATH if timing else _build.LIB_PATH)
        if not _build.is_current(checked, timing) and _build.nvcc_path() is not None:
            _build.build(checked=checked, timing=timing)
        if not os.path.exists(path):
            raise RuntimeError(
                "deepshift_b200: CUDA library %s is missing and cannot be built (no nvcc); "
                "there is no CPU fallback" % path)
        l = ctypes.CDLL(path)
        for name, args in _SIGNATURES.items():
            fn = getattr(l, name)
            fn.argtypes = args
            fn.restype = ctypes.c_int
        l.ds_strerror.argtypes = [ctypes.c_int]
        l.ds_strerror.restype = ctypes.c_char_p
        l.ds_version.restype = ctypes.c_int
        l.ds_launch_count.argtypes = []
        l.ds_launch_count.restype = ctypes.c_longlong
        l.ds_staged_bytes.argtypes = [_I] * 5
        l.ds_staged_bytes.restype = ctypes.c_longlong
        _lib = l
    return _lib


def check(status, what):
    if status != 0:
        raise RuntimeError("deepshift_b200.%s failed: %s (status %d)"
                           % (what, lib().ds_strerror(status).decode(), status))
