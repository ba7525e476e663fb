"""Drop-in for the reference's pybind extension ``deepshift_cuda`` (pytorch/deepshift/kernels/cuda/
shift_cuda.cpp:64-68), backed by libdeepshift_b200.so through ctypes.

Put this directory on ``sys.path`` ahead of anything else that provides ``deepshift_cuda`` and the
reference's own Python package keeps working unchanged: ``deepshift/kernels/kernels.py:4-8`` imports
this module, and its ``linear`` / ``conv2d`` / ``compress_sign_and_shift`` (kernels.py:10-74) call
the three functions below with torch CUDA tensors exactly as they call the pybind ones.

``act_bits`` is passed as 0 (no promise about the activations' range), which selects the exact
integer path for any int32 input; the fused entry points (``ds_conv2d_ex`` with a workspace and
``DS_ACT_BITS_AUTO``) can pick the faster FP32-pipe path by looking at the data.
``kernels.py:32-36`` hands over an already padded tensor, so the convolution is asked for no
padding of its own.
"""
import ctypes
import os

import torch

_P, _I = ctypes.c_void_p, ctypes.c_int
_lib = None


def _library():
    global _lib
    if _lib is None:
        here = os.path.dirname(os.path.abspath(__file__))
        path = os.environ.get("DEEPSHIFT_B200_LIB") or os.path.join(os.path.dirname(here), "_lib", "libdeepshift_b200.so")
        lib = ctypes.CDLL(path)
        lib.ds_linear_i32.argtypes = [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P]
        lib.ds_conv2d_i32.argtypes = [_P, _P, _P, _P] + [_I] * 14 + [_P]
        lib.ds_compress.argtypes = [_P, _P, _P, _I, _I, _I, _I, _P]
        lib.ds_strerror.argtypes = [_I]
        lib.ds_strerror.restype = ctypes.c_char_p
        _lib = lib
    return _lib


def _stream(t):
    return torch.cuda.current_stream(t.device).cuda_stream if t.is_cuda else None


def _check(rc, what):
    if rc:
        raise RuntimeError("%s: %s" % (what, _library().ds_strerror(rc).decode()))


def _input(*tensors):
    # CHECK_INPUT of shift_cuda.cpp:22-24
    for t in tensors:
        if not t.is_contiguous():
            raise RuntimeError("tensor must be contiguous")


def DEEP_SHIFT_LINEAR(input, shift, bias, output, base, bits, out_features):
    """shift_cuda.cpp:26-39.  ``shift`` is the packed weight tensor (ConcWeight.data)."""
    _input(input, shift, bias, output)
    with torch.cuda.device(input.device) if input.is_cuda else _Null():
        _check(_library().ds_linear_i32(input.data_ptr(), shift.data_ptr(), bias.data_ptr(), output.data_ptr(),
                                        input.size(0), input.size(1), out_features, bits, base, 0, _stream(input)),
               "DEEP_SHIFT_LINEAR")


def DEEP_SHIFT_CONV(data_im, shift, bias, output, strides, padding, filter_height, filter_width, base, bits):
    """shift_cuda.cpp:41-53.  ``data_im`` is already padded (kernels.py:32-36); ``padding`` is ignored,
    as the reference's CUDA code ignores it (shift.cu:399-669 derives the output size from the padded tensor)."""
    _input(data_im, shift, bias, output)
    strides = list(strides)
    sh, sw = (strides[0], strides[0]) if len(strides) == 1 else (strides[0], strides[1])
    B, C, H, W = data_im.shape
    with torch.cuda.device(data_im.device) if data_im.is_cuda else _Null():
        _check(_library().ds_conv2d_i32(data_im.data_ptr(), shift.data_ptr(), bias.data_ptr(), output.data_ptr(),
                                        B, C, H, W, output.size(1), filter_height, filter_width, sh, sw, 0, 0,
                                        bits, base, 0, _stream(data_im)), "DEEP_SHIFT_CONV")


def COMPRESS_SIGN_SHIFT(shift, sign, weight, base, bits, out_c, in_c, height, width, row_length, num):
    """shift_cuda.cpp:55-61: packs (shift', sign) int32 [out_c, in_c, height, width] into ``weight``."""
    _input(shift, sign, weight)
    with torch.cuda.device(shift.device) if shift.is_cuda else _Null():
        _check(_library().ds_compress(shift.data_ptr(), sign.data_ptr(), weight.data_ptr(), out_c,
                                      in_c * height * width, bits, base, _stream(shift)), "COMPRESS_SIGN_SHIFT")


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False
