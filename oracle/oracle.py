"""Python face of the CPU oracle (TEST INFRASTRUCTURE ONLY).

Only tests/, ``__graft_entry__.smoke()`` and the cpu_baseline / reference legs of
``bench.py`` import this module, and only as the checker.  Nothing under ``deepshift_b200/``
imports it.

The integer kernels live in ``ds_oracle.c`` (built by ``oracle/Makefile``); the float glue of
the reference's Python layer is restated here in numpy:

* ``round_to_fixed``       <- pytorch/deepshift/utils.py:7-21
* ``to_fixed_linear``      <- pytorch/deepshift/modules.py:24-27   (trunc toward zero, no clamp)
* ``to_fixed_conv``        <- pytorch/deepshift/modules.py:152-157,317-321 (floor + clamp)
* ``from_fixed``           <- pytorch/deepshift/modules.py:30-31,161-162
* ``compress_bits``        <- pytorch/deepshift/utils.py:61-88 (host half of the packing)

Parity pin: ``tests/test_oracle.py`` checks the C functions against the reference's compiled
``deepshift_cpu`` module (``oracle/_ref``, when present) and against ``tests/golden/*.npz``
(outputs of that module, written by ``tests/golden/make_golden.py``).
"""
import ctypes
import importlib.util
import math
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(HERE, "_build", "libds_oracle.so")
_lib = None

_I32P = ctypes.POINTER(ctypes.c_int32)


def build(force=False):
    """Compile ds_oracle.c (a few hundred ms)."""
    src = os.path.join(HERE, "ds_oracle.c")
    if (not force and os.path.exists(_LIB_PATH)
            and os.path.getmtime(_LIB_PATH) >= os.path.getmtime(src)):
        return _LIB_PATH
    env = dict(os.environ)
    env.pop("CC", None)
    subprocess.run(["make", "-C", HERE, "-B"], check=True, env=env,
                   stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(_I32P)


def _i32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.int32)


def num_threads():
    return int(lib().dso_num_threads())


# ----------------------------------------------------------------------------- integer kernels
def linear(x, shift, sign, bias=None):
    """int32 [M,K] x (shift,sign [N,K]) -> int32 [M,N]; shift_cpu.cpp:109-229."""
    x, shift, sign, bias = _i32(x), _i32(shift), _i32(sign), _i32(bias)
    M, K = x.shape
    N = shift.shape[0]
    assert shift.shape == (N, K) and sign.shape == (N, K)
    out = np.empty((M, N), dtype=np.int32)
    lib().dso_linear(_p(x), _p(shift), _p(sign), _p(bias), _p(out), M, K, N)
    return out


def pad_nchw(x, ph, pw):
    x = _i32(x)
    B, C, H, W = x.shape
    ph, pw = int(ph), int(pw)
    xp = np.empty((B, C, H + 2 * ph, W + 2 * pw), dtype=np.int32)
    lib().dso_pad_nchw(_p(x), _p(xp), B, C, H, W, ph, pw)
    return xp


def conv2d(x, shift, sign, bias=None, stride=(1, 1), padding=(0, 0), zero_sign_as_plus=False):
    """Unpadded int32 NCHW in, int32 NCHW out.

    Zero padding as kernels.py:32-36, then the direct convolution of shift_cpu.cpp:295-374.
    ``zero_sign_as_plus=True`` reproduces that kernel's treatment of sign == 0 (added as +1);
    the default is the canonical rule of the linear kernel (sign 0 contributes nothing).
    """
    x, shift, sign, bias = _i32(x), _i32(shift), _i32(sign), _i32(bias)
    sh, sw = int(stride[0]), int(stride[1])
    ph, pw = int(padding[0]), int(padding[1])
    xp = pad_nchw(x, ph, pw) if (ph or pw) else x
    B, C, Hp, Wp = xp.shape
    OC, C2, KH, KW = shift.shape
    assert C2 == C and sign.shape == shift.shape
    OH, OW = (Hp - KH) // sh + 1, (Wp - KW) // sw + 1
    out = np.empty((B, OC, OH, OW), dtype=np.int32)
    lib().dso_conv2d_prepadded(_p(xp), _p(shift), _p(sign), _p(bias), _p(out), B, C, Hp, Wp,
                               OC, KH, KW, sh, sw, int(bool(zero_sign_as_plus)))
    return out


def im2col(xp, KH, KW, stride=(1, 1)):
    xp = _i32(xp)
    B, C, Hp, Wp = xp.shape
    sh, sw = int(stride[0]), int(stride[1])
    OH, OW = (Hp - KH) // sh + 1, (Wp - KW) // sw + 1
    col = np.empty((B * OH * OW, C * KH * KW), dtype=np.int32)
    lib().dso_im2col(_p(xp), _p(col), B, C, Hp, Wp, KH, KW, sh, sw)
    return col


def col2im(col, B, OC, OH, OW):
    col = _i32(col)
    im = np.empty((B, OC, OH, OW), dtype=np.int32)
    lib().dso_col2im(_p(col), _p(im), B, OC, OH, OW)
    return im


def conv2d_via_gemm(x, shift, sign, bias=None, stride=(1, 1), padding=(0, 0)):
    """The reference CUDA decomposition (shift.cu:399-669): pad, IM2COL, shift-GEMM, COL2IM,
    evaluated with the linear kernel's arithmetic.  Used to cross-check ``conv2d``."""
    x, shift = _i32(x), _i32(shift)
    OC, C, KH, KW = shift.shape
    stride = (int(stride[0]), int(stride[1]))
    xp = pad_nchw(x, *padding) if (padding[0] or padding[1]) else x
    B, _, Hp, Wp = xp.shape
    OH, OW = (Hp - KH) // stride[0] + 1, (Wp - KW) // stride[1] + 1
    col = im2col(xp, KH, KW, stride)
    o = linear(col, shift.reshape(OC, -1), _i32(sign).reshape(OC, -1), bias)
    return col2im(o, B, OC, OH, OW)


def compress(shiftp, sign, bits, base):
    """(shift', sign) [OC,K] -> packed int32 [OC, ceil(K/num)]; shift.cu:27-55."""
    shiftp, sign = _i32(shiftp), _i32(sign)
    OC, K = shiftp.shape
    num = 32 // (bits + 1)
    packed = np.empty((OC, (K + num - 1) // num), dtype=np.int32)
    lib().dso_compress(_p(shiftp), _p(sign), _p(packed), OC, K, bits, base)
    return packed


def linear_packed(x, packed, bias, K, bits, base):
    """Shift-GEMM on packed words with the decode of shift.cu:92-111."""
    x, packed, bias = _i32(x), _i32(packed), _i32(bias)
    M = x.shape[0]
    N = packed.shape[0]
    out = np.empty((M, N), dtype=np.int32)
    lib().dso_linear_packed(_p(x), _p(packed), _p(bias), _p(out), M, K, N, bits, base)
    return out


# ----------------------------------------------------------------------------- float glue
def round_to_fixed(v, integer_bits=16, fraction_bits=16):
    """utils.py:7-21 in float32: floor to the 2^-F grid, clamp to [-2^(I-1), 2^(I-1)-1]."""
    v = np.asarray(v, dtype=np.float32)
    assert integer_bits >= 1
    if integer_bits == 1:
        return (np.sign(v) - 1).astype(np.float32)
    delta = np.float32(math.pow(2.0, -fraction_bits))
    bound = math.pow(2.0, integer_bits - 1)
    rounded = np.floor(v / delta).astype(np.float32) * delta
    return np.clip(rounded, np.float32(-bound), np.float32(bound - 1)).astype(np.float32)


def to_fixed_linear(v, fraction_bits):
    """modules.py:25,27: (v * 2^F).int() -- truncation toward zero, no clamp."""
    return np.trunc(np.asarray(v, np.float32) * np.float32(2 ** fraction_bits)).astype(np.int32)


def to_fixed_conv(v, integer_bits, fraction_bits):
    """modules.py:317-321 then 153-157: round_to_fixed followed by (v * 2^F).int()."""
    q = round_to_fixed(v, integer_bits, fraction_bits)
    return np.trunc(q * np.float32(2 ** fraction_bits)).astype(np.int32)


def from_fixed(o, fraction_bits):
    """modules.py:30-31,161-162: out.float() / 2^F."""
    return np.asarray(o, np.int32).astype(np.float32) / np.float32(2 ** fraction_bits)


def global_avg(x):
    """Global average pool of fp32 NCHW planes as torch computes it on the CPU for the reference's
    ResNets (cifar10_models/resnet.py:122-134 ``F.avg_pool2d(out, out.size()[3])``; torchvision's
    ``AdaptiveAvgPool2d(1)`` behind imagenet.py:199-219, which is ``mean`` over H and W): an fp32
    sum followed by an IEEE division by H*W.  The sum is formed exactly (float64) and rounded
    once; that equals torch's vectorised fp32 sum whenever the plane's sum of 2^-F codes stays
    below 2^24 (pinned by tests/golden/gap_ref.npz).  Beyond that torch's own result depends on
    the vector width of the CPU, and its CUDA kernel multiplies by a rounded 1/(H*W) instead."""
    x = np.asarray(x, dtype=np.float32)
    s = x.astype(np.float64).sum(axis=(2, 3)).astype(np.float32)
    return (s / np.float32(x.shape[2] * x.shape[3])).astype(np.float32)


def compress_bits(shift, sign):
    """Host half of the packing, utils.py:61-88, with the evident intent of lines 67-70
    (a weight whose sign is 0 becomes sign +1, shift -32) applied by mask on copies.

    Returns (packed [OC,row_len], base, bits).  For base < 0 (some positive shift) the stored
    field is ``-shift - base`` so that field + base is the true right-shift amount.
    """
    shift = np.array(shift, dtype=np.int64)
    sign = np.array(sign, dtype=np.int64)
    if shift.ndim == 2:
        shift = shift[:, :, None, None]
        sign = sign[:, :, None, None]
    zero = sign == 0
    shift[zero] = -32
    sign[zero] = 1
    shiftp = -shift
    minimum = int(shiftp.min())
    base = minimum if minimum < 0 else 0
    bits = max(1, (int(shiftp.max()) - base).bit_length())  # == ceil(log2(max + 1)), utils.py:72
    OC = shift.shape[0]
    return compress(shiftp.reshape(OC, -1), sign.reshape(OC, -1), bits, base), base, bits


# ----------------------------------------------------------------------------- compiled reference
_ref_mod = None


def ref_module():
    """The reference's own ``deepshift_cpu`` pybind module from oracle/_ref, or None."""
    global _ref_mod
    if _ref_mod is None:
        import sysconfig
        path = os.path.join(HERE, "_ref", "deepshift_cpu" + sysconfig.get_config_var("EXT_SUFFIX"))
        if not os.path.exists(path):
            return None
        import torch  # noqa: F401  (the module links against libtorch)
        spec = importlib.util.spec_from_file_location("deepshift_cpu", path)
        _ref_mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(_ref_mod)
    return _ref_mod


def ref_linear(x, shift, sign, bias):
    """deepshift_cpu.linear_kernel exactly as kernels.py:23 calls it."""
    out = ref_module().linear_kernel(_i32(x), np.ascontiguousarray(shift, dtype=np.int8),
                                     _i32(sign), _i32(bias))
    return np.asarray(out, dtype=np.int32)


def ref_conv2d_prepadded(xp, shift, sign, bias, stride):
    """deepshift_cpu.convolution_kernel on an already padded input (kernels.py:59-62)."""
    out = ref_module().convolution_kernel(_i32(xp), np.ascontiguousarray(shift, dtype=np.int8),
                                          _i32(sign), _i32(bias), list(stride), [0, 0])
    return np.asarray(out, dtype=np.int32)
