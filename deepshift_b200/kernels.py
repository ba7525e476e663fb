"""Python operator layer: the reference's ``deepshift.kernels`` API on the B200 kernels.

``linear``, ``conv2d`` and ``compress_sign_and_shift`` keep the names, argument order and
return values of pytorch/deepshift/kernels/kernels.py:10,28,69.  They call the C ABI of
include/deepshift_b200.h through ctypes on torch's current stream.  ``use_cuda=False`` raises:
this package has no CPU path.  Calls may be issued on several streams of a device at once: the
scratch memory the kernels share along K is kept per (device, stream).

Differences from the reference, all deliberate:
  * the convolution reads the unpadded tensor (no ``F.pad`` copy, no im2col/col2im buffers);
    ``padding=(ph, pw)`` pads H by ``ph`` and W by ``pw`` as ``torch.nn.functional.conv2d``
    does (kernels.py:32-36 swaps the two for asymmetric padding);
  * outputs are allocated with ``torch.empty`` (every element is written);
  * kernels run on the current stream of the input's device, not the legacy default stream;
  * a weight whose decoded right shift is >= 32 contributes exactly 0 (the zero-sign
    encoding of utils.py:67-70; the reference CUDA kernel yields -1 for negative inputs);
  * ``dilation != 1`` or ``groups != 1`` raises instead of being ignored (kernels.py:28).
"""
import ctypes

import torch

from . import _ffi


def _stream_ptr(device):
    return torch.cuda.current_stream(device).cuda_stream


def _check_tensor(t, name, dtype=None):
    # The reference's CHECK_INPUT (shift_cuda.cpp:22-24) plus a dtype check it lacks.
    if not t.is_cuda:
        raise RuntimeError(name + " must be a CUDA tensor")
    if not t.is_contiguous():
        raise RuntimeError(name + " must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise RuntimeError("%s must be %s, got %s" % (name, dtype, t.dtype))


def _pair(v):
    if isinstance(v, int):
        return (v, v)
    v = tuple(int(e) for e in v)
    return (v[0], v[0]) if len(v) == 1 else (v[0], v[1])


def _no_cpu():
    raise RuntimeError("deepshift_b200 has no CPU kernel path: use_cuda must be True")


_WORKSPACES = {}


_WS_COUNTERS = 16384                 # int32 arrival counters at the start of the workspace
_WS_PARTIAL_INTS = 444 * 32768 + (8 << 20)  # expanded weights of one layer (32 MiB) and partial sums:
                                             # up to 444 (tile, split) slots of 128 KiB


def workspace(device, stream=None):
    """Scratch for sharing output tiles between CTAs along K (see ds_fuse_t.workspace): zeroed
    arrival counters followed by room for expanded weights and partial sums.  One tensor per
    (device, stream): launches that share a workspace must not overlap on the GPU, and launches on
    one stream never do.  ``stream`` defaults to torch's current stream of ``device``.  Kernels leave
    the counters zero, so the tensor serves every launch of its stream in order."""
    device = torch.device(device)
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    if stream is None:
        stream = torch.cuda.current_stream(device)
    key = (device, int(stream.cuda_stream))
    ws = _WORKSPACES.get(key)
    if ws is None:
        ws = _WORKSPACES[key] = new_workspace(device)
    return ws


def new_workspace(device):
    """A workspace of its own for a caller that manages streams itself (the integer pipeline keeps
    one per instance, so two pipelines may run on two streams at once)."""
    return torch.zeros(_WS_COUNTERS + _WS_PARTIAL_INTS, dtype=torch.int32, device=device)


def last_kernel_error():
    """1 if a kernel's bounded wait ran out since the last call (its output is then undefined), else
    0.  Synchronises the current device and clears the flag."""
    flag = ctypes.c_int(-1)
    _ffi.check(_ffi.lib().ds_last_kernel_error(ctypes.byref(flag)), "last_kernel_error")
    return flag.value


def _fuse(in_kind=0, out_kind=0, act_integer_bits=0, act_fraction_bits=0, relu=False, requant=False,
          residual=None, act_bits=0, round_f32=False, workspace=None):
    f = _ffi.Fuse()
    f.in_kind, f.out_kind = in_kind, out_kind
    f.act_integer_bits, f.act_fraction_bits = int(act_integer_bits), int(act_fraction_bits)
    f.relu, f.requant = int(bool(relu)), int(bool(requant))
    f.residual = residual.data_ptr() if residual is not None else None
    f.act_bits = int(act_bits)
    f.round_f32 = int(bool(round_f32))
    if workspace is not None:
        f.workspace = workspace.data_ptr()
        f.workspace_bytes = workspace.numel() * workspace.element_size()
    return f


ACT_BITS_AUTO = -1   # DS_ACT_BITS_AUTO: the library measures the range of the activations on the device


def linear(input, shift, sign, bias=None, conc_weight=None, use_cuda=True, act_bits=None):
    """int32 [M,K] -> int32 [M,N].  ``shift``/``sign`` only give N (as in kernels.py:14).

    ``act_bits`` (not in the reference): a promise that every |x| <= 2^(act_bits-1), which selects the
    FP32-pipe path (1..18); 0 = the exact integer path; None (default) = let the library look at the
    data and take the FP32-pipe path when it can (see DS_ACT_BITS_AUTO).  Results are identical."""
    if not use_cuda:
        _no_cpu()
    assert conc_weight is not None
    _check_tensor(input, "input", torch.int32)
    _check_tensor(conc_weight.data, "conc_weight.data", torch.int32)
    if bias is not None:
        _check_tensor(bias, "bias", torch.int32)
    M, K = input.shape
    N = shift.size(0)
    out = torch.empty([M, N], dtype=torch.int32, device=input.device)
    # ds_linear_i32 plus the workspace (expanded weights, shared tiles when few tiles fill the SMs)
    f = _fuse(act_bits=ACT_BITS_AUTO if act_bits is None else act_bits,
              workspace=workspace(input.device) if M > 64 else None)
    with torch.cuda.device(input.device):
        rc = _ffi.lib().ds_linear_ex(input.data_ptr(), conc_weight.data.data_ptr(),
                                     bias.data_ptr() if bias is not None else None, out.data_ptr(),
                                     M, K, N, conc_weight.bits, conc_weight.base, f,
                                     _stream_ptr(input.device))
    _ffi.check(rc, "linear")
    return out


def _conv_geometry(input, shift, stride, padding, dilation, groups):
    if _pair(dilation) != (1, 1) or groups != 1:
        raise RuntimeError("the shift convolution kernel supports neither dilation nor groups")
    sh, sw = _pair(stride)
    ph, pw = _pair(padding)
    B, C, H, W = input.shape
    OC, KH, KW = shift.size(0), shift.size(2), shift.size(3)
    OH, OW = (H + 2 * ph - KH) // sh + 1, (W + 2 * pw - KW) // sw + 1
    return B, C, H, W, OC, KH, KW, sh, sw, ph, pw, OH, OW


def conv2d(input, shift, sign, bias=None, conc_weight=None, stride=1, padding=0, dilation=1, groups=1,
           use_cuda=True, act_bits=None):
    """int32 NCHW (unpadded) -> int32 NCHW.  ``act_bits``: see ``linear``."""
    if not use_cuda:
        _no_cpu()
    assert conc_weight is not None
    _check_tensor(input, "input", torch.int32)
    _check_tensor(conc_weight.data, "conc_weight.data", torch.int32)
    if bias is not None:
        _check_tensor(bias, "bias", torch.int32)
    B, C, H, W, OC, KH, KW, sh, sw, ph, pw, OH, OW = _conv_geometry(input, shift, stride, padding, dilation, groups)
    out = torch.empty([B, OC, OH, OW], dtype=torch.int32, device=input.device)
    # ds_conv2d_i32 plus the split-K counter workspace (layers with few output tiles)
    f = _fuse(act_bits=ACT_BITS_AUTO if act_bits is None else act_bits, workspace=workspace(input.device))
    with torch.cuda.device(input.device):
        rc = _ffi.lib().ds_conv2d_ex(input.data_ptr(), conc_weight.data.data_ptr(),
                                     bias.data_ptr() if bias is not None else None, out.data_ptr(),
                                     B, C, H, W, OC, KH, KW, sh, sw, ph, pw, conc_weight.bits,
                                     conc_weight.base, f, _stream_ptr(input.device))
    _ffi.check(rc, "conv2d")
    return out


def compress_sign_and_shift(shift, sign, comp_size, base, bits, row_length, num):
    """(shift', sign) int32 [OC,IC,KH,KW] -> packed int32 [comp_size] (kernels.py:69-74)."""
    _check_tensor(shift, "shift", torch.int32)
    _check_tensor(sign, "sign", torch.int32)
    OC = shift.shape[0]
    K = shift.numel() // OC
    if num != 32 // (bits + 1) or row_length != (K + num - 1) // num or comp_size != row_length * OC:
        raise RuntimeError("inconsistent packing geometry")
    comp_weight = torch.empty([comp_size], dtype=torch.int32, device=shift.device)
    with torch.cuda.device(shift.device):
        rc = _ffi.lib().ds_compress(shift.data_ptr(), sign.data_ptr(), comp_weight.data_ptr(), OC, K,
                                    bits, base, _stream_ptr(shift.device))
    _ffi.check(rc, "compress_sign_and_shift")
    return comp_weight


# ------------------------------------------------------------------------------------------------
# Fused forms used by the modules and the integer pipeline (no counterpart in the reference,
# which runs the quantise / convert / ReLU steps as separate torch passes).

def linear_fused(input, out_features, bias_i32, conc_weight, *, in_kind=_ffi.IN_I32, out_kind=_ffi.OUT_I32,
                 act_integer_bits=16, act_fraction_bits=16, relu=False, requant=False, residual=None,
                 act_bits=0, round_f32=False, out=None):
    _check_tensor(input, "input", torch.int32 if in_kind in (_ffi.IN_I32, _ffi.IN_I32_CLAMP) else torch.float32)
    M, K = input.shape
    if out is None:
        out = torch.empty([M, out_features], device=input.device,
                          dtype=torch.int32 if out_kind == _ffi.OUT_I32 else torch.float32)
    f = _fuse(in_kind, out_kind, act_integer_bits, act_fraction_bits, relu, requant, residual, act_bits, round_f32,
              workspace(input.device) if M > 64 else None)
    with torch.cuda.device(input.device):
        rc = _ffi.lib().ds_linear_ex(input.data_ptr(), conc_weight.data.data_ptr(),
                                     bias_i32.data_ptr() if bias_i32 is not None else None, out.data_ptr(),
                                     M, K, out_features, conc_weight.bits, conc_weight.base, f,
                                     _stream_ptr(input.device))
    _ffi.check(rc, "linear_fused")
    return out


def _prepared_weights(conc_weight, geometry, fuse, device):
    """The layer's weights expanded once for this geometry and arithmetic path (ds_conv2d_prepare),
    kept on the ``ConcWeight`` they were made from: a new ``ConcWeight`` (re-packed weights) starts
    with an empty cache; packed data changed in place would not be noticed.  None when launches of
    this geometry do not use expanded weights."""
    cache = conc_weight.__dict__.setdefault("_prepared", {})
    key = geometry + (fuse.in_kind, fuse.act_bits, fuse.act_integer_bits, fuse.act_fraction_bits,
                      conc_weight.data.data_ptr(), str(device))
    if key not in cache:
        lib, need = _ffi.lib(), ctypes.c_longlong(0)
        args = (conc_weight.data.data_ptr(),) + geometry + (conc_weight.bits, conc_weight.base)
        fuse.prepared, fuse.prepared_bytes = None, 0
        _ffi.check(lib.ds_conv2d_prepare(*args, fuse, ctypes.byref(need), _stream_ptr(device)), "conv2d_prepare")
        buf = None
        if need.value > 0:
            buf = torch.empty(need.value // 4, dtype=torch.int32, device=device)
            fuse.prepared, fuse.prepared_bytes = buf.data_ptr(), need.value
            _ffi.check(lib.ds_conv2d_prepare(*args, fuse, ctypes.byref(need), _stream_ptr(device)),
                       "conv2d_prepare")
            fuse.prepared, fuse.prepared_bytes = None, 0
        cache[key] = buf
    return cache[key]


def conv2d_fused(input, weight_shape, bias_i32, conc_weight, stride=1, padding=0, *, in_kind=_ffi.IN_I32,
                 out_kind=_ffi.OUT_I32, act_integer_bits=16, act_fraction_bits=16, relu=False, requant=False,
                 residual=None, act_bits=0, round_f32=False, out=None):
    _check_tensor(input, "input", torch.int32 if in_kind in (_ffi.IN_I32, _ffi.IN_I32_CLAMP) else torch.float32)
    sh, sw = _pair(stride)
    ph, pw = _pair(padding)
    B, C, H, W = input.shape
    OC, C2, KH, KW = weight_shape
    if C2 != C:
        raise RuntimeError("input has %d channels, weight expects %d" % (C, C2))
    OH, OW = (H + 2 * ph - KH) // sh + 1, (W + 2 * pw - KW) // sw + 1
    if out is None:
        out = torch.empty([B, OC, OH, OW], device=input.device,
                          dtype=torch.int32 if out_kind == _ffi.OUT_I32 else torch.float32)
    if residual is not None:
        _check_tensor(residual, "residual", torch.int32)
        if residual.shape != out.shape:
            raise RuntimeError("residual shape %s != output shape %s" % (tuple(residual.shape), tuple(out.shape)))
    f = _fuse(in_kind, out_kind, act_integer_bits, act_fraction_bits, relu, requant, residual, act_bits, round_f32,
              workspace(input.device))
    geometry = (B, C, H, W, OC, KH, KW, sh, sw, ph, pw)
    with torch.cuda.device(input.device):
        prepared = _prepared_weights(conc_weight, geometry, f, input.device)
        if prepared is not None:
            f.prepared = prepared.data_ptr()
            f.prepared_bytes = prepared.numel() * 4
        rc = _ffi.lib().ds_conv2d_ex(input.data_ptr(), conc_weight.data.data_ptr(),
                                     bias_i32.data_ptr() if bias_i32 is not None else None, out.data_ptr(),
                                     B, C, H, W, OC, KH, KW, sh, sw, ph, pw, conc_weight.bits,
                                     conc_weight.base, f, _stream_ptr(input.device))
    _ffi.check(rc, "conv2d_fused")
    return out


def quantize(input, act_integer_bits, act_fraction_bits, like_conv=True):
    """fp32 -> int32 fixed point in one pass (utils.py:7-21 + modules.py:153, or modules.py:25)."""
    _check_tensor(input, "input", torch.float32)
    out = torch.empty(input.shape, dtype=torch.int32, device=input.device)
    with torch.cuda.device(input.device):
        rc = _ffi.lib().ds_quantize_f32(input.data_ptr(), out.data_ptr(), input.numel(),
                                        _ffi.IN_F32_CONV if like_conv else _ffi.IN_F32_LINEAR,
                                        act_integer_bits, act_fraction_bits, _stream_ptr(input.device))
    _ffi.check(rc, "quantize")
    return out


def maxpool2d_i32(input, kernel_size, stride, padding=0, out=None):
    """Max pooling of int32 fixed-point NCHW activations (exact counterpart of F.max_pool2d on
    the fp32 values)."""
    _check_tensor(input, "input", torch.int32)
    B, C, H, W = input.shape
    OH = (H + 2 * padding - kernel_size) // stride + 1
    OW = (W + 2 * padding - kernel_size) // stride + 1
    if out is None:
        out = torch.empty([B, C, OH, OW], dtype=torch.int32, device=input.device)
    with torch.cuda.device(input.device):
        rc = _ffi.lib().ds_maxpool2d_i32(input.data_ptr(), out.data_ptr(), B, C, H, W, kernel_size, stride,
                                         padding, _stream_ptr(input.device))
    _ffi.check(rc, "maxpool2d_i32")
    return out


def maxpool2d_f32(input, kernel_size, stride, padding=0):
    """``F.max_pool2d(input, kernel_size, stride, padding)`` on fp32 NCHW, bit for bit (square window, no
    dilation, floor mode), on this library's pooling kernels."""
    _check_tensor(input, "input", torch.float32)
    B, C, H, W = input.shape
    OH = (H + 2 * padding - kernel_size) // stride + 1
    OW = (W + 2 * padding - kernel_size) // stride + 1
    out = torch.empty([B, C, OH, OW], dtype=torch.float32, device=input.device)
    with torch.cuda.device(input.device):
        rc = _ffi.lib().ds_maxpool2d_f32(input.data_ptr(), out.data_ptr(), B, C, H, W, kernel_size, stride,
                                         padding, _stream_ptr(input.device))
    _ffi.check(rc, "maxpool2d_f32")
    return out


def add_relu_f32_(y, residual=None, relu=False):
    """In place, one pass: ``y += residual`` (when given), then ``y = relu(y)`` (when asked) -- the
    fp32 glue after a shift layer in a residual block, bit-identical to the two torch ops."""
    _check_tensor(y, "y", torch.float32)
    if residual is not None:
        _check_tensor(residual, "residual", torch.float32)
        if residual.shape != y.shape:
            raise RuntimeError("residual shape %s != output shape %s" % (tuple(residual.shape), tuple(y.shape)))
    with torch.cuda.device(y.device):
        rc = _ffi.lib().ds_add_relu_f32(y.data_ptr(), residual.data_ptr() if residual is not None else None,
                                        y.numel(), int(bool(relu)), _stream_ptr(y.device))
    _ffi.check(rc, "add_relu_f32_")
    return y


def avgpool_fix_i32(input, act_fraction_bits, out=None):
    """Global average pooling of int32 activations followed by the LinearShift entry conversion;
    returns int32 [B, C]."""
    _check_tensor(input, "input", torch.int32)
    B, C, H, W = input.shape
    if out is None:
        out = torch.empty([B, C], dtype=torch.int32, device=input.device)
    with torch.cuda.device(input.device):
        rc = _ffi.lib().ds_avgpool_fix_i32(input.data_ptr(), out.data_ptr(), B, C, H, W, act_fraction_bits,
                                           _stream_ptr(input.device))
    _ffi.check(rc, "avgpool_fix_i32")
    return out


def pipe_peak(mode, iters=20000):
    """Sustained shift-accumulate operations per second of one instruction mix (see the header)."""
    import ctypes
    v = ctypes.c_double(0.0)
    rc = _ffi.lib().ds_pipe_peak(mode, iters, ctypes.byref(v), _stream_ptr(torch.cuda.current_device()))
    _ffi.check(rc, "pipe_peak")
    return v.value
