"""Staged activations and the TMA-fed convolution (see the "Staged activations" part of
include/deepshift_b200.h).  No counterpart in the reference, which materialises the im2col matrix
(pytorch/deepshift/kernels/cuda/shift.cu:122-153) and keeps activations fp32 NCHW between layers.

``StagedTensor`` owns a staged buffer (fp32 NHWC, value = code + 0.5, halo of 0.5);
``conv2d`` runs one shift convolution on it and writes any of: int32 NHWC codes, fp32 NHWC, NCHW
(int32 or fp32) and the staged operand of the next layer.  Bit-identical to ``kernels.conv2d``.
"""
import ctypes

import torch

from . import _ffi, kernels


class StagedTensor:
    def __init__(self, B, H, W, C, halo, device):
        self.B, self.H, self.W, self.C, self.halo = int(B), int(H), int(W), int(C), int(halo)
        self.Cs = (self.C + 3) // 4 * 4
        self.device = torch.device(device)
        self.data = torch.empty((self.B, self.H + 2 * self.halo, self.W + 2 * self.halo, self.Cs),
                                dtype=torch.float32, device=self.device)
        self.c = _ffi.Staged(self.data.data_ptr(), self.B, self.H, self.W, self.C, self.halo)
        with torch.cuda.device(self.device):
            _ffi.check(_ffi.lib().ds_staged_fill(ctypes.byref(self.c), kernels._stream_ptr(self.device)), "staged_fill")

    def codes(self):
        """The int32 codes of the interior as an NCHW tensor (for tests)."""
        h = self.halo
        v = self.data[:, h:h + self.H, h:h + self.W, :self.C] - 0.5
        return v.permute(0, 3, 1, 2).contiguous().to(torch.int32)


def stage_nchw(x, act_integer_bits, act_fraction_bits, halo, in_kind=None, out=None):
    """NCHW fp32 (quantised as Conv2dShift does) or int32 codes -> StagedTensor."""
    kernels._check_tensor(x, "input")
    if in_kind is None:
        in_kind = _ffi.IN_F32_CONV if x.dtype == torch.float32 else _ffi.IN_I32_CLAMP
    want = torch.float32 if in_kind == _ffi.IN_F32_CONV else torch.int32
    if x.dtype != want:
        raise RuntimeError("input must be %s for this input kind" % want)
    B, C, H, W = x.shape
    if out is None:
        out = StagedTensor(B, H, W, C, halo, x.device)
    with torch.cuda.device(x.device):
        rc = _ffi.lib().ds_stage_nchw(x.data_ptr(), in_kind, act_integer_bits, act_fraction_bits, ctypes.byref(out.c),
                                      kernels._stream_ptr(x.device))
    _ffi.check(rc, "stage_nchw")
    return out


def prepared_weights(conc_weight, C, OC, KH, KW, device):
    """The layer's weights expanded for the staged kernel, cached on the ``ConcWeight``."""
    if conc_weight.base != 0:
        raise RuntimeError("the staged convolution needs right shifts only (base == 0)")
    cache = conc_weight.__dict__.setdefault("_prepared", {})
    key = ("staged", C, OC, KH, KW, conc_weight.data.data_ptr(), str(device))
    if key not in cache:
        lib, need = _ffi.lib(), ctypes.c_longlong(0)
        args = (conc_weight.data.data_ptr(), C, OC, KH, KW, conc_weight.bits, conc_weight.base)
        with torch.cuda.device(device):
            _ffi.check(lib.ds_staged_prepare(*args, None, 0, ctypes.byref(need), kernels._stream_ptr(device)),
                       "staged_prepare")
            buf = torch.empty(need.value // 4, dtype=torch.int32, device=device)
            _ffi.check(lib.ds_staged_prepare(*args, buf.data_ptr(), need.value, ctypes.byref(need),
                                             kernels._stream_ptr(device)), "staged_prepare")
        cache[key] = buf
    return cache[key]


def conv2d(x, weight_shape, bias_i32, conc_weight, stride=1, padding=0, *, act_integer_bits=4, act_fraction_bits=12,
           in_act_bits=None, relu=False, round_f32=False, residual=None, out_codes=None, out_f32=None, out_nchw=None,
           out_staged=None, workspace=None):
    """x: StagedTensor.  Outputs are the tensors passed in (``out_codes`` int32 [B,OH,OW,OC], ``out_f32`` fp32
    of the same shape, ``out_nchw`` int32 or fp32 [B,OC,OH,OW], ``out_staged`` a StagedTensor); at least
    one is needed.  ``residual``: int32 [B,OH,OW,OC].  Returns None."""
    sh, sw = kernels._pair(stride)
    ph, pw = kernels._pair(padding)
    OC, C, KH, KW = weight_shape
    if C != x.C:
        raise RuntimeError("input has %d channels, weight expects %d" % (x.C, C))
    prepared = prepared_weights(conc_weight, C, OC, KH, KW, x.device)
    o = _ffi.StagedOut()
    o.codes = out_codes.data_ptr() if out_codes is not None else None
    o.f32 = out_f32.data_ptr() if out_f32 is not None else None
    if out_nchw is not None:
        o.nchw, o.nchw_is_f32 = out_nchw.data_ptr(), int(out_nchw.dtype == torch.float32)
    if out_staged is not None:
        o.staged = ctypes.pointer(out_staged.c)
    o.residual = residual.data_ptr() if residual is not None else None
    o.relu, o.round_f32 = int(bool(relu)), int(bool(round_f32))
    o.act_integer_bits, o.act_fraction_bits = int(act_integer_bits), int(act_fraction_bits)
    from . import utils
    o.in_act_bits = int(in_act_bits if in_act_bits is not None else utils.code_bits(act_integer_bits, act_fraction_bits))
    if workspace is None:
        workspace = kernels.workspace(x.device)
    with torch.cuda.device(x.device):
        rc = _ffi.lib().ds_staged_conv2d(ctypes.byref(x.c), prepared.data_ptr(), prepared.numel() * 4,
                                         bias_i32.data_ptr() if bias_i32 is not None else None, OC, KH, KW, sh, sw,
                                         ph, pw, ctypes.byref(o), workspace.data_ptr(),
                                         workspace.numel() * workspace.element_size(), kernels._stream_ptr(x.device))
    _ffi.check(rc, "staged_conv2d")
