"""DeepShift-Q modules with the reference's constructor signatures and attributes
(pytorch/deepshift/modules_q.py:70-135, 200-300), inference only.

A DeepShift-Q layer keeps an fp32 ``weight`` and rounds it to a signed power of two on the fly:
``sign = sign(w)``, ``shift = round(log2 |w|)`` after ``|w|`` was clamped to
``[2^shift_range[0], 1]`` (modules_q.py:117-118, 283-284).  With ``use_kernel=True`` the
reference hands that (shift, sign) pair to the same ``deepshift.kernels`` entry points as
DeepShift-PS (modules_q.py:21-31, 147-161), so here the layer packs the rounded weights into a
``ConcWeight`` once per weight version and runs the same fused B200 kernels as
``deepshift_b200.modules``: input quantised by ``round_to_fixed`` (both layer kinds do that in
DeepShift-Q, modules_q.py:119, 285), bias rounded to fixed point, int32 shift-accumulate,
``out.float() / 2**F``.

Where the reference cannot serve as the rule:
  * ``LinearShiftQ.forward`` passes its arguments to ``LinearShiftQFunction`` one position off
    (modules_q.py:126: ``act_integer_bits`` lands in ``rounding``) and ``bias_fixed_point`` is
    unbound without a bias (modules_q.py:25-29); the layer here does what ``Conv2dShiftQ`` does.
  * ``convert_to_shift`` packs the weights before the first forward pass clamps them
    (convert.py:29-30, 61-62); here the packed weights always come from the clamped ones, so the
    kernel path and the ``use_kernel=False`` path use the same rounded weights.
``use_cuda=False`` raises: there is no CPU kernel path.
"""
import math

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.nn import init
from torch.nn.modules.utils import _pair

from . import _ffi, kernels, utils


class _ShiftQBase(nn.Module):
    """Cached fixed-point bias and packed weights, both keyed on the parameter's version."""

    def _clamped_weight(self):
        # modules_q.py:117, 283: the clamp is written back into the parameter
        self.weight.data = utils.clampabs(self.weight.data, 2 ** self.shift_range[0], 2 ** self.shift_range[1])
        return self.weight

    def _bias_fixed(self):
        if self.bias is None:
            return None
        key = (self.bias.data_ptr(), self.bias._version, self.bias.device)
        if getattr(self, "_bias_key", None) != key:
            b = utils.round_to_fixed(self.bias.detach().float(), self.act_integer_bits, self.act_fraction_bits)
            self._bias_i32 = (b * (2 ** self.act_fraction_bits)).int().contiguous()
            self._bias_key = key
        return self._bias_i32

    def _packed(self, device):
        key = (self.weight.data_ptr(), self.weight._version, device)
        if self.conc_weight is None or getattr(self, "_weight_key", None) != key:
            w = self._clamped_weight().detach().float()
            key = (self.weight.data_ptr(), self.weight._version, device)
            shift, sign = utils.get_shift_and_sign(w, 'deterministic')
            self.conc_weight = utils.compress_bits(shift, sign, device=device)
            self._weight_key = key
        return self.conc_weight

    def _check_kernel_mode(self):
        if not self.use_cuda:
            raise RuntimeError("deepshift_b200 has no CPU kernel path: use_kernel=True needs use_cuda=True")

    def _input_codes(self, x):
        """round_to_fixed(x, I, F) * 2^F as int32 (modules_q.py:119 + 24, 285 + 150), one pass."""
        return kernels.quantize(x.float().contiguous(), self.act_integer_bits, self.act_fraction_bits,
                                like_conv=True)

    def _act_bits(self):
        # the bound on the codes, which is what the FP32-pipe path needs to know
        return utils.code_bits(self.act_integer_bits, self.act_fraction_bits)


class LinearShiftQ(_ShiftQBase):
    def __init__(self, in_features, out_features, bias=True, check_grad=False, use_kernel=False,
                 use_cuda=True, rounding='deterministic', weight_bits=5, act_integer_bits=16,
                 act_fraction_bits=16):
        super(LinearShiftQ, self).__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.use_kernel = use_kernel
        self.check_grad = check_grad
        self.use_cuda = use_cuda
        self.conc_weight = None
        self.rounding = rounding
        self.shift_range = (-1 * (2 ** (weight_bits - 1) - 1), 0)  # modules_q.py:81
        self.act_integer_bits, self.act_fraction_bits = act_integer_bits, act_fraction_bits
        dtype = torch.float64 if check_grad else torch.float32
        self.weight = nn.Parameter(torch.empty(out_features, in_features, dtype=dtype))
        if bias:
            self.bias = nn.Parameter(torch.empty(out_features, dtype=dtype))
        else:
            self.register_parameter('bias', None)
        self.reset_parameters()

    def reset_parameters(self):
        init.kaiming_uniform_(self.weight, a=math.sqrt(5))
        if self.bias is not None:
            fan_in, _ = init._calculate_fan_in_and_fan_out(self.weight)
            bound = 1 / math.sqrt(fan_in)
            init.uniform_(self.bias, -bound, bound)

    def forward(self, input, residual=None, relu=False):
        """``residual`` and ``relu`` are optional fusion hints (no counterpart in the reference, whose
        forward takes the input only): the result equals ``F.relu(self(input) + residual)`` (each part
        only when given) bit for bit.  With ``use_kernel=True`` a ReLU alone happens in the layer's
        epilogue; with a residual, addition and ReLU are one in-place pass over the output instead of
        two torch kernels."""
        if self.use_kernel:
            self._check_kernel_mode()
            x = self._input_codes(input.reshape(-1, self.in_features))
            out = kernels.linear_fused(x, self.out_features, self._bias_fixed(), self._packed(x.device),
                                       in_kind=_ffi.IN_I32, out_kind=_ffi.OUT_F32,
                                       act_integer_bits=self.act_integer_bits,
                                       act_fraction_bits=self.act_fraction_bits, act_bits=self._act_bits(),
                                       relu=relu and residual is None)
            if residual is not None:
                kernels.add_relu_f32_(out, residual.reshape(-1, self.out_features).float().contiguous(), relu)
            return out.reshape(*input.shape[:-1], self.out_features)
        weight_q = utils.round_power_of_2(self._clamped_weight(), self.rounding)
        input_fixed_point = utils.round_to_fixed(input, self.act_integer_bits, self.act_fraction_bits)
        out = input_fixed_point.mm(weight_q.t())
        if self.bias is not None:
            out += self.bias.unsqueeze(0).expand_as(out)  # unrounded, as modules_q.py:130
        if residual is not None:
            out = out + residual
        return F.relu(out) if relu else out

    def extra_repr(self):
        return 'in_features={}, out_features={}, bias={}'.format(
            self.in_features, self.out_features, self.bias is not None)


class _ConvNdShiftQ(_ShiftQBase):
    __constants__ = ['stride', 'padding', 'dilation', 'groups', 'bias', 'padding_mode']

    def __init__(self, in_channels, out_channels, kernel_size, stride, padding, dilation, transposed,
                 output_padding, groups, bias, padding_mode, check_grad=False, rounding='deterministic',
                 weight_bits=5, act_integer_bits=16, act_fraction_bits=16):
        super(_ConvNdShiftQ, self).__init__()
        if in_channels % groups != 0:
            raise ValueError('in_channels must be divisible by groups')
        if out_channels % groups != 0:
            raise ValueError('out_channels must be divisible by groups')
        self.in_channels = in_channels
        self.out_channels = out_channels
        self.kernel_size = kernel_size
        self.stride = stride
        self.padding = padding
        self.dilation = dilation
        self.transposed = transposed
        self.output_padding = output_padding
        self.groups = groups
        self.padding_mode = padding_mode
        dtype = torch.float64 if check_grad else torch.float32
        if transposed:
            shape = (in_channels, out_channels // groups, *kernel_size)
        else:
            shape = (out_channels, in_channels // groups, *kernel_size)
        self.weight = nn.Parameter(torch.empty(*shape, dtype=dtype))
        if bias:
            self.bias = nn.Parameter(torch.empty(out_channels, dtype=dtype))
        else:
            self.register_parameter('bias', None)
        self.rounding = rounding
        self.shift_range = (-1 * (2 ** (weight_bits - 1) - 1), 0)  # modules_q.py:236
        self.act_integer_bits, self.act_fraction_bits = act_integer_bits, act_fraction_bits
        self.reset_parameters()

    def reset_parameters(self):
        init.kaiming_uniform_(self.weight, a=math.sqrt(5))
        if self.bias is not None:
            fan_in, _ = init._calculate_fan_in_and_fan_out(self.weight)
            bound = 1 / math.sqrt(fan_in)
            init.uniform_(self.bias, -bound, bound)

    def extra_repr(self):
        s = ('{in_channels}, {out_channels}, kernel_size={kernel_size}'
             ', stride={stride}')
        if self.padding != (0,) * len(self.padding):
            s += ', padding={padding}'
        if self.dilation != (1,) * len(self.dilation):
            s += ', dilation={dilation}'
        if self.groups != 1:
            s += ', groups={groups}'
        if self.bias is None:
            s += ', bias=False'
        return s.format(**self.__dict__)


class Conv2dShiftQ(_ConvNdShiftQ):
    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, groups=1,
                 bias=True, padding_mode='zeros', check_grad=False, use_kernel=False, use_cuda=True,
                 rounding='deterministic', weight_bits=5, act_integer_bits=16, act_fraction_bits=16):
        kernel_size = _pair(kernel_size)
        stride = _pair(stride)
        padding = _pair(padding)
        dilation = _pair(dilation)
        self.use_kernel = use_kernel
        self.use_cuda = use_cuda
        self.conc_weight = None
        super(Conv2dShiftQ, self).__init__(
            in_channels, out_channels, kernel_size, stride, padding, dilation, False, _pair(0), groups, bias,
            padding_mode, check_grad, rounding, weight_bits, act_integer_bits, act_fraction_bits)

    def forward(self, input, residual=None, relu=False):
        """``residual`` and ``relu`` are optional fusion hints (no counterpart in the reference, whose
        forward takes the input only): the result equals ``F.relu(self(input) + residual)`` (each part
        only when given) bit for bit.  With ``use_kernel=True`` a ReLU alone happens in the layer's
        epilogue; with a residual, addition and ReLU are one in-place pass over the output instead of
        two torch kernels."""
        padding = self.padding
        if self.padding_mode == 'circular':  # modules_q.py:291-296
            expanded_padding = ((self.padding[1] + 1) // 2, self.padding[1] // 2,
                                (self.padding[0] + 1) // 2, self.padding[0] // 2)
            input = F.pad(input, expanded_padding, mode='circular')
            padding = _pair(0)
        if self.use_kernel:
            self._check_kernel_mode()
            if self.dilation != (1, 1) or self.groups != 1:
                raise RuntimeError("the shift convolution kernel supports neither dilation nor groups")
            x = input.float().contiguous()
            in_kind, act_bits = _ffi.IN_F32_CONV, 0
            if utils.quantise_in_own_pass(self.kernel_size, self.out_channels):
                # every input value is staged once per filter tap and tile of 128 output channels:
                # from 9 uses on, quantise once, in a pass of its own
                x = self._input_codes(x)
                in_kind, act_bits = _ffi.IN_I32, self._act_bits()
            out = kernels.conv2d_fused(x, tuple(self.weight.shape), self._bias_fixed(), self._packed(x.device),
                                       self.stride, padding, in_kind=in_kind, out_kind=_ffi.OUT_F32,
                                       act_integer_bits=self.act_integer_bits,
                                       act_fraction_bits=self.act_fraction_bits, act_bits=act_bits,
                                       relu=relu and residual is None)
            if residual is not None:
                kernels.add_relu_f32_(out, residual.float().contiguous(), relu)
            return out
        weight_q = utils.round_power_of_2(self._clamped_weight(), self.rounding)
        input_fixed_point = utils.round_to_fixed(input, self.act_integer_bits, self.act_fraction_bits)
        bias_fixed_point = None
        if self.bias is not None:
            bias_fixed_point = utils.round_to_fixed(self.bias, self.act_integer_bits, self.act_fraction_bits)
        out = F.conv2d(input_fixed_point, weight_q, bias_fixed_point, self.stride, padding, self.dilation,
                       self.groups)
        if residual is not None:
            out = out + residual
        return F.relu(out) if relu else out
