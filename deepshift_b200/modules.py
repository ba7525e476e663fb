"""DeepShift-PS modules with the reference's constructor signatures and attributes
(pytorch/deepshift/modules.py:78-142, 292-340), inference only.

With ``use_kernel=True`` the forward pass is ONE fused B200 kernel per layer: the fp32 input is
quantised to fixed point while it is staged, the shift-accumulate runs on the packed weights
``conc_weight`` and the int32 result is converted back to fp32 in the epilogue -- bit-identical
to the reference's quantise -> ``deepshift.kernels`` -> ``out.float() / 2**F`` sequence
(modules.py:23-31, 150-162, 312-340).  ``use_cuda=False`` raises: there is no CPU kernel path.
With ``use_kernel=False`` the forward pass is the reference's plain PyTorch expression
(modules.py:135, 339-340) without the straight-through estimators, which only matter to
training.
"""
import math

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.nn import init
from torch.nn.modules.utils import _pair

from . import _ffi, kernels, ste, utils


def _kernel_mode_check(module):
    if not module.use_cuda:
        raise RuntimeError("deepshift_b200 has no CPU kernel path: use_kernel=True needs use_cuda=True")


class _ShiftBase(nn.Module):
    """State shared by both layers: cached fixed-point bias and lazily packed weights."""

    def _bias_fixed(self, like_conv):
        # Conv2dShift rounds the bias with round_to_fixed first (modules.py:318-321,154-157);
        # LinearShift only truncates bias * 2^F (modules.py:26-27).
        if self.bias is None:
            return None
        key = (self.bias.data_ptr(), self.bias._version, self.bias.device)
        if getattr(self, "_bias_key", None) != key:
            b = self.bias.detach().float()
            if like_conv:
                b = utils.round_to_fixed(b, self.act_integer_bits, self.act_fraction_bits)
            self._bias_i32 = (b * (2 ** self.act_fraction_bits)).int().contiguous()
            self._bias_key = key
        return self._bias_i32

    # ``conc_weight`` as the reference names it (modules.py:86,306).  Assigning it (convert_to_shift
    # does, convert.py:39-40,75-76) hands over packed weights that match the parameters of that
    # moment; the version key is taken at the next forward pass.
    @property
    def conc_weight(self):
        return self.__dict__.get("_conc_weight")

    @conc_weight.setter
    def conc_weight(self, value):
        self.__dict__["_conc_weight"] = value
        self.__dict__["_weight_key"] = None

    def _packed(self, device):
        """Packed weights that match the current ``shift`` / ``sign``: packed on first use when the
        module was built by hand, and again whenever either parameter was replaced or changed in
        place (``load_state_dict``, an optimiser step) since they were packed.  An in-place edit
        through ``.data`` does not move the version counter: set ``conc_weight = None`` after one."""
        key = (self.shift.data_ptr(), self.shift._version, self.sign.data_ptr(), self.sign._version)
        cw, have = self.conc_weight, self.__dict__.get("_weight_key")
        if cw is None or (have is not None and have != key):
            self.conc_weight = utils.compress_bits(self.shift.data.round(), self.sign.data.round().sign(),
                                                   device=device)
            cw = self.conc_weight
        elif cw.data.device != device:
            cw.data = cw.data.to(device)
            cw.__dict__.pop("_prepared", None)   # expanded copies live on the old device
        self.__dict__["_weight_key"] = key
        return cw

    def _float_weight(self):
        shift_rounded = ste.round(self.shift, rounding=self.rounding)
        sign_rounded_signed = ste.sign(ste.round(self.sign, rounding=self.rounding))
        return ste.unsym_grad_mul(2 ** shift_rounded, sign_rounded_signed)


class LinearShift(_ShiftBase):
    def __init__(self, in_features, out_features, bias=True, check_grad=False, freeze_sign=False,
                 use_kernel=False, use_cuda=True, rounding='deterministic', weight_bits=5,
                 act_integer_bits=16, act_fraction_bits=16):
        super(LinearShift, self).__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.use_kernel = use_kernel
        self.check_grad = check_grad
        self.use_cuda = use_cuda
        self.conc_weight = None
        self.rounding = rounding
        self.shift_range = (-1 * (2 ** (weight_bits - 1) - 2), 0)  # modules.py:88
        self.act_integer_bits, self.act_fraction_bits = act_integer_bits, act_fraction_bits
        dtype = torch.float64 if check_grad else torch.float32
        self.shift = nn.Parameter(torch.empty(out_features, in_features, dtype=dtype))
        self.sign = nn.Parameter(torch.empty(out_features, in_features, dtype=dtype),
                                 requires_grad=(freeze_sign == False))
        if bias:
            self.bias = nn.Parameter(torch.empty(out_features, dtype=dtype))
        else:
            self.register_parameter('bias', None)
        self.reset_parameters()

    def reset_parameters(self):
        self.shift.data.uniform_(*self.shift_range)
        self.sign.data.uniform_(-1, 1)
        if self.bias is not None:
            fan_in, _ = init._calculate_fan_in_and_fan_out(self.shift)
            bound = 1 / math.sqrt(fan_in)
            init.uniform_(self.bias, -bound, bound)

    def forward(self, input, residual=None, relu=False):
        """``residual`` and ``relu`` are optional fusion hints (no counterpart in the reference, whose
        forward takes the input only): the result equals ``F.relu(self(input) + residual)`` (each part
        only when given) bit for bit.  With ``use_kernel=True`` a ReLU alone happens in the layer's
        epilogue; with a residual, addition and ReLU are one in-place pass over the output instead of
        two torch kernels."""
        if self.use_kernel:
            _kernel_mode_check(self)
            x = input.reshape(-1, self.in_features).float().contiguous()
            out = kernels.linear_fused(x, self.out_features, self._bias_fixed(like_conv=False),
                                       self._packed(x.device), in_kind=_ffi.IN_F32_LINEAR,
                                       out_kind=_ffi.OUT_F32, act_integer_bits=self.act_integer_bits,
                                       act_fraction_bits=self.act_fraction_bits,
                                       relu=relu and residual is None)
            if residual is not None:
                kernels.add_relu_f32_(out, residual.reshape(-1, self.out_features).float().contiguous(), relu)
            return out.reshape(*input.shape[:-1], self.out_features)
        self.shift.data = ste.clamp(self.shift.data, *self.shift_range)
        out = F.linear(input, self._float_weight(), self.bias)
        if residual is not None:
            out = out + residual
        return F.relu(out) if relu else out

    def extra_repr(self):
        return 'in_features={}, out_features={}, bias={}'.format(
            self.in_features, self.out_features, self.bias is not None)


class _ConvNdShift(_ShiftBase):
    __constants__ = ['stride', 'padding', 'dilation', 'groups', 'bias', 'padding_mode']

    def __init__(self, in_channels, out_channels, kernel_size, stride, padding, dilation, transposed,
                 output_padding, groups, bias, padding_mode, check_grad=False, freeze_sign=False,
                 rounding='deterministic', weight_bits=5, act_integer_bits=16, act_fraction_bits=16):
        super(_ConvNdShift, self).__init__()
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
        self.rounding = rounding
        self.shift_range = (-1 * (2 ** (weight_bits - 1) - 2), 0)  # modules.py:242
        self.act_integer_bits, self.act_fraction_bits = act_integer_bits, act_fraction_bits
        dtype = torch.float64 if check_grad else torch.float32
        if transposed:
            shape = (in_channels, out_channels // groups, *kernel_size)
        else:
            shape = (out_channels, in_channels // groups, *kernel_size)
        self.shift = nn.Parameter(torch.empty(*shape, dtype=dtype))
        self.sign = nn.Parameter(torch.empty(*shape, dtype=dtype), requires_grad=(freeze_sign == False))
        if bias:
            self.bias = nn.Parameter(torch.empty(out_channels, dtype=dtype))
        else:
            self.register_parameter('bias', None)
        self.reset_parameters()

    def reset_parameters(self):
        self.shift.data.uniform_(-10, -1)
        self.sign.data.uniform_(-1, 1)
        if self.bias is not None:
            fan_in, _ = init._calculate_fan_in_and_fan_out(self.shift)
            bound = 1 / math.sqrt(fan_in)
            init.uniform_(self.bias, -bound, bound)

    def extra_repr(self):
        s = ('{in_channels}, {out_channels}, kernel_size={kernel_size}, stride={stride}')
        if self.padding != (0,) * len(self.padding):
            s += ', padding={padding}'
        if self.dilation != (1,) * len(self.dilation):
            s += ', dilation={dilation}'
        if self.groups != 1:
            s += ', groups={groups}'
        if self.bias is None:
            s += ', bias=False'
        return s.format(**self.__dict__)


class Conv2dShift(_ConvNdShift):
    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, groups=1,
                 bias=True, padding_mode='zeros', check_grad=False, freeze_sign=False, use_kernel=False,
                 use_cuda=True, rounding='determinstic', weight_bits=5, act_integer_bits=16,
                 act_fraction_bits=16):
        # 'determinstic' is the reference's own default spelling (modules.py:296); utils.round
        # accepts it.
        kernel_size = _pair(kernel_size)
        stride = _pair(stride)
        padding = _pair(padding)
        dilation = _pair(dilation)
        self.use_kernel = use_kernel
        self.use_cuda = use_cuda
        self.conc_weight = None
        super(Conv2dShift, self).__init__(
            in_channels, out_channels, kernel_size, stride, padding, dilation, False, _pair(0), groups,
            bias, padding_mode, check_grad, freeze_sign, rounding, weight_bits, act_integer_bits,
            act_fraction_bits)

    def forward(self, input, residual=None, relu=False):
        """``residual`` and ``relu`` are optional fusion hints (no counterpart in the reference, whose
        forward takes the input only): the result equals ``F.relu(self(input) + residual)`` (each part
        only when given) bit for bit.  With ``use_kernel=True`` a ReLU alone happens in the layer's
        epilogue; with a residual, addition and ReLU are one in-place pass over the output instead of
        two torch kernels."""
        if self.padding_mode == 'circular':
            # modules.py:323-331; padding fp32 before the quantiser equals padding after it.
            expanded_padding = ((self.padding[1] + 1) // 2, self.padding[1] // 2,
                                (self.padding[0] + 1) // 2, self.padding[0] // 2)
            input = F.pad(input, expanded_padding, mode='circular')
            padding = _pair(0)
        else:
            padding = self.padding
        if self.use_kernel:
            _kernel_mode_check(self)
            if self.dilation != (1, 1) or self.groups != 1:
                raise RuntimeError("the shift convolution kernel supports neither dilation nor groups")
            x = input.float().contiguous()
            in_kind, act_bits = _ffi.IN_F32_CONV, 0
            if utils.quantise_in_own_pass(self.kernel_size, self.out_channels):
                # the kernel stages every input value once per filter tap and per tile of 128 output
                # channels: from 9 such uses on, quantising once in a pass of its own is cheaper than
                # quantising at every use; the codes are final (round_to_fixed is not idempotent for
                # one integer bit), so the kernel gets them as plain int32 with their bound
                x = kernels.quantize(x, self.act_integer_bits, self.act_fraction_bits, like_conv=True)
                in_kind, act_bits = _ffi.IN_I32, utils.code_bits(self.act_integer_bits, self.act_fraction_bits)
            out = kernels.conv2d_fused(x, tuple(self.shift.shape), self._bias_fixed(like_conv=True),
                                       self._packed(x.device), self.stride, padding,
                                       in_kind=in_kind, out_kind=_ffi.OUT_F32,
                                       act_integer_bits=self.act_integer_bits,
                                       act_fraction_bits=self.act_fraction_bits, act_bits=act_bits,
                                       relu=relu and residual is None)
            if residual is not None:
                kernels.add_relu_f32_(out, residual.float().contiguous(), relu)
            return out
        self.shift.data = ste.clamp(self.shift.data, *self.shift_range)
        input_fixed_point = ste.round_fixed_point(input, self.act_integer_bits, self.act_fraction_bits)
        bias_fixed_point = None
        if self.bias is not None:
            bias_fixed_point = ste.round_fixed_point(self.bias, self.act_integer_bits, self.act_fraction_bits)
        out = F.conv2d(input_fixed_point, self._float_weight(), bias_fixed_point, self.stride, padding,
                       self.dilation, self.groups)
        if residual is not None:
            out = out + residual
        return F.relu(out) if relu else out
