"""The reference's ``unoptimized`` package (pytorch/unoptimized/): fp32 layers on a deliberately
plain CUDA kernel, the strawman its README times the shift kernels against.

``UnoptimizedLinear`` / ``UnoptimizedConv2d`` keep the constructors of unoptimized/modules/linear.py
and conv.py; ``convert_to_unoptimized`` is unoptimized/convert.py:8-30.  Unlike the reference's
kernels.py:9-36 the outputs live on the input's device (not always cuda:0) and the convolution pads
implicitly.  Results agree with ``torch.nn.functional`` to fp32 rounding.
"""
import math

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.nn import init
from torch.nn.modules.utils import _pair

from . import _ffi, kernels


def linear(input, weight, bias):
    kernels._check_tensor(input, "input", torch.float32)
    kernels._check_tensor(weight, "weight", torch.float32)
    out = torch.empty([input.size(0), weight.size(0)], dtype=torch.float32, device=input.device)
    with torch.cuda.device(input.device):
        rc = _ffi.lib().ds_unopt_linear_f32(input.data_ptr(), weight.data_ptr(),
                                            bias.data_ptr() if bias is not None else None, out.data_ptr(),
                                            input.size(0), input.size(1), weight.size(0), kernels._stream_ptr(input.device))
    _ffi.check(rc, "unoptimized.linear")
    return out


def conv2d(input, weight, bias, stride, padding):
    kernels._check_tensor(input, "input", torch.float32)
    kernels._check_tensor(weight, "weight", torch.float32)
    sh, sw = _pair(stride) if not isinstance(stride, int) else (stride, stride)
    ph, pw = _pair(padding) if not isinstance(padding, int) else (padding, padding)
    B, C, H, W = input.shape
    OC, C2, KH, KW = weight.shape
    if C2 != C:
        raise RuntimeError("input has %d channels, weight expects %d" % (C, C2))
    out = torch.empty([B, OC, (H + 2 * ph - KH) // sh + 1, (W + 2 * pw - KW) // sw + 1], dtype=torch.float32,
                      device=input.device)
    with torch.cuda.device(input.device):
        rc = _ffi.lib().ds_unopt_conv2d_f32(input.data_ptr(), weight.data_ptr(),
                                            bias.data_ptr() if bias is not None else None, out.data_ptr(),
                                            B, C, H, W, OC, KH, KW, sh, sw, ph, pw, kernels._stream_ptr(input.device))
    _ffi.check(rc, "unoptimized.conv2d")
    return out


class UnoptimizedLinear(nn.Module):
    def __init__(self, in_features, out_features, bias=True):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features))
        if bias:
            self.bias = nn.Parameter(torch.empty(out_features))
        else:
            self.register_parameter('bias', None)
        init.kaiming_uniform_(self.weight, a=math.sqrt(5))
        if self.bias is not None:
            bound = 1 / math.sqrt(in_features)
            init.uniform_(self.bias, -bound, bound)

    def forward(self, input):
        x = input.reshape(-1, self.in_features).float().contiguous()
        return linear(x, self.weight.contiguous(), self.bias).reshape(*input.shape[:-1], self.out_features)

    def extra_repr(self):
        return 'in_features={}, out_features={}, bias={}'.format(self.in_features, self.out_features, self.bias is not None)


class UnoptimizedConv2d(nn.Module):
    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, groups=1, bias=True,
                 padding_mode='zeros'):
        super().__init__()
        if _pair(dilation) != (1, 1) or groups != 1:
            raise ValueError("the unoptimized kernel supports neither dilation nor groups")
        self.in_channels, self.out_channels = in_channels, out_channels
        self.kernel_size, self.stride, self.padding = _pair(kernel_size), _pair(stride), _pair(padding)
        self.dilation, self.groups, self.padding_mode = _pair(dilation), groups, padding_mode
        self.weight = nn.Parameter(torch.empty(out_channels, in_channels, *self.kernel_size))
        if bias:
            self.bias = nn.Parameter(torch.empty(out_channels))
        else:
            self.register_parameter('bias', None)
        init.kaiming_uniform_(self.weight, a=math.sqrt(5))
        if self.bias is not None:
            fan_in, _ = init._calculate_fan_in_and_fan_out(self.weight)
            init.uniform_(self.bias, -1 / math.sqrt(fan_in), 1 / math.sqrt(fan_in))

    def forward(self, input):
        padding = self.padding
        if self.padding_mode == 'circular':
            input = F.pad(input, ((self.padding[1] + 1) // 2, self.padding[1] // 2, (self.padding[0] + 1) // 2,
                                  self.padding[0] // 2), mode='circular')
            padding = (0, 0)
        return conv2d(input.float().contiguous(), self.weight.contiguous(), self.bias, self.stride, padding)


def convert_to_unoptimized(model):
    """Replaces every nn.Linear / nn.Conv2d by its unoptimized twin, sharing the parameters."""
    for name, module in model._modules.items():
        if len(list(module.children())) > 0:
            model._modules[name] = convert_to_unoptimized(module)
        if type(module) == nn.Linear:
            m = UnoptimizedLinear(module.in_features, module.out_features, module.bias is not None)
            m.weight, m.bias = module.weight, module.bias
            model._modules[name] = m
        if type(module) == nn.Conv2d:
            m = UnoptimizedConv2d(module.in_channels, module.out_channels, module.kernel_size, module.stride,
                                  module.padding, module.dilation, module.groups, module.bias is not None,
                                  module.padding_mode)
            m.weight, m.bias = module.weight, module.bias
            model._modules[name] = m
    return model
