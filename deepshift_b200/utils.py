"""Fixed-point and packing helpers with the reference's names (pytorch/deepshift/utils.py)."""
import math

import numpy as np
import torch

from . import kernels


def round_to_fixed(input, integer_bits=16, fraction_bits=16):
    """utils.py:7-21: floor to the 2^-F grid, clamp to [-2^(I-1), 2^(I-1) - 1]."""
    assert integer_bits >= 1, integer_bits
    if integer_bits == 1:
        return torch.sign(input) - 1
    delta = math.pow(2.0, -(fraction_bits))
    bound = math.pow(2.0, integer_bits - 1)
    rounded = torch.floor(input / delta) * delta
    return torch.clamp(rounded, -bound, bound - 1)


def quantise_in_own_pass(kernel_size, out_channels):
    """Whether a shift convolution with fp32 input should quantise it in a separate pass: the
    convolution kernel converts a value every time it stages it, once per filter tap and per tile
    of 128 output channels; a pass of its own costs one read and one write of the tensor."""
    uses = kernel_size[0] * kernel_size[1] * ((out_channels + 127) // 128)
    return uses >= 9


def code_bits(integer_bits, fraction_bits):
    """Bits b such that every int32 code of round_to_fixed(., I, F) * 2^F lies in
    [-2^(b-1), 2^(b-1)]: I + F, or F + 2 for one integer bit (codes -2^(F+1), -2^F, 0)."""
    return fraction_bits + 2 if integer_bits == 1 else integer_bits + fraction_bits


def round(x, rounding='deterministic'):
    """utils.py:36-42.  The misspelling 'determinstic' (Conv2dShift's default,
    modules.py:296) is accepted as 'deterministic'."""
    if rounding == 'determinstic':
        rounding = 'deterministic'
    assert rounding in ['deterministic', 'stochastic']
    if rounding == 'stochastic':
        x_floor = x.floor()
        return x_floor + torch.bernoulli(x - x_floor)
    return x.round()


def get_shift_and_sign(x, rounding='deterministic'):
    """utils.py:23-29: sign = sign(x), shift = round(log2|x|)."""
    sign = torch.sign(x)
    x_abs = torch.abs(x)
    shift = round(torch.log(x_abs) / np.log(2), rounding)
    return shift, sign


def round_power_of_2(x, rounding='deterministic'):
    shift, sign = get_shift_and_sign(x, rounding)
    return (2.0 ** shift) * sign


def clampabs(input, min, max):
    """utils.py:44-52: |x| clamped into [min, max] in place, zeros left alone."""
    assert min >= 0 and max >= 0
    input[input > max] = max
    input[input < -max] = -max
    input[(input > 0) & (input < min)] = min
    input[(input < 0) & (input > -min)] = -min
    return input


class ConcWeight():
    """utils.py:54-58: packed weights, the (non-positive) shift base and the field width."""

    def __init__(self, data=None, base=0, bits=8):
        self.data = data
        self.base = base
        self.bits = bits


def compress_bits(shift, sign, device=None):
    """utils.py:61-88: packs a layer's (shift, sign) parameters into a ``ConcWeight``.

    Differences from the reference, which mutates its arguments and mis-indexes
    (utils.py:64-70 assigns through ``nonzero()`` coordinates and overwrites whole rows):
    zero-sign weights become (sign +1, shift -32) by boolean mask on copies, and
    ``shift``/``sign`` are left untouched.  With a positive shift present (base < 0) the stored
    field is ``-shift - base`` exactly once, so field + base is the true right shift.
    """
    conc_weight = ConcWeight()
    shift = shift.detach().clone()
    sign = sign.detach().clone()
    if len(shift.shape) == 2:
        shift = shift.unsqueeze(-1).unsqueeze(-1)
        sign = sign.unsqueeze(-1).unsqueeze(-1)

    zero = sign == 0
    shift[zero] = -32
    sign[zero] = +1

    shift = (shift * -1).round().to(torch.int64)          # right shift as the default
    minimum, maximum = int(shift.min()), int(shift.max())
    conc_weight.base = minimum if minimum < 0 else 0
    # ceil(log2(max + 1)) of utils.py:72 in exact integer arithmetic, on the stored field
    conc_weight.bits = max(1, (maximum - conc_weight.base).bit_length())

    num = int(32 / (conc_weight.bits + 1))
    row_length = int((shift.shape[1] * shift.shape[2] * shift.shape[3] + num - 1) / num)
    size = row_length * shift.shape[0]
    if device is None:
        device = shift.device if shift.is_cuda else torch.device('cuda', torch.cuda.current_device())
    conc_weight.data = kernels.compress_sign_and_shift(
        shift.int().to(device).contiguous(), sign.int().to(device).contiguous(), size,
        conc_weight.base, conc_weight.bits, row_length, num)
    return conc_weight
