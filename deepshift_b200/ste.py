"""Forward halves of the reference's straight-through helpers (pytorch/deepshift/ste.py).

Only inference is in scope, so these are the plain operations the reference applies in its
forward passes (ste.py:17-63); no custom backward is defined.
"""
import torch

from . import utils


def round_fixed_point(input, act_integer_bits=16, act_fraction_bits=16):
    """ste.py:17-27."""
    return utils.round_to_fixed(input, act_integer_bits, act_fraction_bits)


def round(input, rounding='deterministic'):
    """ste.py:29-39."""
    return utils.round(input, rounding)


def sign(input):
    """ste.py:41-51."""
    return torch.sign(input)


def clamp(input, min, max):
    """ste.py:53-63."""
    return torch.clamp(input, min, max)


def unsym_grad_mul(input_1, input_2):
    """ste.py:96-108 (forward: a product)."""
    return torch.mul(input_1, input_2)
