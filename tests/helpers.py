"""Seeded generators shared by the tests."""
import numpy as np


def weights(rng, shape, lo=-15, zeros=True):
    shift = rng.integers(lo, 1, shape).astype(np.int32)
    p = [0.45, 0.10, 0.45] if zeros else [0.5, 0.0, 0.5]
    sign = rng.choice([-1, 0, 1], shape, p=p).astype(np.int32)
    return shift, sign


def acts_q16(rng, shape):
    """int32 codes that round_to_fixed(., 4, 12) * 4096 can produce."""
    v = np.floor(rng.normal(0, 1, shape) * 4096)
    return np.clip(v, -32768, 28672).astype(np.int32)


def acts_wide(rng, shape, bits=27):
    return rng.integers(-(1 << bits), 1 << bits, shape).astype(np.int32)


def np_weights(ws):
    return [dict(shift=w['shift'].numpy(), sign=w['sign'].numpy(), bias=w['bias'].numpy()) for w in ws]
