"""Run by test_gpu_memory_safety.py in a process of its own with DEEPSHIFT_B200_CHECKED=1: a spread of
linear and convolution shapes on the bounds-checking flavour of the library.  Every result must equal
the oracle's and the status word must stay 0; then the activations are declared 64 bytes shorter than
they are and the checks must report loads beyond that end (kind 1) -- while every access still lies
inside the real buffer."""
import ctypes
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, HERE)

from helpers import acts_q16, acts_wide, weights  # noqa: E402


def status(lib):
    st, ck = ctypes.c_int(-1), ctypes.c_int(-1)
    assert lib.ds_bounds_status(ctypes.byref(st), ctypes.byref(ck)) == 0
    return st.value, ck.value


def main():
    from deepshift_b200 import _ffi, kernels, utils
    from oracle import oracle as O
    O.build()
    lib = _ffi.lib()
    dev = torch.device("cuda:0")
    assert status(lib) == (0, 1), "not the checked flavour"
    rng = np.random.default_rng(77)

    def cw_of(shift, sign):
        return utils.compress_bits(torch.from_numpy(shift).float(), torch.from_numpy(sign).float(), device=dev)

    convs = [(3, 16, 28, 28, 40, 3, 1, 1), (3, 24, 14, 14, 70, 3, 1, 1), (2, 3, 32, 32, 64, 7, 2, 3), (4, 20, 7, 9, 70, 3, 1, 1),
             (3, 12, 10, 10, 33, 1, 2, 0), (2, 5, 9, 9, 12, 2, 1, 0), (5, 128, 7, 7, 130, 3, 1, 1), (49, 32, 28, 28, 100, 3, 1, 1)]
    for (B, C, H, W, OC, k, s, p) in convs:
        shift, sign = weights(rng, (OC, C, k, k))
        bias = rng.integers(-2000, 2000, OC).astype(np.int32)
        cw = cw_of(shift, sign)
        for x, ab in ((acts_q16(rng, (B, C, H, W)), 16), (acts_q16(rng, (B, C, H, W)), None), (acts_wide(rng, (B, C, H, W), 24), 0)):
            out = kernels.conv2d(torch.from_numpy(x).to(dev), torch.from_numpy(shift).to(dev), None,
                                 torch.from_numpy(bias).to(dev), cw, s, p, act_bits=ab)
            assert np.array_equal(out.cpu().numpy(), O.conv2d(x, shift, sign, bias, (s, s), (p, p))), (B, C, H, W, OC, k, ab)
    for (M, K, N) in [(1, 4096, 33), (5, 1031, 300), (16, 96, 4100), (40, 3000, 70), (300, 512, 200), (2304, 260, 130)]:
        shift, sign = weights(rng, (N, K))
        cw = cw_of(shift, sign)
        for ab in (16, 0):
            x = acts_q16(rng, (M, K))
            out = kernels.linear(torch.from_numpy(x).to(dev), torch.from_numpy(shift).to(dev), None, None, cw, act_bits=ab)
            assert np.array_equal(out.cpu().numpy(), O.linear(x, shift, sign, None)), (M, K, N, ab)
    assert status(lib) == (0, 1), "an access left its extent"
    # the checks fire: x declared 64 bytes short, nothing leaves the real buffer
    B, C, H, OC = 2, 8, 12, 20
    shift, sign = weights(rng, (OC, C, 3, 3))
    x = acts_q16(rng, (B, C, H, H))
    assert lib.ds_bounds_debug_shrink_x(64) == 0
    kernels.conv2d(torch.from_numpy(x).to(dev), torch.from_numpy(shift).to(dev), None, None, cw_of(shift, sign), 1, 1, act_bits=16)
    assert status(lib) == (1, 1), "loads beyond the declared end went unnoticed"
    assert lib.ds_bounds_debug_shrink_x(0) == 0
    out = kernels.conv2d(torch.from_numpy(x).to(dev), torch.from_numpy(shift).to(dev), None, None, cw_of(shift, sign), 1, 1, act_bits=16)
    assert np.array_equal(out.cpu().numpy(), O.conv2d(x, shift, sign, None, (1, 1), (1, 1)))
    assert status(lib) == (0, 1)
    print("checked build: ok")


if __name__ == "__main__":
    main()
