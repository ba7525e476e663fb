"""Standalone shift-GEMM / shift-convolution timing (BASELINE.json configs[4]).

    python -m deepshift_b200.sweep                      # the whole sweep, one JSON line per case
    python -m deepshift_b200.sweep conv B C H OC K S P  # one 2-D convolution (square image/window)
    python -m deepshift_b200.sweep gemm M K N           # one linear layer
    options: --bits b (weight bits 2..5, default 5)  --dense (no zero signs: 32//b weights per word)
             --act-bits n (0 = exact integer path, 16 = FP32-pipe path, default 16)  --iters n

Weights: shift uniform in [-(2^(b-1)-1), 0], sign -1/0/+1 with P = 0.45/0.10/0.45 (ternary; the
zero-weight encoding then needs the 6-bit field, 4 weights per word) or -1/+1 (--dense).
Activations: int32 codes of round_to_fixed(N(0,1), 4, 12).  Times are CUDA-event averages after
3 warm-up launches; 1 shift-op = one (activation, weight) pair = 2 integer ops.
"""
import argparse
import json

import numpy as np
import torch

from . import kernels, utils


def _weights(rng, shape, bits, dense):
    lo = -(2 ** (bits - 1) - 1)
    shift = rng.integers(lo, 1, shape).astype(np.float32)
    if dense:
        sign = rng.choice([-1.0, 1.0], shape).astype(np.float32)
    else:
        sign = rng.choice([-1.0, 0.0, 1.0], shape, p=[0.45, 0.10, 0.45]).astype(np.float32)
    return torch.from_numpy(shift), torch.from_numpy(sign)


def _acts(rng, shape):
    v = np.clip(np.floor(rng.normal(0, 1, shape) * 4096), -32768, 28672).astype(np.int32)
    return torch.from_numpy(v)


def _time(fn, iters):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def run_gemm(M, K, N, bits=5, dense=False, act_bits=16, iters=10, dev="cuda"):
    rng = np.random.default_rng(20254)
    x = _acts(rng, (M, K)).to(dev)
    shift, sign = _weights(rng, (N, K), bits, dense)
    cw = utils.compress_bits(shift, sign, device=torch.device(dev))
    shift_d = shift.to(dev)
    ms = _time(lambda: kernels.linear(x, shift_d, None, None, cw, act_bits=act_bits), iters)
    ops = M * K * N
    num = 32 // (cw.bits + 1)
    nbytes = 4 * (M * K + N * ((K + num - 1) // num) + M * N)
    return dict(case="gemm", M=M, K=K, N=N, weight_bits=bits, dense=dense, field_bits=cw.bits, act_bits=act_bits,
                ms=ms, Tshift_ops_per_s=ops / ms / 1e9, Gops_per_s=2 * ops / ms / 1e6, GBps=nbytes / ms / 1e6)


def run_conv(B, C, H, OC, k, stride, pad, bits=5, dense=False, act_bits=16, iters=10, dev="cuda"):
    rng = np.random.default_rng(20254)
    x = _acts(rng, (B, C, H, H)).to(dev)
    shift, sign = _weights(rng, (OC, C, k, k), bits, dense)
    cw = utils.compress_bits(shift, sign, device=torch.device(dev))
    shift_d = shift.to(dev)
    ms = _time(lambda: kernels.conv2d(x, shift_d, None, None, cw, (stride, stride), (pad, pad), act_bits=act_bits),
               iters)
    OH = (H + 2 * pad - k) // stride + 1
    ops = B * OC * OH * OH * C * k * k
    num = 32 // (cw.bits + 1)
    nbytes = 4 * (B * C * H * H + OC * ((C * k * k + num - 1) // num) + B * OC * OH * OH)
    return dict(case="conv", B=B, C=C, H=H, OC=OC, k=k, stride=stride, pad=pad, weight_bits=bits, dense=dense,
                field_bits=cw.bits, act_bits=act_bits, ms=ms, Tshift_ops_per_s=ops / ms / 1e9,
                Gops_per_s=2 * ops / ms / 1e6, GBps=nbytes / ms / 1e6)


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("case", nargs="?", choices=["gemm", "conv"])
    ap.add_argument("dims", nargs="*", type=int)
    ap.add_argument("--bits", type=int, default=5)
    ap.add_argument("--dense", action="store_true")
    ap.add_argument("--act-bits", type=int, default=16)
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    kw = dict(bits=a.bits, dense=a.dense, act_bits=a.act_bits, iters=a.iters)
    if a.case == "gemm":
        print(json.dumps(run_gemm(*a.dims, **kw)))
    elif a.case == "conv":
        print(json.dumps(run_conv(*a.dims, **kw)))
    else:
        for dense in (False, True):
            for bits in (2, 3, 4, 5):
                for KN in (512, 1024, 2048, 4096):
                    for M in (1, 64, 1024, 8192):
                        print(json.dumps(run_gemm(M, KN, KN, bits=bits, dense=dense, act_bits=a.act_bits,
                                                  iters=a.iters)), flush=True)
        for dense in (False, True):
            for (C, H) in ((64, 56), (128, 28), (256, 14), (512, 7)):
                print(json.dumps(run_conv(256, C, H, C, 3, 1, 1, bits=5, dense=dense, act_bits=a.act_bits,
                                          iters=a.iters)), flush=True)


if __name__ == "__main__":
    main()
