"""Regenerates tests/golden/*.npz by RUNNING THE REFERENCE (never by hand).

Two sources, both executed in a container where the reference checkout is mounted:

* the reference's compiled CPU kernel ``deepshift_cpu`` (oracle/_ref, built unmodified by
  oracle/build_ref.py from pytorch/deepshift/kernels/cpu/shift_cpu.cpp) for the integer
  kernels ``linear_kernel`` and ``convolution_kernel``;
* the reference's Python package imported from the checkout (``deepshift.utils``,
  ``deepshift.modules``) for the float glue: ``round_to_fixed``, ``get_shift_and_sign`` and
  the ``use_kernel=True, use_cuda=False`` forward of ``LinearShift`` / ``Conv2dShift``.

Inputs are seeded; each file stores inputs and the reference's outputs.

Usage: python tests/golden/make_golden.py [--only-q | --only-sign | --only-gap] path-to-reference-checkout
(--only-q: write q_ref.npz, the DeepShift-Q module vectors, and leave the other files alone;
 --only-sign: write sign_ref.npz, modules with one integer bit; --only-gap: write gap_ref.npz, the
 average-pool glue, which needs torch only).  The checkout path may also come from the environment
variable DEEPSHIFT_REFERENCE.
"""
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import build_ref, oracle as O  # noqa: E402


def weights(rng, shape, lo=-15, zeros=True):
    shift = rng.integers(lo, 1, shape).astype(np.int32)
    p = [0.45, 0.10, 0.45] if zeros else [0.5, 0.0, 0.5]
    sign = rng.choice([-1, 0, 1], shape, p=p).astype(np.int32)
    return shift, sign


def acts(rng, shape, kind="q16"):
    if kind == "q16":   # what round_to_fixed(., 4, 12) * 4096 can produce
        v = np.floor(rng.normal(0, 1, shape) * 4096)
        return np.clip(v, -32768, 28672).astype(np.int32)
    if kind == "wide":  # unclamped linear inputs
        return rng.integers(-(1 << 27), 1 << 27, shape).astype(np.int32)
    raise ValueError(kind)


def _import_reference(reference_root):
    sys.path.insert(0, os.path.join(reference_root, "pytorch"))
    # kernels.py:4-8 binds deepshift_cpu only if deepshift_cuda imports first.
    sys.modules.setdefault("deepshift_cuda", types.ModuleType("deepshift_cuda"))
    sys.modules["deepshift_cpu"] = O.ref_module()


def main_q(reference_root):
    """q_ref.npz: the reference's Conv2dShiftQ forward with use_kernel=True, use_cuda=False
    (modules_q.py:283-300 -> 141-161 -> kernels.py:54-66 -> deepshift_cpu.convolution_kernel).
    padding = 0, because kernels.conv2d pads only W on the CPU path (kernels.py:58), and no zero
    weights, because convolution_kernel adds them as +1 (shift_cpu.cpp:351-353)."""
    assert build_ref.build(reference_root) is not None, "reference checkout not found"
    _import_reference(reference_root)
    import deepshift.modules_q as ref_q
    out = {}
    rng = np.random.default_rng(4000)
    for i, (cin, cout, k, stride, hw, scale) in enumerate([(3, 6, 3, 1, 8, 1.0), (4, 5, 5, 2, 11, 40.0),
                                                           (2, 7, 1, 1, 6, 1e-4)]):
        torch.manual_seed(40 + i)
        conv = ref_q.Conv2dShiftQ(cin, cout, k, stride=stride, padding=0, bias=True, use_kernel=True,
                                  use_cuda=False, act_integer_bits=4, act_fraction_bits=12)
        conv.weight.data.mul_(scale)   # beyond 1 and below 2^-15: the module's clamp acts
        xin = torch.from_numpy(rng.normal(0, 3, (2, cin, hw, hw)).astype(np.float32))
        out[f"w{i}"], out[f"bias{i}"] = conv.weight.data.numpy().copy(), conv.bias.data.numpy().copy()
        out[f"x{i}"], out[f"stride{i}"] = xin.numpy().copy(), np.int32(stride)
        with torch.no_grad():
            out[f"y{i}"] = conv(xin.clone()).numpy()
    out["n"] = np.int32(3)
    np.savez_compressed(os.path.join(HERE, "q_ref.npz"), **out)
    print("q_ref.npz", os.path.getsize(os.path.join(HERE, "q_ref.npz")), "bytes")


def main_sign(reference_root):
    """sign_ref.npz: forward passes of the reference's Conv2dShift and Conv2dShiftQ with
    act_integer_bits = 1, where round_to_fixed is sign(x) - 1 (utils.py:12-13), on windows of 25 and
    49 taps, use_kernel=True on the reference's CPU kernel.  padding = 0 and no zero weights for the
    reasons given at main_q."""
    assert build_ref.build(reference_root) is not None, "reference checkout not found"
    _import_reference(reference_root)
    import deepshift.modules as ref_modules
    import deepshift.modules_q as ref_q
    out = {}
    rng = np.random.default_rng(5000)
    cases = [("ps", 3, 6, 5, 1, 12, 7), ("ps", 2, 5, 7, 2, 17, 12), ("q", 3, 4, 5, 1, 11, 7), ("q", 2, 6, 7, 2, 16, 10)]
    for i, (kind, cin, cout, k, stride, hw, F) in enumerate(cases):
        torch.manual_seed(50 + i)
        xin = rng.normal(0, 1, (2, cin, hw, hw)).astype(np.float32)
        xin[rng.random(xin.shape) < 0.15] = 0.0      # exact zeros: the middle code -2^F
        xin = torch.from_numpy(xin)
        if kind == "ps":
            conv = ref_modules.Conv2dShift(cin, cout, k, stride=stride, padding=0, bias=True, use_kernel=True,
                                           use_cuda=False, rounding="deterministic", act_integer_bits=1,
                                           act_fraction_bits=F)
            conv.shift.data = torch.from_numpy(rng.integers(-14, 1, (cout, cin, k, k)).astype(np.float32))
            conv.sign.data = torch.from_numpy(rng.choice([-1.0, 1.0], (cout, cin, k, k)).astype(np.float32))
            out[f"shift{i}"], out[f"sign{i}"] = conv.shift.data.numpy().copy(), conv.sign.data.numpy().copy()
        else:
            conv = ref_q.Conv2dShiftQ(cin, cout, k, stride=stride, padding=0, bias=True, use_kernel=True,
                                      use_cuda=False, act_integer_bits=1, act_fraction_bits=F)
            out[f"w{i}"] = conv.weight.data.numpy().copy()
        out[f"kind{i}"], out[f"bias{i}"] = np.array(kind), conv.bias.data.numpy().copy()
        out[f"x{i}"], out[f"stride{i}"], out[f"F{i}"] = xin.numpy().copy(), np.int32(stride), np.int32(F)
        with torch.no_grad():
            out[f"y{i}"] = conv(xin.clone()).numpy()
    out["n"] = np.int32(len(cases))
    np.savez_compressed(os.path.join(HERE, "sign_ref.npz"), **out)
    print("sign_ref.npz", os.path.getsize(os.path.join(HERE, "sign_ref.npz")), "bytes")


def main_gap():
    """gap_ref.npz: the glue between the last convolution and the classifier of the reference's
    ResNets (cifar10_models/resnet.py:122-134, torchvision's ResNet via imagenet.py:199-219):
    torch's CPU ``F.adaptive_avg_pool2d(x, 1)`` on fp32 planes of values on the 2^-12 grid, then the
    LinearShift entry conversion ``(x * 2^F).int()`` (modules.py:25).  Plane sums stay below 2^24
    codes, where fp32 summation is exact in any order; beyond that torch's own CPU result depends
    on the vector width of the machine and its CUDA kernel multiplies by a rounded reciprocal."""
    import torch.nn.functional as Fnn
    out = {}
    rng = np.random.default_rng(6000)
    cases = [(7, 1 << 16), (7, 1 << 18), (8, 1 << 17), (4, 1 << 19), (14, 1 << 16), (1, 1 << 23)]
    for i, (hw, top) in enumerate(cases):
        codes = rng.integers(-(top // 8), top, (3, 24, hw, hw)).astype(np.int32)
        codes[0] = np.maximum(codes[0], 0)                      # what follows a ReLU
        x = torch.from_numpy(codes.astype(np.float32) / np.float32(4096))
        pooled = Fnn.adaptive_avg_pool2d(x, 1).flatten(1)
        out[f"codes{i}"] = codes
        out[f"pooled{i}"] = pooled.numpy().copy()
        out[f"fixed{i}"] = (pooled * (2 ** 12)).int().numpy().copy()
    out["n"], out["F"] = np.int32(len(cases)), np.int32(12)
    np.savez_compressed(os.path.join(HERE, "gap_ref.npz"), **out)
    print("gap_ref.npz", os.path.getsize(os.path.join(HERE, "gap_ref.npz")), "bytes")


def main(reference_root):
    assert build_ref.build(reference_root) is not None, "reference checkout not found"
    assert O.ref_module() is not None

    # ---- integer kernels from the compiled reference -------------------------------------
    lin_cases = [  # (M, K, N, act kind, min shift, zeros)
        (1, 1, 1, "q16", -15, True), (3, 7, 5, "q16", -15, True), (64, 784, 32, "q16", -15, True),
        (17, 131, 19, "wide", -15, True), (8, 96, 24, "q16", -1, False), (5, 40, 11, "q16", -3, False),
        (9, 33, 13, "q16", -7, True), (4, 64, 10, "wide", -31, True),
    ]
    out = {}
    for i, (M, K, N, kind, lo, zeros) in enumerate(lin_cases):
        rng = np.random.default_rng(1000 + i)
        x = acts(rng, (M, K), kind)
        shift, sign = weights(rng, (N, K), lo, zeros)
        bias = rng.integers(-2000, 2000, N).astype(np.int32)
        out[f"x{i}"], out[f"shift{i}"], out[f"sign{i}"], out[f"bias{i}"] = x, shift, sign, bias
        out[f"y{i}"] = O.ref_linear(x, shift, sign, bias)
    out["n"] = np.int32(len(lin_cases))
    np.savez_compressed(os.path.join(HERE, "linear_ref.npz"), **out)

    conv_cases = [  # (B, C, H, W, OC, KH, KW, stride, pad, zeros)
        (2, 3, 8, 8, 4, 3, 3, (1, 1), (1, 1), False), (2, 4, 9, 7, 5, 3, 3, (2, 2), (1, 1), False),
        (1, 1, 12, 12, 6, 5, 5, (1, 1), (0, 0), False), (2, 3, 15, 15, 8, 7, 7, (2, 2), (3, 3), False),
        (3, 8, 6, 6, 16, 1, 1, (2, 2), (0, 0), False), (2, 5, 7, 7, 3, 3, 3, (1, 1), (1, 1), True),
        (1, 2, 6, 10, 4, 3, 5, (2, 1), (1, 2), False),
    ]
    out = {}
    for i, (B, C, H, W, OC, KH, KW, st, pad, zeros) in enumerate(conv_cases):
        rng = np.random.default_rng(2000 + i)
        x = acts(rng, (B, C, H, W))
        shift, sign = weights(rng, (OC, C, KH, KW), -15, zeros)
        bias = rng.integers(-2000, 2000, OC).astype(np.int32)
        xp = O.pad_nchw(x, *pad)
        out[f"x{i}"], out[f"shift{i}"], out[f"sign{i}"], out[f"bias{i}"] = x, shift, sign, bias
        out[f"stride{i}"], out[f"pad{i}"] = np.array(st, np.int32), np.array(pad, np.int32)
        # convolution_kernel treats sign 0 as +1 (shift_cpu.cpp:351-353); stored as it is.
        out[f"y{i}"] = O.ref_conv2d_prepadded(xp, shift, sign, bias, st)
    out["n"] = np.int32(len(conv_cases))
    np.savez_compressed(os.path.join(HERE, "conv_ref.npz"), **out)

    # ---- float glue from the reference's Python package ----------------------------------
    _import_reference(reference_root)
    import deepshift.modules as ref_modules
    import deepshift.utils as ref_utils

    out = {}
    rng = np.random.default_rng(3000)
    v = np.concatenate([rng.normal(0, 3, 4000), [7.5, 6.99999, -9.0, 7.0, -8.0, 0.0, -0.0, 1e-9, -1e-9,
                                                 8.0, 6.9998779296875, -7.999878]]).astype(np.float32)
    out["rtf_in"] = v
    for I, F in [(4, 12), (16, 16), (8, 8), (1, 7), (2, 3)]:
        out[f"rtf_{I}_{F}"] = ref_utils.round_to_fixed(torch.from_numpy(v), I, F).numpy()
    w = rng.normal(0, 0.05, (6, 50)).astype(np.float32)
    w[0, :5] = 0.0
    s, g = ref_utils.get_shift_and_sign(torch.from_numpy(w))
    out["gss_w"], out["gss_shift"], out["gss_sign"] = w, s.numpy(), g.numpy()

    torch.manual_seed(7)
    lin = ref_modules.LinearShift(40, 12, bias=True, use_kernel=True, use_cuda=False,
                                  act_integer_bits=4, act_fraction_bits=12)
    lin.shift.data = torch.from_numpy(rng.integers(-14, 1, (12, 40)).astype(np.float32))
    lin.sign.data = torch.from_numpy(rng.choice([-1.0, 0.0, 1.0], (12, 40), p=[.45, .1, .45]).astype(np.float32))
    xin = torch.from_numpy(rng.normal(0, 1, (9, 40)).astype(np.float32))
    out["lin_x"], out["lin_shift"], out["lin_sign"] = xin.numpy(), lin.shift.data.numpy(), lin.sign.data.numpy()
    out["lin_bias"] = lin.bias.data.numpy().copy()
    with torch.no_grad():
        out["lin_y"] = lin(xin).numpy()

    conv = ref_modules.Conv2dShift(3, 6, 3, stride=1, padding=0, bias=True, use_kernel=True, use_cuda=False,
                                   rounding="deterministic", act_integer_bits=4, act_fraction_bits=12)
    conv.shift.data = torch.from_numpy(rng.integers(-14, 1, (6, 3, 3, 3)).astype(np.float32))
    conv.sign.data = torch.from_numpy(rng.choice([-1.0, 1.0], (6, 3, 3, 3)).astype(np.float32))
    xin = torch.from_numpy(rng.normal(0, 3, (2, 3, 8, 8)).astype(np.float32))
    out["conv_x"], out["conv_shift"], out["conv_sign"] = xin.numpy().copy(), conv.shift.data.numpy(), conv.sign.data.numpy()
    out["conv_bias"] = conv.bias.data.numpy().copy()
    with torch.no_grad():
        out["conv_y"] = conv(xin).numpy()
    np.savez_compressed(os.path.join(HERE, "glue_ref.npz"), **out)
    for f in ("linear_ref.npz", "conv_ref.npz", "glue_ref.npz"):
        print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")


if __name__ == "__main__":
    flags = [a for a in sys.argv[1:] if a.startswith("--only-")]
    args = [a for a in sys.argv[1:] if not a.startswith("--only-")]
    root = args[0] if args else os.environ.get("DEEPSHIFT_REFERENCE")
    if flags == ["--only-gap"]:
        main_gap()
        sys.exit(0)
    if not root:
        sys.exit("give the path of the reference checkout (argument or DEEPSHIFT_REFERENCE)")
    if not flags:
        main(root)
    if not flags or "--only-q" in flags:
        main_q(root)
    if not flags or "--only-sign" in flags:
        main_sign(root)
    if not flags or "--only-gap" in flags:
        main_gap()
