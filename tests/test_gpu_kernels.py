"""Parity of the CUDA kernels with the CPU oracle, through the Python operator layer and the
C ABI.  Integer results must be bit-identical; fp32 results are exact conversions of them, so
they are compared with array_equal as well."""
import ctypes
import os

import numpy as np
import pytest
import torch

from helpers import acts_q16, acts_wide, weights

pytestmark = pytest.mark.gpu


def _cw(shift, sign, dev):
    from deepshift_b200 import utils
    return utils.compress_bits(torch.from_numpy(shift).float(), torch.from_numpy(sign).float(), device=dev)


def _t(a, dev):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


# ----------------------------------------------------------------------------------------- packing
@pytest.mark.parametrize("lo,zeros", [(-1, False), (-3, False), (-7, False), (-15, False), (-15, True), (-31, True)])
@pytest.mark.parametrize("K", [1, 5, 16, 131])
def test_compress_matches_oracle(oracle, cuda_device, lo, zeros, K):
    rng = np.random.default_rng(K - lo)
    shift, sign = weights(rng, (7, K), lo, zeros)
    cw = _cw(shift, sign, cuda_device)
    packed, base, bits = oracle.compress_bits(shift, sign)
    assert (cw.base, cw.bits) == (base, bits)
    assert np.array_equal(cw.data.cpu().numpy().reshape(packed.shape), packed)


def test_compress_api_matches_reference_signature(oracle, cuda_device):
    from deepshift_b200 import kernels
    rng = np.random.default_rng(3)
    shiftp = rng.integers(0, 16, (4, 3, 3, 3)).astype(np.int32)
    sign = rng.choice([-1, 1], (4, 3, 3, 3)).astype(np.int32)
    bits, num = 4, 6
    row = (27 + num - 1) // num
    out = kernels.compress_sign_and_shift(_t(shiftp, cuda_device), _t(sign, cuda_device), 4 * row, 0, bits, row, num)
    assert out.dtype == torch.int32 and out.shape == (4 * row,)
    assert np.array_equal(out.cpu().numpy().reshape(4, row), oracle.compress(shiftp.reshape(4, -1), sign.reshape(4, -1), bits, 0))
    with pytest.raises(RuntimeError, match="inconsistent"):
        kernels.compress_sign_and_shift(_t(shiftp, cuda_device), _t(sign, cuda_device), 4 * row, 0, bits, row + 1, num)


# ----------------------------------------------------------------------------------------- linear
LINEAR_SHAPES = [(1, 1, 1), (3, 7, 5), (64, 784, 512), (130, 131, 129), (257, 500, 10), (64, 512, 10), (200, 96, 70),
                 (1000, 300, 40), (1, 4096, 33), (513, 29, 260),
                 (1, 4096, 4096), (64, 4096, 4096),     # the small-batch corner of the shift-GEMM sweep
                 (256, 512, 1000),                      # a classifier head at the benchmark batch
                 (2, 640, 37), (5, 1031, 300), (8, 512, 1000), (13, 2048, 24), (16, 96, 4100), (17, 520, 130), (40, 3000, 70)]


@pytest.mark.parametrize("M,K,N", LINEAR_SHAPES)
@pytest.mark.parametrize("act_bits", [0, 16])
def test_linear_matches_oracle(oracle, cuda_device, M, K, N, act_bits):
    from deepshift_b200 import kernels
    rng = np.random.default_rng(M * 7 + K * 3 + N)
    x = acts_q16(rng, (M, K))
    shift, sign = weights(rng, (N, K))
    bias = rng.integers(-2000, 2000, N).astype(np.int32)
    out = kernels.linear(_t(x, cuda_device), _t(shift, cuda_device), None, _t(bias, cuda_device),
                         _cw(shift, sign, cuda_device), act_bits=act_bits)
    assert out.dtype == torch.int32 and tuple(out.shape) == (M, N)
    assert np.array_equal(out.cpu().numpy(), oracle.linear(x, shift, sign, bias))


@pytest.mark.parametrize("lo,zeros", [(-1, False), (-3, False), (-7, False), (-15, False), (-31, True), (-15, True)])
@pytest.mark.parametrize("act_bits", [0, 16])
def test_linear_every_field_width(oracle, cuda_device, lo, zeros, act_bits):
    """bits = 1..6, i.e. 16, 10, 8, 6, 5 and 4 weights per word, ragged K."""
    from deepshift_b200 import kernels
    rng = np.random.default_rng(-lo * 13 + act_bits)
    M, K, N = 70, 203, 37
    x = acts_q16(rng, (M, K))
    shift, sign = weights(rng, (N, K), lo, zeros)
    cw = _cw(shift, sign, cuda_device)
    out = kernels.linear(_t(x, cuda_device), _t(shift, cuda_device), None, None, cw, act_bits=act_bits)
    assert np.array_equal(out.cpu().numpy(), oracle.linear(x, shift, sign, None))


# Linear layers whose rows are whole 16-byte groups (K % 4 == 0) and more than 32 columns run on
# the warp-specialised kernel: a producer thread per row of x, 16-byte loads along k.
WS_LINEAR_SHAPES = [(65, 4, 33),        # one k-group, one ragged tile
                    (300, 512, 200),    # producers decode the packed words (few row tiles)
                    (2304, 260, 130),   # nine row tiles: weights expanded once per launch, ragged last k-tile
                    (1024, 2048, 96),   # four tiles on 148 SMs: every tile is shared along K through the workspace
                    (2100, 1000, 64),   # 256 x 64 tile
                    (257, 36, 129)]


@pytest.mark.parametrize("M,K,N", WS_LINEAR_SHAPES)
def test_linear_on_warp_specialised_kernel(oracle, cuda_device, M, K, N):
    from deepshift_b200 import _ffi, kernels
    rng = np.random.default_rng(M + K * 5 + N * 11)
    x = acts_q16(rng, (M, K))
    shift, sign = weights(rng, (N, K))
    bias = rng.integers(-2000, 2000, N).astype(np.int32)
    ref = oracle.linear(x, shift, sign, bias)
    xt, bt, cw = _t(x, cuda_device), _t(bias, cuda_device), _cw(shift, sign, cuda_device)
    for _ in range(2):  # the second launch finds the arrival counters as the first left them
        out = kernels.linear(xt, _t(shift, cuda_device), None, bt, cw, act_bits=16)
        assert np.array_equal(out.cpu().numpy(), ref)
    assert int(kernels.workspace(cuda_device)[:16383].abs().sum()) == 0
    # the same layer without a workspace (plain C entry point) and on the exact integer path
    for act_bits in (16, 0):
        out2 = torch.empty_like(out)
        rc = _ffi.lib().ds_linear_i32(xt.data_ptr(), cw.data.data_ptr(), bt.data_ptr(), out2.data_ptr(), M, K, N,
                                      cw.bits, cw.base, act_bits, torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        assert np.array_equal(out2.cpu().numpy(), ref)
    flag = ctypes.c_int(-1)
    assert _ffi.lib().ds_last_kernel_error(ctypes.byref(flag)) == 0 and flag.value == 0


@pytest.mark.parametrize("lo,zeros", [(-1, False), (-3, False), (-7, False), (-15, False), (-31, True), (-15, True)])
@pytest.mark.parametrize("M", [200, 2200])
def test_linear_on_warp_specialised_kernel_every_field_width(oracle, cuda_device, lo, zeros, M):
    """16, 10, 8, 6, 5 and 4 weights per word: k-tiles of 16, 20, 24, 24, 20 and 28 when the
    producers decode (M = 200), the k-tile that pads K least with expanded weights (M = 2200)."""
    from deepshift_b200 import kernels
    rng = np.random.default_rng(-lo * 17 + M)
    K, N = 204, 70
    x = acts_q16(rng, (M, K))
    shift, sign = weights(rng, (N, K), lo, zeros)
    out = kernels.linear(_t(x, cuda_device), _t(shift, cuda_device), None, None, _cw(shift, sign, cuda_device),
                         act_bits=16)
    assert np.array_equal(out.cpu().numpy(), oracle.linear(x, shift, sign, None))


def test_linear_unaligned_rows_stay_on_the_block_kernel(oracle, cuda_device):
    """A view whose first row does not start on a 16-byte boundary."""
    from deepshift_b200 import kernels
    rng = np.random.default_rng(41)
    M, K, N = 300, 64, 48
    x = acts_q16(rng, (M, K))
    shift, sign = weights(rng, (N, K))
    buf = torch.zeros(M * K + 1, dtype=torch.int32, device=cuda_device)
    xt = buf[1:].view(M, K)
    xt.copy_(_t(x, cuda_device))
    assert xt.data_ptr() % 16 != 0
    out = kernels.linear(xt, _t(shift, cuda_device), None, None, _cw(shift, sign, cuda_device), act_bits=16)
    assert np.array_equal(out.cpu().numpy(), oracle.linear(x, shift, sign, None))


def test_linear_golden_vectors_of_the_reference(oracle, cuda_device, golden_dir):
    from deepshift_b200 import kernels
    g = np.load(os.path.join(golden_dir, "linear_ref.npz"))
    for i in range(int(g["n"])):
        x, shift, sign, bias = g[f"x{i}"], g[f"shift{i}"], g[f"sign{i}"], g[f"bias{i}"]
        out = kernels.linear(_t(x, cuda_device), _t(shift, cuda_device), None, _t(bias, cuda_device),
                             _cw(shift, sign, cuda_device))
        assert np.array_equal(out.cpu().numpy(), g[f"y{i}"]), i


def test_linear_wide_inputs_wrap_like_the_reference(oracle, cuda_device):
    """Unbounded int32 activations take the integer path; sums wrap modulo 2^32."""
    from deepshift_b200 import kernels
    rng = np.random.default_rng(8)
    x = acts_wide(rng, (33, 300), 30)
    shift, sign = weights(rng, (17, 300), -3, zeros=False)
    out = kernels.linear(_t(x, cuda_device), _t(shift, cuda_device), None, None, _cw(shift, sign, cuda_device))
    assert np.array_equal(out.cpu().numpy(), oracle.linear(x, shift, sign, None))


def test_linear_left_shifts(oracle, cuda_device):
    from deepshift_b200 import kernels
    rng = np.random.default_rng(9)
    x = acts_wide(rng, (20, 50), 12)
    shift = rng.integers(-6, 4, (9, 50)).astype(np.int32)
    sign = rng.choice([-1, 0, 1], (9, 50)).astype(np.int32)
    cw = _cw(shift, sign, cuda_device)
    assert cw.base < 0
    out = kernels.linear(_t(x, cuda_device), _t(shift, cuda_device), None, None, cw, act_bits=16)  # hint ignored: base != 0
    assert np.array_equal(out.cpu().numpy(), oracle.linear(x, shift, sign, None))


def test_linear_empty_batch_and_errors(cuda_device):
    from deepshift_b200 import kernels, utils
    rng = np.random.default_rng(1)
    shift, sign = weights(rng, (4, 8))
    cw = _cw(shift, sign, cuda_device)
    out = kernels.linear(torch.zeros((0, 8), dtype=torch.int32, device=cuda_device), _t(shift, cuda_device), None, None, cw)
    assert tuple(out.shape) == (0, 4)
    with pytest.raises(RuntimeError, match="must be torch.int32"):
        kernels.linear(torch.zeros((2, 8), device=cuda_device), _t(shift, cuda_device), None, None, cw)
    with pytest.raises(RuntimeError, match="must be contiguous"):
        kernels.linear(torch.zeros((8, 2), dtype=torch.int32, device=cuda_device).t(), _t(shift, cuda_device), None, None, cw)
    bad = utils.ConcWeight(cw.data, 0, 9)
    with pytest.raises(RuntimeError, match="unsupported"):
        kernels.linear(torch.zeros((2, 8), dtype=torch.int32, device=cuda_device), _t(shift, cuda_device), None, None, bad)


# ----------------------------------------------------------------------------------------- convolution
CONV_CASES = [  # B, C, H, W, OC, KH, KW, stride, pad, zeros
    (2, 3, 8, 8, 4, 3, 3, (1, 1), (1, 1), True), (2, 4, 9, 7, 5, 3, 3, (2, 2), (1, 1), True),
    (3, 1, 28, 28, 20, 5, 5, (1, 1), (0, 0), True), (2, 3, 30, 30, 64, 7, 7, (2, 2), (3, 3), True),
    (3, 64, 14, 14, 128, 1, 1, (2, 2), (0, 0), False), (4, 64, 7, 7, 64, 3, 3, (1, 1), (1, 1), True),
    (2, 16, 12, 12, 33, 3, 3, (1, 1), (1, 1), True), (5, 32, 8, 8, 130, 3, 3, (1, 1), (1, 1), True),
    (2, 5, 9, 11, 7, 2, 4, (1, 2), (1, 0), True), (1, 3, 6, 6, 3, 6, 6, (1, 1), (0, 0), True),
    (2, 20, 12, 12, 50, 5, 5, (1, 1), (0, 0), True), (300, 2, 5, 5, 3, 3, 3, (1, 1), (1, 1), True),
    (2, 3, 13, 13, 8, 9, 9, (2, 2), (4, 4), True),
    # 7x7 stride 2 padding 3 on widths that are multiples of 8: four output pixels per producer thread
    (2, 3, 32, 32, 64, 7, 7, (2, 2), (3, 3), True), (3, 4, 22, 40, 70, 7, 7, (2, 2), (3, 3), True),
    (2, 2, 9, 16, 5, 7, 7, (3, 2), (1, 3), True), (1, 3, 8, 8, 9, 7, 7, (2, 2), (3, 3), True),
]


@pytest.mark.parametrize("case", CONV_CASES, ids=lambda c: "x".join(str(v) for v in c[:7]))
@pytest.mark.parametrize("act_bits", [0, 16])
def test_conv_matches_oracle(oracle, cuda_device, case, act_bits):
    from deepshift_b200 import kernels
    B, C, H, W, OC, KH, KW, st, pad, zeros = case
    rng = np.random.default_rng(B * 31 + C * 17 + OC)
    x = acts_q16(rng, (B, C, H, W))
    shift, sign = weights(rng, (OC, C, KH, KW), -15, zeros)
    bias = rng.integers(-2000, 2000, OC).astype(np.int32)
    out = kernels.conv2d(_t(x, cuda_device), _t(shift, cuda_device), None, _t(bias, cuda_device),
                         _cw(shift, sign, cuda_device), st, pad, act_bits=act_bits)
    ref = oracle.conv2d(x, shift, sign, bias, st, pad)
    assert tuple(out.shape) == ref.shape
    assert np.array_equal(out.cpu().numpy(), ref)


def test_conv_golden_vectors_of_the_reference(cuda_device, golden_dir):
    """Zero-free cases equal the reference's CPU convolution output verbatim."""
    from deepshift_b200 import kernels
    g = np.load(os.path.join(golden_dir, "conv_ref.npz"))
    checked = 0
    for i in range(int(g["n"])):
        if (g[f"sign{i}"] == 0).any():
            continue
        x, shift, sign, bias = g[f"x{i}"], g[f"shift{i}"], g[f"sign{i}"], g[f"bias{i}"]
        out = kernels.conv2d(_t(x, cuda_device), _t(shift, cuda_device), None, _t(bias, cuda_device),
                             _cw(shift, sign, cuda_device), tuple(int(v) for v in g[f"stride{i}"]),
                             tuple(int(v) for v in g[f"pad{i}"]), act_bits=16)
        assert np.array_equal(out.cpu().numpy(), g[f"y{i}"]), i
        checked += 1
    assert checked >= 5


def test_conv_rejects_dilation_and_groups(cuda_device):
    from deepshift_b200 import kernels
    rng = np.random.default_rng(2)
    shift, sign = weights(rng, (4, 2, 3, 3))
    cw = _cw(shift, sign, cuda_device)
    x = torch.zeros((1, 2, 6, 6), dtype=torch.int32, device=cuda_device)
    with pytest.raises(RuntimeError, match="dilation"):
        kernels.conv2d(x, _t(shift, cuda_device), None, None, cw, 1, 0, dilation=2)
    with pytest.raises(RuntimeError, match="dilation"):
        kernels.conv2d(x, _t(shift, cuda_device), None, None, cw, 1, 0, groups=2)


# ----------------------------------------------------------------------------------------- fused forms
@pytest.mark.parametrize("shape", [(2, 8, 12, 12, 16, 3, 1, 1), (3, 16, 9, 9, 140, 3, 2, 1), (2, 6, 10, 10, 70, 1, 1, 0),
                                   (2, 3, 24, 24, 40, 7, 2, 3)])
def test_conv_fused_epilogues(oracle, cuda_device, shape):
    from deepshift_b200 import _ffi, kernels
    B, C, H, OC, k, s, p = shape[0], shape[1], shape[2], shape[4], shape[5], shape[6], shape[7]
    I, F = 4, 12
    rng = np.random.default_rng(sum(shape))
    xf = rng.normal(0, 3, (B, C, H, H)).astype(np.float32)
    shift, sign = weights(rng, (OC, C, k, k))
    bias = rng.integers(-2000, 2000, OC).astype(np.int32)
    cw = _cw(shift, sign, cuda_device)
    xi = oracle.to_fixed_conv(xf, I, F)
    ref = oracle.conv2d(xi, shift, sign, bias, (s, s), (p, p))
    wshape = (OC, C, k, k)
    # fp32 in (quantised in the kernel), fp32 out
    out = kernels.conv2d_fused(_t(xf, cuda_device), wshape, _t(bias, cuda_device), cw, s, p, in_kind=_ffi.IN_F32_CONV,
                               out_kind=_ffi.OUT_F32, act_integer_bits=I, act_fraction_bits=F)
    assert np.array_equal(out.cpu().numpy(), oracle.from_fixed(ref, F))
    # unclamped int32 in, clamped on read; residual + ReLU + fp32 rounding in the epilogue
    wide = (xi.astype(np.int64) * 3).astype(np.int32)
    res = rng.integers(-50000, 50000, ref.shape).astype(np.int32)
    lo, hi = -(1 << (I - 1 + F)), ((1 << (I - 1)) - 1) << F
    ref2 = oracle.conv2d(np.clip(wide, lo, hi), shift, sign, bias, (s, s), (p, p))
    ref2 = np.maximum(ref2.astype(np.float32) + res.astype(np.float32), 0).astype(np.int64).astype(np.int32)
    out = kernels.conv2d_fused(_t(wide, cuda_device), wshape, _t(bias, cuda_device), cw, s, p,
                               in_kind=_ffi.IN_I32_CLAMP, act_integer_bits=I, act_fraction_bits=F, relu=True,
                               residual=_t(res, cuda_device), round_f32=True)
    assert np.array_equal(out.cpu().numpy(), ref2)
    # requantise clamp on write
    out = kernels.conv2d_fused(_t(xi, cuda_device), wshape, _t(bias, cuda_device), cw, s, p, act_bits=16,
                               act_integer_bits=I, act_fraction_bits=F, relu=True, requant=True)
    assert np.array_equal(out.cpu().numpy(), np.clip(np.maximum(ref, 0), lo, hi))


def test_linear_fused_fp32(oracle, cuda_device):
    from deepshift_b200 import _ffi, kernels
    rng = np.random.default_rng(4)
    xf = rng.normal(0, 2, (37, 90)).astype(np.float32)
    shift, sign = weights(rng, (21, 90))
    bias = rng.integers(-2000, 2000, 21).astype(np.int32)
    ref = oracle.linear(oracle.to_fixed_linear(xf, 12), shift, sign, bias)
    out = kernels.linear_fused(_t(xf, cuda_device), 21, _t(bias, cuda_device), _cw(shift, sign, cuda_device),
                               in_kind=_ffi.IN_F32_LINEAR, out_kind=_ffi.OUT_F32, act_fraction_bits=12, relu=True)
    assert np.array_equal(out.cpu().numpy(), oracle.from_fixed(np.maximum(ref, 0), 12))


def test_quantize_matches_round_to_fixed(oracle, cuda_device):
    from deepshift_b200 import kernels
    rng = np.random.default_rng(6)
    v = np.concatenate([rng.normal(0, 4, 5000), [7.5, 6.99999, -9.0, 7.0, -8.0, 0.0, 1e-9, -1e-9]]).astype(np.float32)
    for I, F in [(4, 12), (8, 8), (2, 3), (1, 7)]:
        got = kernels.quantize(_t(v, cuda_device), I, F, like_conv=True).cpu().numpy()
        assert np.array_equal(got, oracle.to_fixed_conv(v, I, F)), (I, F)
    got = kernels.quantize(_t(v, cuda_device), 4, 12, like_conv=False).cpu().numpy()
    assert np.array_equal(got, oracle.to_fixed_linear(v, 12))


def test_pooling_on_codes(cuda_device):
    from deepshift_b200 import kernels
    rng = np.random.default_rng(7)
    x = rng.integers(-40000, 40000, (3, 5, 13, 13)).astype(np.int32)
    xt = _t(x, cuda_device)
    for k, s, p in [(2, 2, 0), (3, 2, 1)]:
        ref = torch.nn.functional.max_pool2d(xt.double(), k, s, p).to(torch.int32)
        assert torch.equal(kernels.maxpool2d_i32(xt, k, s, p), ref)
    # widths that are a multiple of 8 take the four-outputs-per-thread kernel of the 3x3/2/1 pool
    for shape in [(2, 3, 16, 16), (1, 2, 9, 24), (2, 1, 112, 112)]:
        y = _t(rng.integers(-40000, 40000, shape).astype(np.int32), cuda_device)
        ref = torch.nn.functional.max_pool2d(y.double(), 3, 2, 1).to(torch.int32)
        assert torch.equal(kernels.maxpool2d_i32(y, 3, 2, 1), ref)
    F = 12
    got = kernels.avgpool_fix_i32(xt, F).cpu().numpy()
    mean = (x.astype(np.int64).sum(axis=(2, 3)).astype(np.float32) / np.float32(1 << F)) / np.float32(169)
    assert np.array_equal(got, np.trunc(mean.astype(np.float32) * np.float32(1 << F)).astype(np.int32))


# ----------------------------------------------------------------------------------------- modules
def test_modules_match_reference_golden_forward(cuda_device, golden_dir):
    """LinearShift / Conv2dShift with use_kernel=True reproduce the fp32 outputs recorded from the
    reference's own modules (use_cuda=False there)."""
    from deepshift_b200 import modules
    g = np.load(os.path.join(golden_dir, "glue_ref.npz"))
    lin = modules.LinearShift(40, 12, use_kernel=True, act_integer_bits=4, act_fraction_bits=12).to(cuda_device)
    lin.shift.data, lin.sign.data, lin.bias.data = (_t(g["lin_shift"], cuda_device), _t(g["lin_sign"], cuda_device),
                                                    _t(g["lin_bias"], cuda_device))
    assert np.array_equal(lin(_t(g["lin_x"], cuda_device)).cpu().numpy(), g["lin_y"])
    conv = modules.Conv2dShift(3, 6, 3, use_kernel=True, act_integer_bits=4, act_fraction_bits=12).to(cuda_device)
    conv.shift.data, conv.sign.data, conv.bias.data = (_t(g["conv_shift"], cuda_device), _t(g["conv_sign"], cuda_device),
                                                       _t(g["conv_bias"], cuda_device))
    assert np.array_equal(conv(_t(g["conv_x"], cuda_device)).cpu().numpy(), g["conv_y"])


def test_convert_to_shift_use_kernel_end_to_end(oracle, cuda_device):
    import torch.nn as nn
    from deepshift_b200 import convert, modules
    torch.manual_seed(3)
    model = nn.Sequential(nn.Conv2d(3, 8, 3, padding=1), nn.ReLU(), nn.MaxPool2d(2), nn.Flatten(), nn.Linear(8 * 16, 10))
    model, n = convert.convert_to_shift(model, 1000, 'PS', convert_weights=True, use_kernel=True,
                                        act_integer_bits=4, act_fraction_bits=12)
    model = convert.round_shift_weights(model.to(cuda_device), act_integer_bits=4, act_fraction_bits=12)
    assert n == 1 and isinstance(model[0], modules.Conv2dShift) and model[0].conc_weight is not None
    x = torch.randn(5, 3, 8, 8)
    y = model(x.to(cuda_device)).cpu().numpy()
    c, l = model[0], model[4]
    I, F = 4, 12
    ci = oracle.conv2d(oracle.to_fixed_conv(x.numpy(), I, F), c.shift.data.cpu().numpy().astype(np.int32),
                       c.sign.data.cpu().numpy().astype(np.int32), oracle.to_fixed_conv(c.bias.data.cpu().numpy(), I, F),
                       (1, 1), (1, 1))
    h = np.maximum(oracle.from_fixed(ci, F), 0)
    h = torch.nn.functional.max_pool2d(torch.from_numpy(h), 2).flatten(1).numpy()
    li = oracle.linear(oracle.to_fixed_linear(h, F), l.shift.data.cpu().numpy().astype(np.int32),
                       l.sign.data.cpu().numpy().astype(np.int32), oracle.to_fixed_linear(l.bias.data.cpu().numpy(), F))
    assert np.array_equal(y, oracle.from_fixed(li, F))


@pytest.mark.parametrize("I,F", [(4, 12), (8, 16)])
def test_q_modules_use_kernel_match_oracle(oracle, cuda_device, I, F):
    """DeepShift-Q layers: weights rounded to powers of two on the fly, then the same kernels.
    (4, 12) takes the FP32-pipe path, (8, 16) the exact integer path."""
    from deepshift_b200 import modules_q, utils
    torch.manual_seed(17 + I)
    rng = np.random.default_rng(I)
    conv = modules_q.Conv2dShiftQ(6, 40, 3, stride=1, padding=1, use_kernel=True, act_integer_bits=I,
                                  act_fraction_bits=F).to(cuda_device)
    conv.weight.data.mul_(torch.from_numpy(rng.choice([1.0, 0.02, 30.0], conv.weight.shape).astype(np.float32)).to(cuda_device))
    conv.weight.data[0, 0] = 0.0
    xf = (rng.normal(0, 3, (3, 6, 10, 12))).astype(np.float32)
    y = conv(_t(xf, cuda_device))
    w = conv.weight.data.cpu()
    assert float(w.abs().max()) <= 1.0 and float(w[w != 0].abs().min()) >= 2.0 ** -15
    shift, sign = utils.get_shift_and_sign(w)
    shift = torch.where(sign == 0, torch.zeros_like(shift), shift)   # log2(0): any value, the sign is 0
    bias_i = (utils.round_to_fixed(conv.bias.data.cpu(), I, F) * 2 ** F).int().numpy()
    xi = oracle.to_fixed_conv(xf, I, F)
    ref = oracle.conv2d(xi, shift.numpy().astype(np.int32), sign.numpy().astype(np.int32), bias_i, (1, 1), (1, 1))
    assert np.array_equal(y.cpu().numpy(), oracle.from_fixed(ref, F))
    assert conv(_t(xf, cuda_device)).equal(y)            # packed weights are cached
    conv.weight.data.neg_()                               # same storage, no version bump: repack on request
    conv.conc_weight = None
    assert np.array_equal(conv(_t(xf, cuda_device)).cpu().numpy(),
                          oracle.from_fixed(oracle.conv2d(xi, shift.numpy().astype(np.int32),
                                                          -sign.numpy().astype(np.int32), bias_i, (1, 1), (1, 1)), F))

    lin = modules_q.LinearShiftQ(52, 70, use_kernel=True, act_integer_bits=I, act_fraction_bits=F).to(cuda_device)
    xl = rng.normal(0, 2, (5, 13, 52)).astype(np.float32)   # 65 rows after flattening
    yl = lin(_t(xl, cuda_device))
    assert tuple(yl.shape) == (5, 13, 70)
    wl = lin.weight.data.cpu()
    shift, sign = utils.get_shift_and_sign(wl)
    bias_i = (utils.round_to_fixed(lin.bias.data.cpu(), I, F) * 2 ** F).int().numpy()
    xi = oracle.to_fixed_conv(xl.reshape(-1, 52), I, F)
    ref = oracle.linear(xi, shift.numpy().astype(np.int32), sign.numpy().astype(np.int32), bias_i)
    assert np.array_equal(yl.cpu().numpy().reshape(-1, 70), oracle.from_fixed(ref, F))


def test_q_module_golden_forward_of_the_reference(cuda_device, golden_dir):
    from deepshift_b200 import modules_q
    g = np.load(os.path.join(golden_dir, "q_ref.npz"))
    for i in range(int(g["n"])):
        w = g[f"w{i}"]
        conv = modules_q.Conv2dShiftQ(w.shape[1], w.shape[0], w.shape[2], stride=int(g[f"stride{i}"]), padding=0,
                                      use_kernel=True, act_integer_bits=4, act_fraction_bits=12).to(cuda_device)
        conv.weight.data = _t(w, cuda_device)
        conv.bias.data = _t(g[f"bias{i}"], cuda_device)
        assert np.array_equal(conv(_t(g[f"x{i}"], cuda_device)).cpu().numpy(), g[f"y{i}"]), i


def test_convert_to_shift_q_use_kernel_end_to_end(cuda_device):
    """A converted DeepShift-Q model with use_kernel=True agrees with its own fp32 path up to the
    truncation of the right shifts: at most one unit of 2^-F per term."""
    import torch.nn as nn
    from deepshift_b200 import convert
    torch.manual_seed(23)
    I, F = 4, 12
    model = nn.Sequential(nn.Conv2d(3, 16, 3, padding=1), nn.ReLU(), nn.Conv2d(16, 8, 3, stride=2, padding=1), nn.ReLU(),
                          nn.Flatten(), nn.Linear(8 * 16, 10)).to(cuda_device)
    model, n = convert.convert_to_shift(model, 10, 'Q', use_kernel=True, act_integer_bits=I, act_fraction_bits=F)
    assert n == 2
    x = torch.randn(70, 3, 8, 8, device=cuda_device)
    y = model(x)
    for m in model:
        if hasattr(m, 'use_kernel'):
            m.use_kernel = False
    y_float = model(x)
    assert y.shape == y_float.shape == (70, 10)
    assert float((y - y_float).detach().abs().max()) < 0.2


def test_reference_default_activation_bits_16_16(oracle, cuda_device):
    """The constructors' defaults, act_integer_bits = act_fraction_bits = 16: codes fill the whole
    int32 range ([-2^31, 32767 * 2^16]) and sums wrap modulo 2^32 as in the reference."""
    from deepshift_b200 import kernels, modules
    rng = np.random.default_rng(1616)
    xf = (rng.normal(0, 1, (2, 3, 9, 9)) * rng.choice([1.0, 300.0, 40000.0], (2, 3, 9, 9))).astype(np.float32)
    xf[0, 0, 0, :4] = [-32768.0, 32767.99, 1e9, -1e9]
    codes = kernels.quantize(_t(xf, cuda_device), 16, 16, like_conv=True)
    xi = oracle.to_fixed_conv(xf, 16, 16)
    assert xi.min() == -2 ** 31 and xi.max() == 32767 * 65536
    assert np.array_equal(codes.cpu().numpy(), xi)
    conv = modules.Conv2dShift(3, 40, 3, padding=1, use_kernel=True).to(cuda_device)   # default bits
    shift, sign = weights(rng, (40, 3, 3, 3))
    conv.shift.data = _t(shift.astype(np.float32), cuda_device)
    conv.sign.data = _t(sign.astype(np.float32), cuda_device)
    conv.bias.data = _t(rng.normal(0, 100, 40).astype(np.float32), cuda_device)
    y = conv(_t(xf, cuda_device))
    bias_i = oracle.to_fixed_conv(conv.bias.data.cpu().numpy(), 16, 16)
    ref = oracle.conv2d(xi, shift, sign, bias_i, (1, 1), (1, 1))
    assert np.array_equal(y.cpu().numpy(), oracle.from_fixed(ref, 16))


def test_no_kernel_wait_ran_out(cuda_device):
    """The warp-specialised kernel's bounded waits never give up in a correct run."""
    from deepshift_b200 import _ffi
    flag = ctypes.c_int(-1)
    assert _ffi.lib().ds_last_kernel_error(ctypes.byref(flag)) == 0
    assert flag.value == 0


@pytest.mark.parametrize("out_f32", [False, True])
def test_conv_split_k_with_workspace(oracle, cuda_device, out_f32):
    """Few output tiles and a long K: the tiles are shared between CTAs along K (partial sums
    through the workspace, the last CTA of a tile applies the epilogue).  Same bits as the unsplit
    result, twice in a row (the arrival counters return to zero)."""
    from deepshift_b200 import _ffi, kernels
    rng = np.random.default_rng(21)
    B, C, H, OC = 5, 128, 7, 130
    I, F = 4, 12
    x = acts_q16(rng, (B, C, H, H))
    shift, sign = weights(rng, (OC, C, 3, 3))
    bias = rng.integers(-2000, 2000, OC).astype(np.int32)
    res = rng.integers(-50000, 50000, (B, OC, H, H)).astype(np.int32)
    cw = _cw(shift, sign, cuda_device)
    ref = oracle.conv2d(x, shift, sign, bias, (1, 1), (1, 1))
    ref = np.maximum(ref.astype(np.float32) + res.astype(np.float32), 0).astype(np.int64).astype(np.int32)
    want = oracle.from_fixed(ref, F) if out_f32 else ref
    for _ in range(2):
        out = kernels.conv2d_fused(_t(x, cuda_device), (OC, C, 3, 3), _t(bias, cuda_device), cw, 1, 1,
                                   in_kind=_ffi.IN_I32_CLAMP, out_kind=_ffi.OUT_F32 if out_f32 else _ffi.OUT_I32,
                                   act_integer_bits=I, act_fraction_bits=F, relu=True, residual=_t(res, cuda_device),
                                   round_f32=True)
        assert np.array_equal(out.cpu().numpy(), want)
    assert int(kernels.workspace(cuda_device)[:16383].abs().sum()) == 0


@pytest.mark.parametrize("B", [49, 68])
def test_conv_tail_wave_is_split(oracle, cuda_device, B):
    """A few more output tiles than SMs (151 and 209 on 148): the tiles after the last full wave
    are cut along K, in one and in two rounds of tail units; the other tiles are computed whole
    by the same launch."""
    from deepshift_b200 import kernels
    rng = np.random.default_rng(77 + B)
    C, H, OC = 32, 28, 100
    x = acts_q16(rng, (B, C, H, H))
    shift, sign = weights(rng, (OC, C, 3, 3))
    bias = rng.integers(-2000, 2000, OC).astype(np.int32)
    ref = oracle.conv2d(x, shift, sign, bias, (1, 1), (1, 1))
    for _ in range(2):
        out = kernels.conv2d(_t(x, cuda_device), _t(shift, cuda_device), None, _t(bias, cuda_device),
                             _cw(shift, sign, cuda_device), 1, 1, act_bits=16)
        assert np.array_equal(out.cpu().numpy(), ref)
    assert int(kernels.workspace(cuda_device)[:16383].abs().sum()) == 0


@pytest.mark.parametrize("shape", [(12, 16, 28, 28, 40, 3, 1, 1),    # four-pixel staging, 37 row tiles
                                   (9, 3, 60, 60, 24, 7, 2, 3),      # 7-wide rows: k-tiles of 21 with a workspace
                                   (9, 3, 64, 64, 24, 7, 2, 3),      # the same on a width of 8n: four-pixel stem staging
                                   (9, 5, 48, 72, 100, 7, 2, 3),     # ... 256 x 128 tile, ragged last k-tile
                                   (11, 40, 30, 30, 96, 1, 2, 0),    # 1x1, stride 2
                                   (10, 12, 26, 30, 70, 3, 1, 1)])   # 3x3 on a width that is no multiple of 4
def test_conv_with_and_without_workspace_agree(oracle, cuda_device, shape):
    """The same convolution through ds_conv2d_ex with the Python layer's workspace (weights
    expanded once per launch, k-tile free of the packed-word size, tail tiles shared) and
    through ds_conv2d_i32 without any (the producers decode the packed words): same bits, and
    the library counts three kernels for the first and one for the second."""
    from deepshift_b200 import _ffi, kernels
    B, C, H, W, OC, k, s, p = shape
    rng = np.random.default_rng(sum(shape))
    x = acts_q16(rng, (B, C, H, W))
    shift, sign = weights(rng, (OC, C, k, k))
    bias = rng.integers(-2000, 2000, OC).astype(np.int32)
    cw = _cw(shift, sign, cuda_device)
    xt, bt = _t(x, cuda_device), _t(bias, cuda_device)
    lib = _ffi.lib()
    n0 = lib.ds_launch_count()
    with_ws = kernels.conv2d(xt, _t(shift, cuda_device), None, bt, cw, s, p, act_bits=16)
    n1 = lib.ds_launch_count()
    OH, OW = (H + 2 * p - k) // s + 1, (W + 2 * p - k) // s + 1
    plain = torch.empty((B, OC, OH, OW), dtype=torch.int32, device=cuda_device)
    rc = lib.ds_conv2d_i32(xt.data_ptr(), cw.data.data_ptr(), bt.data_ptr(), plain.data_ptr(), B, C, H, W, OC,
                           k, k, s, s, p, p, cw.bits, cw.base, 16, torch.cuda.current_stream().cuda_stream)
    n2 = lib.ds_launch_count()
    assert rc == 0
    assert torch.equal(with_ws, plain)
    assert np.array_equal(plain.cpu().numpy(), oracle.conv2d(x, shift, sign, bias, (s, s), (p, p)))
    assert (n1 - n0, n2 - n1) == (3, 1)


def test_weights_prepared_once_are_reused(oracle, cuda_device):
    """conv2d_fused expands a layer's weights on its first call for a geometry (ds_conv2d_prepare)
    and hands the buffer to every later call: three kernels, then one, same bits as the oracle;
    a geometry whose launches do not use expanded weights asks for no buffer."""
    from deepshift_b200 import _ffi, kernels
    rng = np.random.default_rng(99)
    B, C, H, OC = 12, 16, 28, 40
    x = acts_q16(rng, (B, C, H, H))
    shift, sign = weights(rng, (OC, C, 3, 3))
    bias = rng.integers(-2000, 2000, OC).astype(np.int32)
    cw = _cw(shift, sign, cuda_device)
    ref = np.maximum(oracle.conv2d(x, shift, sign, bias, (1, 1), (1, 1)), 0)
    lib = _ffi.lib()
    counts = []
    for _ in range(3):
        n0 = lib.ds_launch_count()
        out = kernels.conv2d_fused(_t(x, cuda_device), (OC, C, 3, 3), _t(bias, cuda_device), cw, 1, 1,
                                   in_kind=_ffi.IN_I32_CLAMP, act_integer_bits=4, act_fraction_bits=12, relu=True)
        counts.append(lib.ds_launch_count() - n0)
        assert np.array_equal(out.cpu().numpy(), ref)
    assert counts == [3, 1, 1]
    assert len(cw._prepared) == 1 and next(iter(cw._prepared.values())) is not None
    small = kernels.conv2d_fused(_t(x[:1], cuda_device), (OC, C, 3, 3), _t(bias, cuda_device), cw, 1, 1,
                                 in_kind=_ffi.IN_I32_CLAMP, act_integer_bits=4, act_fraction_bits=12, relu=True)
    assert np.array_equal(small.cpu().numpy(), ref[:1])
    assert len(cw._prepared) == 2 and sum(v is None for v in cw._prepared.values()) == 1
    # a buffer that is too small is refused
    f = kernels._fuse(_ffi.IN_I32_CLAMP, _ffi.OUT_I32, 4, 12, act_bits=0, workspace=kernels.workspace(cuda_device))
    tiny = torch.empty(64, dtype=torch.int32, device=cuda_device)
    f.prepared, f.prepared_bytes = tiny.data_ptr(), 256
    need = ctypes.c_longlong(0)
    rc = lib.ds_conv2d_prepare(cw.data.data_ptr(), B, C, H, H, OC, 3, 3, 1, 1, 1, 1, cw.bits, cw.base, f,
                               ctypes.byref(need), torch.cuda.current_stream().cuda_stream)
    assert rc == 6 and need.value > 256


def test_second_device_in_the_same_process(oracle):
    """One process, two GPUs: function attributes, workspaces and prepared weights are kept per
    device (skipped on a single-GPU machine)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from deepshift_b200 import _ffi, kernels
    rng = np.random.default_rng(5)
    x = acts_q16(rng, (10, 16, 28, 28))
    shift, sign = weights(rng, (40, 16, 3, 3))
    bias = rng.integers(-2000, 2000, 40).astype(np.int32)
    ref = np.maximum(oracle.conv2d(x, shift, sign, bias, (1, 1), (1, 1)), 0)
    for dev in (torch.device("cuda", 0), torch.device("cuda", 1), torch.device("cuda", 0)):
        cw = _cw(shift, sign, dev)
        out = kernels.conv2d_fused(_t(x, dev), (40, 16, 3, 3), _t(bias, dev), cw, 1, 1, in_kind=_ffi.IN_I32_CLAMP,
                                   act_integer_bits=4, act_fraction_bits=12, relu=True)
        assert np.array_equal(out.cpu().numpy(), ref)


def test_plain_c_abi_entry_points(oracle, cuda_device):
    """ds_linear_i32 / ds_conv2d_i32 called directly with raw pointers, as a foreign-language
    binding would (no fused options, no workspace)."""
    from deepshift_b200 import _ffi
    lib = _ffi.lib()
    rng = np.random.default_rng(31)
    stream = torch.cuda.current_stream(cuda_device).cuda_stream
    x = acts_q16(rng, (100, 260))
    shift, sign = weights(rng, (70, 260))
    bias = rng.integers(-2000, 2000, 70).astype(np.int32)
    cw = _cw(shift, sign, cuda_device)
    xt, bt = _t(x, cuda_device), _t(bias, cuda_device)
    out = torch.empty((100, 70), dtype=torch.int32, device=cuda_device)
    for act_bits in (0, 16):
        out.fill_(-1)
        assert lib.ds_linear_i32(xt.data_ptr(), cw.data.data_ptr(), bt.data_ptr(), out.data_ptr(), 100, 260, 70,
                                 cw.bits, cw.base, act_bits, stream) == 0
        assert np.array_equal(out.cpu().numpy(), oracle.linear(x, shift, sign, bias))
    x = acts_q16(rng, (6, 32, 14, 14))
    shift, sign = weights(rng, (200, 32, 3, 3))
    bias = rng.integers(-2000, 2000, 200).astype(np.int32)
    cw = _cw(shift, sign, cuda_device)
    xt, bt = _t(x, cuda_device), _t(bias, cuda_device)
    ref = oracle.conv2d(x, shift, sign, bias, (2, 2), (1, 1))
    out = torch.empty(ref.shape, dtype=torch.int32, device=cuda_device)
    for act_bits in (0, 16):
        out.fill_(-1)
        assert lib.ds_conv2d_i32(xt.data_ptr(), cw.data.data_ptr(), bt.data_ptr(), out.data_ptr(), 6, 32, 14, 14, 200,
                                 3, 3, 2, 2, 1, 1, cw.bits, cw.base, act_bits, stream) == 0
        assert np.array_equal(out.cpu().numpy(), ref)
    # misaligned output pointer is refused
    assert lib.ds_conv2d_i32(xt.data_ptr(), cw.data.data_ptr(), None, out.data_ptr() + 4, 6, 32, 14, 14, 200, 3, 3, 2, 2,
                             1, 1, cw.bits, cw.base, 0, stream) == 5


def test_many_items_per_cta_and_single_tile_items(oracle, cuda_device):
    """More output tiles than SMs (each persistent CTA walks several items) with K so short that an
    item is a single k-tile: the producers run two items ahead of the consumers."""
    from deepshift_b200 import kernels
    rng = np.random.default_rng(41)
    B, C, H, OC = 700, 1, 12, 20   # M = 700 * 64 = 44800 rows -> 175 tiles, K = 25
    x = acts_q16(rng, (B, C, H, H))
    shift, sign = weights(rng, (OC, C, 5, 5))
    bias = rng.integers(-2000, 2000, OC).astype(np.int32)
    out = kernels.conv2d(_t(x, cuda_device), _t(shift, cuda_device), None, _t(bias, cuda_device),
                         _cw(shift, sign, cuda_device), 1, 0, act_bits=16)
    assert np.array_equal(out.cpu().numpy(), oracle.conv2d(x, shift, sign, bias, (1, 1), (0, 0)))


def test_random_shapes_against_oracle(oracle, cuda_device):
    """Seeded random convolution and linear shapes (ragged sizes, odd windows, strides, paddings,
    every field width), both arithmetic paths, fused and plain entry points."""
    from deepshift_b200 import _ffi, kernels
    rng = np.random.default_rng(2025)
    for case in range(60):
        lo = int(rng.choice([-1, -3, -7, -15]))
        zeros = bool(rng.integers(0, 2))
        act_bits = int(rng.choice([0, 16]))
        if case % 3 == 0:
            M, K, N = int(rng.integers(1, 400)), int(rng.integers(1, 700)), int(rng.integers(1, 300))
            x = acts_q16(rng, (M, K))
            shift, sign = weights(rng, (N, K), lo, zeros)
            bias = rng.integers(-2000, 2000, N).astype(np.int32)
            out = kernels.linear(_t(x, cuda_device), _t(shift, cuda_device), None, _t(bias, cuda_device),
                                 _cw(shift, sign, cuda_device), act_bits=act_bits)
            assert np.array_equal(out.cpu().numpy(), oracle.linear(x, shift, sign, bias)), (case, M, K, N, lo, zeros)
            continue
        B, C, OC = int(rng.integers(1, 40)), int(rng.integers(1, 70)), int(rng.integers(1, 200))
        kh, kw = int(rng.integers(1, 6)), int(rng.choice([1, 2, 3, 5, 7]))
        sh, sw = int(rng.integers(1, 3)), int(rng.integers(1, 3))
        ph, pw = int(rng.integers(0, kh)), int(rng.integers(0, kw))
        H, W = int(rng.integers(kh, kh + 20)), int(rng.integers(kw, kw + 20))
        x = acts_q16(rng, (B, C, H, W))
        shift, sign = weights(rng, (OC, C, kh, kw), lo, zeros)
        bias = rng.integers(-2000, 2000, OC).astype(np.int32)
        ref = oracle.conv2d(x, shift, sign, bias, (sh, sw), (ph, pw))
        cw = _cw(shift, sign, cuda_device)
        tag = (case, B, C, H, W, OC, kh, kw, sh, sw, ph, pw, lo, zeros, act_bits)
        out = kernels.conv2d(_t(x, cuda_device), _t(shift, cuda_device), None, _t(bias, cuda_device), cw, (sh, sw),
                             (ph, pw), act_bits=act_bits)
        assert np.array_equal(out.cpu().numpy(), ref), tag
        out = kernels.conv2d_fused(_t(x, cuda_device), (OC, C, kh, kw), _t(bias, cuda_device), cw, (sh, sw), (ph, pw),
                                   in_kind=_ffi.IN_I32_CLAMP, out_kind=_ffi.OUT_F32, act_integer_bits=4,
                                   act_fraction_bits=12, relu=True)
        assert np.array_equal(out.cpu().numpy(), oracle.from_fixed(np.maximum(ref, 0), 12)), tag


# ----------------------------------------------------------------------------------------- one integer bit
def test_sign_mode_modules_match_reference_golden(cuda_device, golden_dir):
    """act_integer_bits = 1 (round_to_fixed = sign(x) - 1) on 5x5 and 7x7 windows, where the modules
    quantise in a pass of their own: forward passes recorded from the reference's Conv2dShift and
    Conv2dShiftQ."""
    from deepshift_b200 import modules, modules_q
    g = np.load(os.path.join(golden_dir, "sign_ref.npz"))
    for i in range(int(g["n"])):
        F, st = int(g[f"F{i}"]), int(g[f"stride{i}"])
        if str(g[f"kind{i}"]) == "ps":
            sh = g[f"shift{i}"]
            conv = modules.Conv2dShift(sh.shape[1], sh.shape[0], sh.shape[2], stride=st, padding=0, use_kernel=True,
                                       rounding="deterministic", act_integer_bits=1, act_fraction_bits=F).to(cuda_device)
            conv.shift.data, conv.sign.data = _t(sh, cuda_device), _t(g[f"sign{i}"], cuda_device)
        else:
            w = g[f"w{i}"]
            conv = modules_q.Conv2dShiftQ(w.shape[1], w.shape[0], w.shape[2], stride=st, padding=0, use_kernel=True,
                                          act_integer_bits=1, act_fraction_bits=F).to(cuda_device)
            conv.weight.data = _t(w, cuda_device)
        conv.bias.data = _t(g[f"bias{i}"], cuda_device)
        assert np.array_equal(conv(_t(g[f"x{i}"], cuda_device)).cpu().numpy(), g[f"y{i}"]), i


@pytest.mark.parametrize("F", [7, 12])
def test_sign_mode_on_int32_codes_matches_oracle(oracle, cuda_device, F):
    """One integer bit on the int32 input kinds: DS_IN_I32_CLAMP and `requant` apply
    round_to_fixed(code / 2^F, 1, F) = sign - 1 to codes that have not been quantised yet; a 3x3
    Conv2dShift (quantiser fused into the staging) and LinearShiftQ give the same as the oracle."""
    from deepshift_b200 import _ffi, kernels, modules, modules_q, utils
    rng = np.random.default_rng(100 + F)
    B, C, H, OC = 3, 20, 9, 70
    codes = rng.integers(-3, 4, (B, C, H, H)).astype(np.int32) * rng.integers(1, 1 << 20, (B, C, H, H)).astype(np.int32)
    shift, sign = weights(rng, (OC, C, 3, 3))
    bias = rng.integers(-2000, 2000, OC).astype(np.int32)
    xq = oracle.to_fixed_conv(oracle.from_fixed(codes, F), 1, F)
    assert np.array_equal(xq, np.where(codes > 0, 0, np.where(codes < 0, -(2 << F), -(1 << F))))
    acc = oracle.conv2d(xq, shift, sign, bias, (1, 1), (1, 1))
    rq = np.where(acc > 0, 0, np.where(acc < 0, -(2 << F), -(1 << F))).astype(np.int32)
    cw = _cw(shift, sign, cuda_device)
    out = kernels.conv2d_fused(_t(codes, cuda_device), (OC, C, 3, 3), _t(bias, cuda_device), cw, 1, 1,
                               in_kind=_ffi.IN_I32_CLAMP, act_integer_bits=1, act_fraction_bits=F)
    assert np.array_equal(out.cpu().numpy(), acc)
    out = kernels.conv2d_fused(_t(codes, cuda_device), (OC, C, 3, 3), _t(bias, cuda_device), cw, 1, 1,
                               in_kind=_ffi.IN_I32_CLAMP, act_integer_bits=1, act_fraction_bits=F, requant=True)
    assert np.array_equal(out.cpu().numpy(), rq)
    # modules: fused quantiser (3x3) and the DeepShift-Q linear layer
    xf = rng.normal(0, 1, (B, C, H, H)).astype(np.float32)
    xf[rng.random(xf.shape) < 0.2] = 0.0
    conv = modules.Conv2dShift(C, OC, 3, padding=1, use_kernel=True, rounding="deterministic", act_integer_bits=1,
                               act_fraction_bits=F).to(cuda_device)
    conv.shift.data, conv.sign.data = _t(shift.astype(np.float32), cuda_device), _t(sign.astype(np.float32), cuda_device)
    bi = oracle.to_fixed_conv(conv.bias.data.cpu().numpy(), 1, F)
    ref = oracle.conv2d(oracle.to_fixed_conv(xf, 1, F), shift, sign, bi, (1, 1), (1, 1))
    assert np.array_equal(conv(_t(xf, cuda_device)).cpu().numpy(), oracle.from_fixed(ref, F))
    torch.manual_seed(F)
    lin = modules_q.LinearShiftQ(300, 70, use_kernel=True, act_integer_bits=1, act_fraction_bits=F).to(cuda_device)
    xl = rng.normal(0, 1, (130, 300)).astype(np.float32)
    sh, sg = utils.get_shift_and_sign(lin.weight.data.cpu())
    ref = oracle.linear(oracle.to_fixed_conv(xl, 1, F), sh.numpy().astype(np.int32), sg.numpy().astype(np.int32),
                        oracle.to_fixed_conv(lin.bias.data.cpu().numpy(), 1, F))
    assert np.array_equal(lin(_t(xl, cuda_device)).cpu().numpy(), oracle.from_fixed(ref, F))


def test_global_average_kernel_matches_torch_golden(cuda_device, golden_dir):
    """ds_avgpool_fix_i32 against torch's CPU adaptive_avg_pool2d followed by the LinearShift entry
    conversion, recorded in gap_ref.npz."""
    from deepshift_b200 import kernels
    g = np.load(os.path.join(golden_dir, "gap_ref.npz"))
    for i in range(int(g["n"])):
        got = kernels.avgpool_fix_i32(_t(g[f"codes{i}"], cuda_device), int(g["F"]))
        assert np.array_equal(got.cpu().numpy(), g[f"fixed{i}"]), i


def test_residual_may_alias_the_output(oracle, cuda_device):
    """An in-place residual add (residual == out) on a shape that would otherwise be split along K
    through the zeroed output."""
    from deepshift_b200 import _ffi, kernels
    rng = np.random.default_rng(515)
    B, C, H, OC = 5, 128, 7, 130
    x = acts_q16(rng, (B, C, H, H))
    shift, sign = weights(rng, (OC, C, 3, 3))
    bias = rng.integers(-2000, 2000, OC).astype(np.int32)
    res = rng.integers(-50000, 50000, (B, OC, H, H)).astype(np.int32)
    ref = oracle.conv2d(x, shift, sign, bias, (1, 1), (1, 1))
    ref = (ref.astype(np.float32) + res.astype(np.float32)).astype(np.int64).astype(np.int32)
    cw = _cw(shift, sign, cuda_device)
    counters = torch.zeros(16384, dtype=torch.int32, device=cuda_device)   # counters only: the atomics scheme
    xd, bd = _t(x, cuda_device), _t(bias, cuda_device)
    for ws in (None, counters):
        buf = _t(res, cuda_device)
        f = kernels._fuse(_ffi.IN_I32_CLAMP, _ffi.OUT_I32, 4, 12, residual=buf, workspace=ws)
        rc = _ffi.lib().ds_conv2d_ex(xd.data_ptr(), cw.data.data_ptr(), bd.data_ptr(),
                                     buf.data_ptr(), B, C, H, H, OC, 3, 3, 1, 1, 1, 1, cw.bits, cw.base, f,
                                     torch.cuda.current_stream(cuda_device).cuda_stream)
        assert rc == 0
        torch.cuda.synchronize(cuda_device)
        assert np.array_equal(buf.cpu().numpy(), ref)


def test_two_streams_run_side_by_side(oracle, cuda_device):
    """Two different convolutions issued on two streams with nothing ordering them: each stream has
    its own scratch memory, so both results are exact (shapes that share tiles along K)."""
    from deepshift_b200 import kernels
    rng = np.random.default_rng(909)
    cases = []
    for (B, C, H, OC) in [(5, 128, 7, 130), (49, 32, 28, 100)]:
        x = acts_q16(rng, (B, C, H, H))
        shift, sign = weights(rng, (OC, C, 3, 3))
        bias = rng.integers(-2000, 2000, OC).astype(np.int32)
        cases.append((_t(x, cuda_device), _t(shift, cuda_device), _t(bias, cuda_device), _cw(shift, sign, cuda_device),
                      oracle.conv2d(x, shift, sign, bias, (1, 1), (1, 1))))
    streams = [torch.cuda.Stream(device=cuda_device) for _ in cases]
    torch.cuda.synchronize(cuda_device)
    assert kernels.workspace(cuda_device, streams[0]).data_ptr() != kernels.workspace(cuda_device, streams[1]).data_ptr()
    outs = [[], []]
    for _ in range(6):
        for i, (x, shift, bias, cw, _) in enumerate(cases):
            with torch.cuda.stream(streams[i]):
                outs[i].append(kernels.conv2d(x, shift, None, bias, cw, 1, 1, act_bits=16))
    torch.cuda.synchronize(cuda_device)
    for i, c in enumerate(cases):
        for o in outs[i]:
            assert np.array_equal(o.cpu().numpy(), c[4]), i
    assert kernels.last_kernel_error() == 0


def test_ps_module_repacks_when_parameters_change(oracle, cuda_device):
    """forward, load_state_dict, forward: the second pass uses the loaded weights (the packed copy
    is keyed on the parameters' versions), and equals a module built fresh from them."""
    from deepshift_b200 import modules
    rng = np.random.default_rng(31)
    kw = dict(use_kernel=True, rounding="deterministic", act_integer_bits=4, act_fraction_bits=12)
    a = modules.Conv2dShift(8, 40, 3, padding=1, **kw).to(cuda_device)
    b = modules.Conv2dShift(8, 40, 3, padding=1, **kw).to(cuda_device)
    for m in (a, b):
        shift, sign = weights(rng, (40, 8, 3, 3))
        m.shift.data, m.sign.data = _t(shift.astype(np.float32), cuda_device), _t(sign.astype(np.float32), cuda_device)
    x = _t(rng.normal(0, 1, (2, 8, 10, 10)).astype(np.float32), cuda_device)
    ya, yb = a(x), b(x)
    assert not torch.equal(ya, yb)
    a.load_state_dict(b.state_dict())
    assert torch.equal(a(x), yb)
    with torch.no_grad():
        a.sign.neg_()                        # in place on the parameter: its version counter moves
    fresh = modules.Conv2dShift(8, 40, 3, padding=1, **kw).to(cuda_device)
    fresh.load_state_dict(a.state_dict())
    assert torch.equal(a(x), fresh(x)) and not torch.equal(a(x), yb)
    lin = modules.LinearShift(30, 70, **kw).to(cuda_device)
    xl = _t(rng.normal(0, 1, (65, 30)).astype(np.float32), cuda_device)
    y0 = lin(xl)
    with torch.no_grad():
        lin.shift.sub_(1.0)
    assert not torch.equal(lin(xl), y0)


@pytest.mark.parametrize("M", [1, 3, 8, 16, 23, 64])
def test_small_batch_linear_with_fused_epilogue(oracle, cuda_device, M):
    """Small batches (the kernels that split K across lanes / across CTAs) with everything fused:
    LinearShift's fp32 entry conversion on read, residual add, ReLU, fp32 output."""
    from deepshift_b200 import _ffi, kernels
    rng = np.random.default_rng(600 + M)
    K, N, F = 515, 130, 12
    xf = rng.normal(0, 4, (M, K)).astype(np.float32)
    shift, sign = weights(rng, (N, K))
    bias = rng.integers(-2000, 2000, N).astype(np.int32)
    res = rng.integers(-50000, 50000, (M, N)).astype(np.int32)
    acc = oracle.linear(oracle.to_fixed_linear(xf, F), shift, sign, bias)
    ref = np.maximum(acc.astype(np.float32) + res.astype(np.float32), 0).astype(np.int64).astype(np.int32)
    out = kernels.linear_fused(_t(xf, cuda_device), N, _t(bias, cuda_device), _cw(shift, sign, cuda_device),
                               in_kind=_ffi.IN_F32_LINEAR, out_kind=_ffi.OUT_F32, act_integer_bits=4,
                               act_fraction_bits=F, relu=True, residual=_t(res, cuda_device))
    assert np.array_equal(out.cpu().numpy(), oracle.from_fixed(ref, F))


def test_reference_binding_stub_against_the_library(oracle, cuda_device):
    """deepshift_b200/reference_binding/deepshift_cuda.py, the module a maintainer of the reference
    tree puts in place of the pybind extension: its three functions, called the way
    deepshift/kernels/kernels.py:10-74 calls them (zeroed outputs, input padded with F.pad, a zero
    bias when there is none), reproduce the oracle."""
    import importlib.util
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "deepshift_b200",
                        "reference_binding", "deepshift_cuda.py")
    spec = importlib.util.spec_from_file_location("deepshift_cuda_stub", path)
    stub = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(stub)
    rng = np.random.default_rng(808)
    # COMPRESS_SIGN_SHIFT as utils.py:74-86 / kernels.py:69-74 use it
    OC, C, k = 37, 6, 3
    shift, sign = weights(rng, (OC, C, k, k), zeros=False)
    bits, num = 4, 6
    row = (C * k * k + num - 1) // num
    packed = torch.zeros([row * OC], dtype=torch.int32, device=cuda_device)
    stub.COMPRESS_SIGN_SHIFT(_t(-shift, cuda_device), _t(sign, cuda_device), packed, 0, bits, OC, C, k, k, row, num)
    assert np.array_equal(packed.cpu().numpy().reshape(OC, row), oracle.compress(-shift.reshape(OC, -1), sign.reshape(OC, -1), bits, 0))
    # DEEP_SHIFT_CONV on the tensor kernels.py:32-36 has padded
    x = acts_wide(rng, (2, C, 9, 11), 20)
    bias = rng.integers(-2000, 2000, OC).astype(np.int32)
    xp = torch.nn.functional.pad(_t(x, cuda_device), (1, 1, 1, 1), mode='constant', value=0)
    out = torch.zeros([2, OC, (xp.size(2) - k) // 2 + 1, (xp.size(3) - k) // 2 + 1], dtype=torch.int32, device=cuda_device)
    stub.DEEP_SHIFT_CONV(xp, packed, _t(bias, cuda_device), out, (2, 2), (1, 1, 1, 1), k, k, 0, bits)
    assert np.array_equal(out.cpu().numpy(), oracle.conv2d(x, shift, sign, bias, (2, 2), (1, 1)))
    # DEEP_SHIFT_LINEAR
    M, K, N = 70, 131, 29
    xl = acts_wide(rng, (M, K), 24)
    sl, gl = weights(rng, (N, K))
    cw = _cw(sl, gl, cuda_device)
    outl = torch.zeros([M, N], dtype=torch.int32, device=cuda_device)
    zero_bias = torch.zeros([N], dtype=torch.int32, device=cuda_device)
    stub.DEEP_SHIFT_LINEAR(_t(xl, cuda_device), cw.data, zero_bias, outl, cw.base, cw.bits, N)
    assert np.array_equal(outl.cpu().numpy(), oracle.linear(xl, sl, gl, None))


def test_act_bits_auto_picks_the_path_by_looking_at_the_data(oracle, cuda_device):
    """The reference signature makes no promise about the activations' range.  By default the
    library measures it on the device and enqueues both arithmetic paths, each gated on the result:
    16-bit activations run on the FP32 pipe, wider ones on the integer pipe, both exact."""
    from deepshift_b200 import kernels
    rng = np.random.default_rng(2718)
    B, C, H, OC = 6, 16, 28, 40
    shift, sign = weights(rng, (OC, C, 3, 3))
    bias = rng.integers(-2000, 2000, OC).astype(np.int32)
    cw = _cw(shift, sign, cuda_device)
    for x, flag in ((acts_q16(rng, (B, C, H, H)), 0), (acts_wide(rng, (B, C, H, H), 24), 1)):
        ref = oracle.conv2d(x, shift, sign, bias, (1, 1), (1, 1))
        out = kernels.conv2d(_t(x, cuda_device), _t(shift, cuda_device), None, _t(bias, cuda_device), cw, 1, 1)
        assert np.array_equal(out.cpu().numpy(), ref)
        assert int(kernels.workspace(cuda_device)[16383]) == flag
    M, K, N = 300, 512, 200
    sl, gl = weights(rng, (N, K))
    cwl = _cw(sl, gl, cuda_device)
    for x, flag in ((acts_q16(rng, (M, K)), 0), (acts_wide(rng, (M, K), 24), 1)):
        out = kernels.linear(_t(x, cuda_device), _t(sl, cuda_device), None, None, cwl)
        assert np.array_equal(out.cpu().numpy(), oracle.linear(x, sl, gl, None))
        assert int(kernels.workspace(cuda_device)[16383]) == flag
    assert int(kernels.workspace(cuda_device)[:16383].abs().sum()) == 0


def test_unoptimized_fp32_baseline_matches_torch(cuda_device):
    """The reference's fp32 strawman (unoptimized/): results agree with a float64 evaluation of
    torch.nn.functional to fp32 rounding (tolerance 1e-5 of the largest output: sums of a few hundred
    products)."""
    from deepshift_b200 import unoptimized as U
    torch.manual_seed(5)
    for (B, C, H, W, OC, k, s, p) in [(2, 3, 17, 13, 20, 3, 1, 1), (3, 8, 9, 9, 33, 5, 2, 2), (2, 16, 7, 7, 40, 1, 1, 0)]:
        x = torch.randn(B, C, H, W, device=cuda_device)
        w = torch.randn(OC, C, k, k, device=cuda_device) * 0.1
        b = torch.randn(OC, device=cuda_device)
        ref = torch.nn.functional.conv2d(x.double(), w.double(), b.double(), s, p)   # float64: torch's fp32 path may use TF32
        got = U.conv2d(x, w, b, (s, s), (p, p))
        assert got.shape == ref.shape and float((got.double() - ref).abs().max()) <= 1e-5 * float(ref.abs().max())
    x, w = torch.randn(70, 301, device=cuda_device), torch.randn(45, 301, device=cuda_device)
    ref = torch.nn.functional.linear(x.double(), w.double())
    assert float((U.linear(x, w, None).double() - ref).abs().max()) <= 1e-5 * float(ref.abs().max())
    model = torch.nn.Sequential(torch.nn.Conv2d(3, 8, 3, padding=1), torch.nn.ReLU(), torch.nn.Flatten(),
                                torch.nn.Linear(8 * 6 * 6, 10)).to(cuda_device)
    xin = torch.randn(4, 3, 6, 6, device=cuda_device)
    with torch.no_grad():
        want = model.double()(xin.double())
        got = U.convert_to_unoptimized(model.float())(xin)
    assert isinstance(model[0], U.UnoptimizedConv2d) and isinstance(model[3], U.UnoptimizedLinear)
    assert float((got.double() - want).abs().max()) <= 1e-5 * float(want.abs().max())


@pytest.mark.parametrize("shape", [(3, 16, 12, 24, 3, 1, 1), (40, 64, 28, 128, 3, 1, 1), (9, 32, 14, 64, 1, 2, 0),
                                   (2, 3, 32, 16, 7, 2, 3)], ids=["small", "ws3x3", "ws1x1s2", "stem7x7"])
def test_module_fusion_hints_equal_the_unfused_ops(oracle, cuda_device, shape):
    """`forward(x, residual=r, relu=True)` of the shift modules equals `F.relu(forward(x) + r)` bit for
    bit: arbitrary fp32 residuals (not just fixed-point values), every kernel the convolution can
    land on, and against the oracle's integer sums."""
    from deepshift_b200 import modules
    B, C, H, OC, k, s, p = shape
    I, F = 4, 12
    rng = np.random.default_rng(sum(shape))
    conv = modules.Conv2dShift(C, OC, k, s, p, use_kernel=True, act_integer_bits=I, act_fraction_bits=F).to(cuda_device)
    shift, sign = weights(rng, (OC, C, k, k), lo=-14)
    with torch.no_grad():
        conv.shift.copy_(_t(shift.astype(np.float32), cuda_device))
        conv.sign.copy_(_t(sign.astype(np.float32), cuda_device))
    x = _t(rng.normal(0, 2, (B, C, H, H)).astype(np.float32), cuda_device)
    with torch.no_grad():
        plain = conv(x)
        r = _t(rng.normal(0, 3, tuple(plain.shape)).astype(np.float32), cuda_device)
        assert torch.equal(conv(x, residual=r, relu=True), torch.relu(plain + r))
        assert torch.equal(conv(x, residual=r), plain + r)
        assert torch.equal(conv(x, relu=True), torch.relu(plain))
    bias = oracle.to_fixed_conv(conv.bias.data.cpu().numpy(), I, F)
    ref = oracle.conv2d(oracle.to_fixed_conv(x.cpu().numpy(), I, F), shift, sign, bias, (s, s), (p, p))
    want = np.maximum(oracle.from_fixed(ref, F) + r.cpu().numpy(), np.float32(0))
    assert np.array_equal(conv(x, residual=r, relu=True).cpu().numpy(), want)


@pytest.mark.parametrize("M", [1, 5, 16, 40, 300])
def test_linear_module_fusion_hints(oracle, cuda_device, M):
    """The same hints on LinearShift / LinearShiftQ, on every linear kernel (M <= 16, <= 64, larger)."""
    from deepshift_b200 import modules, modules_q
    rng = np.random.default_rng(M)
    K, N = 256, 48
    x = _t(rng.normal(0, 1, (M, K)).astype(np.float32), cuda_device)
    r = _t(rng.normal(0, 2, (M, N)).astype(np.float32), cuda_device)
    lin = modules.LinearShift(K, N, use_kernel=True, act_integer_bits=4, act_fraction_bits=12).to(cuda_device)
    linq = modules_q.LinearShiftQ(K, N, use_kernel=True, act_integer_bits=4, act_fraction_bits=12).to(cuda_device)
    with torch.no_grad():
        for m in (lin, linq):
            plain = m(x)
            assert torch.equal(m(x, residual=r, relu=True), torch.relu(plain + r))
            assert torch.equal(m(x, relu=True), torch.relu(plain))


def test_add_relu_glue_kernel(cuda_device):
    """ds_add_relu_f32: in place, equal to the torch ops bit for bit, ragged and unaligned lengths,
    NaN kept, nothing written beyond n."""
    from deepshift_b200 import kernels
    rng = np.random.default_rng(5)
    for n, off in [(1, 0), (7, 0), (4096, 0), (100003, 1), (64, 3)]:
        base = _t(rng.normal(0, 1, n + off + 8).astype(np.float32), cuda_device)
        r = _t(rng.normal(0, 1, n).astype(np.float32), cuda_device)
        y = base[off:off + n]
        want = torch.relu(y + r)
        tail = base[off + n:].clone()
        kernels.add_relu_f32_(y, r, relu=True)
        assert torch.equal(y, want) and torch.equal(base[off + n:], tail)
    y = _t(np.array([np.nan, -1.0, 2.0, -0.5], np.float32), cuda_device)
    kernels.add_relu_f32_(y, None, relu=True)
    out = y.cpu().numpy()
    assert np.isnan(out[0]) and np.array_equal(out[1:], np.array([0, 2, 0], np.float32))
    with pytest.raises(RuntimeError):
        kernels.add_relu_f32_(y, torch.zeros(5, device=cuda_device), relu=True)


@pytest.mark.parametrize("shape,k,s,p", [((3, 5, 32, 32), 3, 2, 1), ((2, 4, 112, 112), 3, 2, 1), ((2, 3, 28, 28), 2, 2, 0),
                                         ((2, 3, 15, 13), 3, 1, 1), ((1, 2, 9, 9), 3, 2, 1), ((2, 2, 24, 24), 5, 3, 2)])
def test_fp32_max_pool_glue_equals_torch(cuda_device, shape, k, s, p):
    """ds_maxpool2d_f32 against F.max_pool2d, bit for bit: the four-outputs-per-thread kernel of the stem's
    pool (W a multiple of 8) and the general one, negative values at the padded border, a NaN."""
    import torch.nn.functional as F
    from deepshift_b200 import kernels
    rng = np.random.default_rng(sum(shape) + k)
    x = _t(rng.normal(-3, 2, shape).astype(np.float32), cuda_device)   # mostly negative: padding must not win
    assert torch.equal(kernels.maxpool2d_f32(x, k, s, p), F.max_pool2d(x, k, s, p))
    x[0, 0, 1, 2] = float('nan')
    got, want = kernels.maxpool2d_f32(x, k, s, p), F.max_pool2d(x, k, s, p)
    assert torch.equal(torch.isnan(got), torch.isnan(want)) and torch.equal(torch.nan_to_num(got), torch.nan_to_num(want))
