"""The CPU oracle against the reference: golden vectors produced by the reference's compiled CPU
kernel and Python package (tests/golden/make_golden.py), and the compiled kernel itself when it
is present (oracle/_ref)."""
import os

import numpy as np
import pytest

from helpers import acts_q16, acts_wide, weights


def test_linear_matches_reference_golden(oracle, golden_dir):
    g = np.load(os.path.join(golden_dir, "linear_ref.npz"))
    for i in range(int(g["n"])):
        out = oracle.linear(g[f"x{i}"], g[f"shift{i}"], g[f"sign{i}"], g[f"bias{i}"])
        assert np.array_equal(out, g[f"y{i}"]), i


def test_conv_matches_reference_golden(oracle, golden_dir):
    g = np.load(os.path.join(golden_dir, "conv_ref.npz"))
    for i in range(int(g["n"])):
        st, pad = tuple(g[f"stride{i}"]), tuple(g[f"pad{i}"])
        # the reference conv kernel adds a zero-sign weight as +1 (shift_cpu.cpp:351-353)
        out = oracle.conv2d(g[f"x{i}"], g[f"shift{i}"], g[f"sign{i}"], g[f"bias{i}"], st, pad,
                            zero_sign_as_plus=True)
        assert np.array_equal(out, g[f"y{i}"]), i
        if not (g[f"sign{i}"] == 0).any():
            canon = oracle.conv2d(g[f"x{i}"], g[f"shift{i}"], g[f"sign{i}"], g[f"bias{i}"], st, pad)
            assert np.array_equal(canon, g[f"y{i}"]), i


def test_float_glue_matches_reference_golden(oracle, golden_dir):
    g = np.load(os.path.join(golden_dir, "glue_ref.npz"))
    for I, F in [(4, 12), (16, 16), (8, 8), (1, 7), (2, 3)]:
        assert np.array_equal(oracle.round_to_fixed(g["rtf_in"], I, F), g[f"rtf_{I}_{F}"]), (I, F)
    # LinearShift(use_kernel=True, use_cuda=False) of the reference
    xi = oracle.to_fixed_linear(g["lin_x"], 12)
    bi = oracle.to_fixed_linear(g["lin_bias"], 12)
    y = oracle.from_fixed(oracle.linear(xi, g["lin_shift"].astype(np.int32), g["lin_sign"].astype(np.int32), bi), 12)
    assert np.array_equal(y, g["lin_y"])
    # Conv2dShift(use_kernel=True, use_cuda=False, padding=0) of the reference
    xi = oracle.to_fixed_conv(g["conv_x"], 4, 12)
    bi = oracle.to_fixed_conv(g["conv_bias"], 4, 12)
    y = oracle.from_fixed(oracle.conv2d(xi, g["conv_shift"].astype(np.int32), g["conv_sign"].astype(np.int32), bi), 12)
    assert np.array_equal(y, g["conv_y"])


def test_sign_mode_modules_of_the_reference_match_the_oracle(oracle, golden_dir):
    """act_integer_bits = 1: round_to_fixed is sign(x) - 1 (utils.py:12-13), codes -2^(F+1), -2^F, 0.
    Forward passes of the reference's Conv2dShift and Conv2dShiftQ (5x5 and 7x7 windows) restated."""
    import torch
    from deepshift_b200 import utils
    g = np.load(os.path.join(golden_dir, "sign_ref.npz"))
    for i in range(int(g["n"])):
        F, st = int(g[f"F{i}"]), int(g[f"stride{i}"])
        if str(g[f"kind{i}"]) == "ps":
            shift, sign = g[f"shift{i}"].astype(np.int32), g[f"sign{i}"].astype(np.int32)
        else:
            w = utils.clampabs(torch.from_numpy(g[f"w{i}"].copy()), 2.0 ** -15, 1.0)
            sh, sg = utils.get_shift_and_sign(w)
            shift, sign = sh.numpy().astype(np.int32), sg.numpy().astype(np.int32)
        xi = oracle.to_fixed_conv(g[f"x{i}"], 1, F)
        assert set(np.unique(xi)) <= {-(2 << F), -(1 << F), 0}
        ref = oracle.conv2d(xi, shift, sign, oracle.to_fixed_conv(g[f"bias{i}"], 1, F), (st, st), (0, 0))
        assert np.array_equal(oracle.from_fixed(ref, F), g[f"y{i}"]), i


def test_global_average_glue_matches_torch_golden(oracle, golden_dir):
    """The pooling glue between the last convolution and the classifier: torch's CPU
    adaptive_avg_pool2d followed by the LinearShift entry conversion (modules.py:25)."""
    g = np.load(os.path.join(golden_dir, "gap_ref.npz"))
    F = int(g["F"])
    for i in range(int(g["n"])):
        x = oracle.from_fixed(g[f"codes{i}"], F)
        pooled = oracle.global_avg(x)
        assert np.array_equal(pooled, g[f"pooled{i}"]), i
        assert np.array_equal(oracle.to_fixed_linear(pooled, F), g[f"fixed{i}"]), i


def test_against_compiled_reference_when_present(oracle):
    if oracle.ref_module() is None:
        pytest.skip("oracle/_ref not built (reference checkout not mounted)")
    rng = np.random.default_rng(11)
    for M, K, N in [(5, 33, 7), (64, 300, 20)]:
        x = acts_wide(rng, (M, K))
        shift, sign = weights(rng, (N, K), -31)
        bias = rng.integers(-5000, 5000, N).astype(np.int32)
        assert np.array_equal(oracle.linear(x, shift, sign, bias), oracle.ref_linear(x, shift, sign, bias))
    x = acts_q16(rng, (2, 5, 11, 9))
    shift, sign = weights(rng, (6, 5, 3, 3), -15, zeros=False)
    bias = rng.integers(-5000, 5000, 6).astype(np.int32)
    for st in [(1, 1), (2, 2), (1, 2)]:
        ref = oracle.ref_conv2d_prepadded(oracle.pad_nchw(x, 1, 1), shift, sign, bias, st)
        assert np.array_equal(oracle.conv2d(x, shift, sign, bias, st, (1, 1)), ref)


@pytest.mark.parametrize("stride,pad,k", [((1, 1), (1, 1), 3), ((2, 2), (1, 1), 3), ((2, 2), (3, 3), 7),
                                          ((1, 1), (0, 0), 5), ((2, 2), (0, 0), 1), ((2, 1), (1, 2), 3)])
def test_direct_conv_equals_im2col_gemm(oracle, stride, pad, k):
    """The reference's CUDA decomposition (IM2COL, GEMM, COL2IM) and its CPU direct convolution
    compute the same thing, zero signs included, under the canonical rule."""
    rng = np.random.default_rng(k * 100 + stride[0])
    x = acts_q16(rng, (3, 4, 10, 9))
    shift, sign = weights(rng, (5, 4, k, k))
    bias = rng.integers(-3000, 3000, 5).astype(np.int32)
    a = oracle.conv2d(x, shift, sign, bias, stride, pad)
    b = oracle.conv2d_via_gemm(x, shift, sign, bias, stride, pad)
    assert np.array_equal(a, b)


@pytest.mark.parametrize("lo", [-1, -3, -7, -15, -31])
@pytest.mark.parametrize("zeros", [False, True])
def test_packed_decode_equals_unpacked(oracle, lo, zeros):
    rng = np.random.default_rng(-lo + 50 * zeros)
    M, K, N = 9, 37, 11
    x = acts_wide(rng, (M, K), 20)
    shift, sign = weights(rng, (N, K), lo, zeros)
    bias = rng.integers(-100, 100, N).astype(np.int32)
    packed, base, bits = oracle.compress_bits(shift, sign)
    assert base == 0
    assert bits == (6 if zeros else max(1, int(-lo).bit_length()))
    num = 32 // (bits + 1)
    assert packed.shape == (N, (K + num - 1) // num)
    assert np.array_equal(oracle.linear_packed(x, packed, bias, K, bits, base), oracle.linear(x, shift, sign, bias))


def test_packing_layout_bit_by_bit(oracle):
    """Field i of a word sits at bits [i*(bits+1), i*(bits+1)+bits), its sign bit above it; unused
    slots are zero (shift.cu:27-38)."""
    shiftp = np.array([[3, 0, 7, 1, 5]], dtype=np.int32)
    sign = np.array([[1, -1, 1, 0, -1]], dtype=np.int32)
    packed = oracle.compress(shiftp, sign, bits=3, base=0)
    assert packed.shape == (1, 1)
    w = int(np.uint32(packed[0, 0]))
    fields = [(w >> (4 * i)) & 0xF for i in range(8)]
    assert fields[:5] == [3 | 8, 0, 7 | 8, 1, 5] and fields[5:] == [0, 0, 0]


def test_left_shift_base(oracle):
    """A positive shift (multiply by 2^s) is stored with a negative base; decoding gives
    x << s with the CPU kernel's semantics."""
    rng = np.random.default_rng(5)
    x = acts_wide(rng, (4, 10), 12)
    shift = rng.integers(-5, 4, (3, 10)).astype(np.int32)
    shift[0, 0] = 3
    sign = rng.choice([-1, 1], (3, 10)).astype(np.int32)
    packed, base, bits = oracle.compress_bits(shift, sign)
    assert base == -3
    assert np.array_equal(oracle.linear_packed(x, packed, None, 10, bits, base), oracle.linear(x, shift, sign, None))


def test_wraparound_is_modulo_2_32(oracle):
    x = np.full((1, 4), 2**30, dtype=np.int32)
    shift = np.zeros((1, 4), dtype=np.int32)
    sign = np.ones((1, 4), dtype=np.int32)
    assert oracle.linear(x, shift, sign, None)[0, 0] == 0  # 4 * 2^30 wraps to 0


def test_empty_batch(oracle):
    out = oracle.linear(np.zeros((0, 5), np.int32), np.zeros((3, 5), np.int32), np.ones((3, 5), np.int32), None)
    assert out.shape == (0, 3)
