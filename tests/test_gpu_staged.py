"""The TMA-fed convolution on staged activations (fp32 NHWC operands with a halo) against the CPU
oracle: bit-identical integer results, whatever the output form."""
import numpy as np
import pytest
import torch

from helpers import acts_q16, weights

pytestmark = pytest.mark.gpu


def _cw(shift, sign, dev):
    from deepshift_b200 import utils
    return utils.compress_bits(torch.from_numpy(shift).float(), torch.from_numpy(sign).float(), device=dev)


def _t(a, dev):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


def _nhwc(a):
    return np.ascontiguousarray(np.transpose(a, (0, 2, 3, 1)))


STAGED_CASES = [  # B, C, H, W, OC, KH, KW, stride, pad, halo
    (2, 3, 8, 8, 4, 3, 3, 1, 1, 1),          # tiny, C padded to 4, one partial tile
    (2, 4, 9, 7, 5, 3, 3, 2, 1, 1),          # stride 2, odd sizes, OC not a multiple of 4
    (1, 1, 12, 12, 6, 5, 5, 1, 0, 0),        # no padding, no halo
    (2, 3, 30, 30, 64, 7, 7, 2, 3, 3),       # the stem's window
    (3, 64, 14, 14, 128, 1, 1, 2, 0, 1),     # 1x1 stride 2 reading a tensor with a halo it does not use
    (4, 64, 7, 7, 64, 3, 3, 1, 1, 1),        # 512 x 64 tile
    (5, 128, 7, 7, 130, 3, 3, 1, 1, 2),      # two column tiles, the second nearly empty; halo wider than the padding
    (3, 20, 11, 13, 70, 3, 3, 1, 1, 1),      # rows wrap inside a 256-position box many times
    (2, 6, 10, 10, 70, 5, 5, 1, 2, 2),
    (40, 32, 28, 28, 64, 3, 3, 1, 1, 1),     # 62 tiles of 512 rows
    (49, 32, 28, 28, 100, 3, 3, 1, 1, 1),    # 151 tiles on 148 SMs: the tail is shared along K
]


@pytest.mark.parametrize("case", STAGED_CASES, ids=[str(c) for c in STAGED_CASES])
def test_staged_conv_matches_oracle(oracle, cuda_device, case):
    from deepshift_b200 import staged
    B, C, H, W, OC, KH, KW, s, p, halo = case
    rng = np.random.default_rng(sum(case))
    x = acts_q16(rng, (B, C, H, W))
    shift, sign = weights(rng, (OC, C, KH, KW))
    bias = rng.integers(-2000, 2000, OC).astype(np.int32)
    ref = oracle.conv2d(x, shift, sign, bias, (s, s), (p, p))
    OH, OW = ref.shape[2], ref.shape[3]
    cw = _cw(shift, sign, cuda_device)
    from deepshift_b200 import _ffi
    xs = staged.stage_nchw(_t(x, cuda_device), 4, 12, halo, in_kind=_ffi.IN_I32)
    assert torch.equal(xs.codes().cpu(), torch.from_numpy(x))
    codes = torch.full((B, OH, OW, OC), 7, dtype=torch.int32, device=cuda_device)
    nchw = torch.full((B, OC, OH, OW), 7, dtype=torch.int32, device=cuda_device)
    f32 = torch.full((B, OH, OW, OC), 7, dtype=torch.float32, device=cuda_device)
    for _ in range(2):   # twice: arrival counters of the shared tiles return to zero
        staged.conv2d(xs, (OC, C, KH, KW), _t(bias, cuda_device), cw, s, p, out_codes=codes, out_nchw=nchw, out_f32=f32)
        assert np.array_equal(nchw.cpu().numpy(), ref)
        assert np.array_equal(codes.cpu().numpy(), _nhwc(ref))
        assert np.array_equal(f32.cpu().numpy(), oracle.from_fixed(_nhwc(ref), 12))


def test_staged_chain_with_residual_relu_and_requantised_operand(oracle, cuda_device):
    """Two convolutions chained through the staged operand the first one writes (clamp of the 4.12
    quantiser + 0.5 into the interior of a tensor with a halo), residual add, ReLU and the fp32
    rounding of large sums; fp32 input quantised while it is staged."""
    from deepshift_b200 import staged
    rng = np.random.default_rng(4242)
    B, C, H, OC = 3, 16, 12, 72
    xf = (rng.normal(0, 3, (B, C, H, H))).astype(np.float32)
    s1, g1 = weights(rng, (OC, C, 3, 3), lo=-3)    # small shifts: sums beyond the clamp and beyond 2^24
    s2, g2 = weights(rng, (OC, OC, 3, 3), lo=-2)
    b1 = rng.integers(-2000, 2000, OC).astype(np.int32)
    b2 = rng.integers(-2000, 2000, OC).astype(np.int32)
    res = (rng.integers(-50000, 50000, (B, OC, H, H)) * 400).astype(np.int32)
    xi = oracle.to_fixed_conv(xf, 4, 12)
    a1 = oracle.conv2d(xi, s1, g1, b1, (1, 1), (1, 1))
    v1 = np.maximum(a1.astype(np.float32) + res.astype(np.float32), 0).astype(np.int64).astype(np.int32)
    v1 = v1.astype(np.float32).astype(np.int64).astype(np.int32)                 # round_f32
    a2 = oracle.conv2d(np.clip(v1, -32768, 28672), s2, g2, b2, (1, 1), (1, 1))
    assert np.abs(v1).max() > 2 ** 24 and (v1 > 28672).any()
    xs = staged.stage_nchw(_t(xf, cuda_device), 4, 12, halo=1)
    assert np.array_equal(xs.codes().cpu().numpy(), xi)
    mid = staged.StagedTensor(B, H, H, OC, 1, cuda_device)
    mid_codes = torch.empty((B, H, H, OC), dtype=torch.int32, device=cuda_device)
    staged.conv2d(xs, (OC, C, 3, 3), _t(b1, cuda_device), _cw(s1, g1, cuda_device), 1, 1, relu=True, round_f32=True,
                  residual=_t(_nhwc(res), cuda_device), out_codes=mid_codes, out_staged=mid)
    assert np.array_equal(mid_codes.cpu().numpy(), _nhwc(v1))
    assert np.array_equal(mid.codes().cpu().numpy(), np.clip(v1, -32768, 28672))
    h = mid.data.cpu().numpy()
    assert (h[:, 0] == 0.5).all() and (h[:, :, 0] == 0.5).all() and (h[:, -1] == 0.5).all() and (h[:, :, -1] == 0.5).all()
    out = torch.empty((B, OC, H, H), dtype=torch.float32, device=cuda_device)
    staged.conv2d(mid, (OC, OC, 3, 3), _t(b2, cuda_device), _cw(s2, g2, cuda_device), 1, 1, out_nchw=out)
    assert np.array_equal(out.cpu().numpy(), oracle.from_fixed(a2, 12))


def test_nhwc_pooling_matches_oracle(oracle, cuda_device, golden_dir):
    import ctypes
    import os
    from deepshift_b200 import _ffi, staged
    rng = np.random.default_rng(99)
    B, C, H, W = 3, 24, 13, 10
    x = (acts_q16(rng, (B, C, H, W)) * 3).astype(np.int32)
    lib, st = _ffi.lib(), torch.cuda.current_stream(cuda_device).cuda_stream
    xd = _t(_nhwc(x), cuda_device)
    for (k, s, p) in [(3, 2, 1), (2, 2, 0)]:
        OH, OW = (H + 2 * p - k) // s + 1, (W + 2 * p - k) // s + 1
        ref = torch.nn.functional.max_pool2d(torch.from_numpy(x).float(), k, s, p).numpy().astype(np.int32)
        codes = torch.empty((B, OH, OW, C), dtype=torch.int32, device=cuda_device)
        op = staged.StagedTensor(B, OH, OW, C, 1, cuda_device)
        assert lib.ds_maxpool_nhwc(xd.data_ptr(), B, H, W, C, k, s, p, codes.data_ptr(), ctypes.byref(op.c), 4, 12, st) == 0
        assert np.array_equal(codes.cpu().numpy(), _nhwc(ref))
        assert np.array_equal(op.codes().cpu().numpy(), np.clip(ref, -32768, 28672))
    g = np.load(os.path.join(golden_dir, "gap_ref.npz"))
    for i in range(int(g["n"])):
        c = g[f"codes{i}"]
        out = torch.empty(c.shape[:2], dtype=torch.int32, device=cuda_device)
        cd = _t(_nhwc(c), cuda_device)
        assert lib.ds_avgpool_fix_nhwc(cd.data_ptr(), out.data_ptr(), c.shape[0], c.shape[2],
                                       c.shape[3], c.shape[1], int(g["F"]), st) == 0
        assert np.array_equal(out.cpu().numpy(), g[f"fixed{i}"]), i


@pytest.mark.parametrize("name,batch,kw", [('resnet20', 6, {}), ('resnet18', 3, dict(in_hw=64, num_classes=100)),
                                           ('resnet18', 2, {})], ids=['resnet20', 'resnet18_64', 'resnet18_224'])
def test_staged_pipeline_bit_exact_against_oracle(oracle, cuda_device, name, batch, kw):
    from deepshift_b200 import workloads as W
    from oracle import reference_nets as R
    from helpers import np_weights
    net = W.NETS[name](**kw)
    ws = W.make_weights(net)
    x = W.make_input(net, batch)
    ref = R.forward(net, np_weights(ws), x.numpy())
    for graph in (False, True):
        pipe = W.StagedPipeline(net, ws, batch, cuda_device, use_graph=graph)
        assert np.array_equal(pipe.run(x.to(cuda_device)).cpu().numpy(), ref), graph
        assert np.array_equal(pipe.run(x.to(cuda_device)).cpu().numpy(), ref), graph
