"""ds_conv2d_noalloc: the convolution entry point for callers that cannot allocate device memory
(its split-K scratch is a fixed array inside the library).  Collected last on purpose, so that a
run that stops at the first failure has already run every other test."""
import ctypes

import numpy as np
import pytest
import torch

from helpers import acts_q16, weights

pytestmark = pytest.mark.gpu


def _run(entry, x, packed, bias, res, out, shape, cw, out_kind, dev):
    """One call through the C ABI on torch's current stream."""
    from deepshift_b200 import _ffi
    B, C, H, OC, k, s, p = shape
    f = _ffi.Fuse()
    f.in_kind, f.out_kind = _ffi.IN_I32_CLAMP, out_kind
    f.act_integer_bits, f.act_fraction_bits = 4, 12
    f.relu, f.round_f32 = 1, 1
    f.residual = res.data_ptr()
    if entry == "ds_conv2d_ex":  # the existing entry point gets a caller-allocated workspace
        ws = torch.zeros(16384, dtype=torch.int32, device=dev)
        f.workspace, f.workspace_bytes = ws.data_ptr(), ws.numel() * 4
    fn = getattr(_ffi.lib(), entry)
    rc = fn(x.data_ptr(), packed.data_ptr(), bias.data_ptr(), out.data_ptr(), B, C, H, H, OC, k, k, s, s, p, p,
            cw.bits, cw.base, ctypes.byref(f), torch.cuda.current_stream(dev).cuda_stream)
    torch.cuda.synchronize(dev)
    return rc


@pytest.mark.parametrize("shape", [(5, 128, 7, 130, 3, 1, 1),     # few tiles, long K: split along K, counters in use
                                   (40, 32, 28, 64, 3, 1, 1),     # plenty of tiles: no split
                                   (3, 64, 14, 256, 1, 2, 0)])    # 1x1 stride 2
@pytest.mark.parametrize("out_f32", [False, True])
def test_noalloc_matches_existing_entry_point_twice(oracle, cuda_device, shape, out_f32):
    """Bit-identical to ds_conv2d_ex (the tolerance of every other test here: none), on two calls
    in a row -- the second one finds the array as the first left it.  Both are also held against the
    CPU oracle, so the scheme this entry point is limited to (counters only: integer atomics on the
    zeroed output) is anchored on its own."""
    from deepshift_b200 import _ffi, utils
    B, C, H, OC, k, s, p = shape
    rng = np.random.default_rng(sum(shape) + out_f32)
    OHW = (H + 2 * p - k) // s + 1
    x_np = acts_q16(rng, (B, C, H, H)) * 2                                 # beyond the clamp: exercises IN_I32_CLAMP
    x = torch.from_numpy(x_np).to(cuda_device)
    shift, sign = weights(rng, (OC, C, k, k))
    cw = utils.compress_bits(torch.from_numpy(shift).float(), torch.from_numpy(sign).float(), device=cuda_device)
    bias_np = rng.integers(-2000, 2000, OC).astype(np.int32)
    res_np = rng.integers(-50000, 50000, (B, OC, OHW, OHW)).astype(np.int32)
    bias, res = torch.from_numpy(bias_np).to(cuda_device), torch.from_numpy(res_np).to(cuda_device)
    kind = _ffi.OUT_F32 if out_f32 else _ffi.OUT_I32
    dtype = torch.float32 if out_f32 else torch.int32
    want = torch.empty((B, OC, OHW, OHW), dtype=dtype, device=cuda_device)
    assert _run("ds_conv2d_ex", x, cw.data, bias, res, want, shape, cw, kind, cuda_device) == 0
    # oracle: clamp of the 4.12 quantiser on read, integer convolution, fp32 residual add, ReLU,
    # the rounding of `out.float()`, optional conversion to fp32
    acc = oracle.conv2d(np.clip(x_np, -32768, 28672), shift, sign, bias_np, (s, s), (p, p))
    ref = np.maximum(acc.astype(np.float32) + res_np.astype(np.float32), 0).astype(np.int64).astype(np.int32)
    ref = ref.astype(np.float32).astype(np.int64).astype(np.int32)
    ref = oracle.from_fixed(ref, 12) if out_f32 else ref
    assert np.array_equal(want.cpu().numpy(), ref)
    for call in range(2):
        got = torch.full_like(want, 7)
        assert _run("ds_conv2d_noalloc", x, cw.data, bias, res, got, shape, cw, kind, cuda_device) == 0
        assert torch.equal(got, want), call


def test_noalloc_rejects_more_tiles_than_its_scratch_holds(cuda_device):
    from deepshift_b200 import _ffi, utils
    rng = np.random.default_rng(1)
    B, C, H, OC = 4, 1, 1100, 1      # 4 * 1100 * 1100 output positions = 18907 tiles of 256 > 16384
    x = torch.zeros((B, C, H, H), dtype=torch.int32, device=cuda_device)
    shift, sign = weights(rng, (OC, C, 1, 1))
    cw = utils.compress_bits(torch.from_numpy(shift).float(), torch.from_numpy(sign).float(), device=cuda_device)
    out = torch.full((B, OC, H, H), 5, dtype=torch.int32, device=cuda_device)
    f = _ffi.Fuse()
    rc = _ffi.lib().ds_conv2d_noalloc(x.data_ptr(), cw.data.data_ptr(), None, out.data_ptr(), B, C, H, H, OC, 1, 1, 1, 1,
                                      0, 0, cw.bits, cw.base, ctypes.byref(f),
                                      torch.cuda.current_stream(cuda_device).cuda_stream)
    assert rc == 6
    assert b"scratch" in _ffi.lib().ds_strerror(rc)
    torch.cuda.synchronize(cuda_device)
    assert int(out.min()) == 5 and int(out.max()) == 5  # nothing ran
    with pytest.raises(RuntimeError, match="scratch"):
        _ffi.check(rc, "conv2d_noalloc")
