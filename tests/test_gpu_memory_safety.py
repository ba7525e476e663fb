"""Memory safety without a sanitiser: every buffer a kernel touches sits inside a larger allocation.

* Outputs, workspaces and prepared-weight buffers are framed by canary words that must survive the
  launch: a store outside the logical extent is seen even where the allocator's slack would hide it.
* Inputs (activations, packed weights, bias, residual) are framed by poison: values so large that a
  single one of them reaching an accumulator breaks the comparison with the oracle.  The kernels
  predicate every load at the edges of images, rows and tiles; a load that strays outside its tensor
  and is used shows up here.
The shapes sit on the edges of the staging modes (four-pixel, two-pixel, the stem's, plain rows,
table), of the tile grid (ragged last tiles), of the K split (tail wave, counters only) and of the
small-batch kernels.
"""
import ctypes

import numpy as np
import pytest
import torch

from helpers import acts_q16, weights

pytestmark = pytest.mark.gpu

CANARY = -559038737          # 0xDEADBEEF
POISON = 0x3FFFFF00          # about 2^30: one stray term changes an int32 sum beyond any doubt
MARGIN = 4096                # int32 words on either side (a multiple of 4: the frame keeps 16-byte alignment)


class Framed:
    """A logical tensor inside a larger allocation whose margins hold `fill`."""

    def __init__(self, shape, dtype, dev, fill, data=None, margin=MARGIN):
        n = int(np.prod(shape))
        self.margin, self.n, self.fill = margin, n, fill
        self.raw = torch.full((n + 2 * margin,), fill, dtype=torch.int32, device=dev)
        self.t = self.raw[margin:margin + n].view(dtype).view(shape) if dtype != torch.int32 else self.raw[margin:margin + n].view(shape)
        if data is not None:
            self.t.copy_(torch.from_numpy(np.ascontiguousarray(data)).to(dev))

    def intact(self):
        m = self.margin
        return bool((self.raw[:m] == self.fill).all()) and bool((self.raw[m + self.n:] == self.fill).all())


def _cw_framed(shift, sign, dev):
    """Packed weights re-homed inside a poisoned frame (all bits set would decode as huge left shifts; the
    poison word decodes as ordinary fields, so a stray word changes the sum)."""
    from deepshift_b200 import utils
    cw = utils.compress_bits(torch.from_numpy(shift).float(), torch.from_numpy(sign).float(), device=dev)
    fr = Framed(cw.data.shape, torch.int32, dev, 0x2AAAAAAA, data=cw.data.cpu().numpy())
    cw.data = fr.t
    return cw, fr


CONV_SAFETY = [  # B, C, H, W, OC, k, stride, pad
    (3, 16, 28, 28, 40, 3, 1, 1),      # four-pixel staging, ragged last row tile
    (2, 16, 12, 8, 130, 3, 1, 1),      # four-pixel staging on the narrowest width, two column tiles
    (3, 24, 14, 14, 70, 3, 1, 1),      # two-pixel staging
    (2, 8, 9, 6, 33, 3, 1, 1),         # two-pixel staging, narrow
    (2, 3, 32, 32, 64, 7, 2, 3),       # the stem's staging (W a multiple of 8)
    (2, 3, 18, 16, 20, 7, 2, 3),
    (4, 20, 7, 9, 70, 3, 1, 1),        # plain rows, odd width
    (3, 12, 10, 10, 33, 1, 2, 0),      # 1x1 stride 2
    (2, 6, 11, 11, 20, 5, 1, 2),       # 5x5
    (2, 5, 9, 9, 12, 2, 1, 0),         # table mode (no row instantiation for a 2-wide window)
    (5, 128, 7, 7, 130, 3, 1, 1),      # few tiles, long K: shared along K
    (49, 32, 28, 28, 100, 3, 1, 1),    # 151 tiles on 148 SMs: tail wave split through the workspace
]


@pytest.mark.parametrize("case", CONV_SAFETY, ids=[str(c) for c in CONV_SAFETY])
@pytest.mark.parametrize("act_bits", [16, 0])
def test_convolution_stays_inside_its_buffers(oracle, cuda_device, case, act_bits):
    from deepshift_b200 import _ffi, kernels
    B, C, H, W, OC, k, s, p = case
    rng = np.random.default_rng(sum(case))
    x = acts_q16(rng, (B, C, H, W))
    shift, sign = weights(rng, (OC, C, k, k))
    bias = rng.integers(-2000, 2000, OC).astype(np.int32)
    ref = oracle.conv2d(x, shift, sign, bias, (s, s), (p, p))
    res = rng.integers(-50000, 50000, ref.shape).astype(np.int32)
    want = np.maximum(ref.astype(np.float32) + res.astype(np.float32), 0).astype(np.int64).astype(np.int32)
    xf = Framed(x.shape, torch.int32, cuda_device, POISON, data=x)
    bf = Framed(bias.shape, torch.int32, cuda_device, POISON, data=bias)
    rf = Framed(res.shape, torch.int32, cuda_device, POISON, data=res)
    cw, wf = _cw_framed(shift, sign, cuda_device)
    ws_sizes = [None, 16384, 16384 + (24 << 20)]     # no workspace, counters only, counters + partial sums
    for ws_ints in ws_sizes:
        of = Framed(ref.shape, torch.int32, cuda_device, CANARY)
        wsf = Framed((ws_ints,), torch.int32, cuda_device, CANARY) if ws_ints else None
        if wsf is not None:
            wsf.t.zero_()
        f = kernels._fuse(_ffi.IN_I32, _ffi.OUT_I32, 4, 12, relu=True, residual=rf.t, act_bits=act_bits,
                          workspace=wsf.t if wsf is not None else None)
        for _ in range(2):
            rc = _ffi.lib().ds_conv2d_ex(xf.t.data_ptr(), cw.data.data_ptr(), bf.t.data_ptr(), of.t.data_ptr(), B, C, H, W,
                                         OC, k, k, s, s, p, p, cw.bits, cw.base, f,
                                         torch.cuda.current_stream(cuda_device).cuda_stream)
            assert rc == 0
            torch.cuda.synchronize(cuda_device)
            assert np.array_equal(of.t.cpu().numpy(), want), ws_ints
        assert of.intact() and (wsf is None or wsf.intact()), ws_ints
        if wsf is not None:
            assert int(wsf.t[:16383].abs().sum()) == 0       # arrival counters back at zero
    assert xf.intact() and bf.intact() and rf.intact() and wf.intact()


def test_prepared_weights_and_noalloc_stay_inside_their_buffers(oracle, cuda_device):
    from deepshift_b200 import _ffi, kernels
    B, C, H, OC = 12, 16, 28, 40
    rng = np.random.default_rng(12)
    x = acts_q16(rng, (B, C, H, H))
    shift, sign = weights(rng, (OC, C, 3, 3))
    bias = rng.integers(-2000, 2000, OC).astype(np.int32)
    ref = oracle.conv2d(x, shift, sign, bias, (1, 1), (1, 1))
    xf = Framed(x.shape, torch.int32, cuda_device, POISON, data=x)
    bf = Framed(bias.shape, torch.int32, cuda_device, POISON, data=bias)
    cw, wf = _cw_framed(shift, sign, cuda_device)
    lib, st = _ffi.lib(), torch.cuda.current_stream(cuda_device).cuda_stream
    wsf = Framed((16384 + (8 << 20),), torch.int32, cuda_device, CANARY)
    wsf.t.zero_()
    f = kernels._fuse(_ffi.IN_I32, _ffi.OUT_I32, 4, 12, act_bits=16, workspace=wsf.t)
    need = ctypes.c_longlong(0)
    geo = (B, C, H, H, OC, 3, 3, 1, 1, 1, 1, cw.bits, cw.base)
    assert lib.ds_conv2d_prepare(cw.data.data_ptr(), *geo, f, ctypes.byref(need), st) == 0 and need.value > 0
    pf = Framed((need.value // 4,), torch.int32, cuda_device, CANARY)
    f.prepared, f.prepared_bytes = pf.t.data_ptr(), need.value
    assert lib.ds_conv2d_prepare(cw.data.data_ptr(), *geo, f, ctypes.byref(need), st) == 0
    of = Framed(ref.shape, torch.int32, cuda_device, CANARY)
    assert lib.ds_conv2d_ex(xf.t.data_ptr(), cw.data.data_ptr(), bf.t.data_ptr(), of.t.data_ptr(), *geo, f, st) == 0
    torch.cuda.synchronize(cuda_device)
    assert np.array_equal(of.t.cpu().numpy(), ref)
    assert pf.intact() and of.intact() and wsf.intact()
    # the entry point that allocates nothing: a shape it splits along K through its built-in counters
    B2, C2, H2, OC2 = 5, 128, 7, 130
    x2 = acts_q16(rng, (B2, C2, H2, H2))
    s2, g2 = weights(rng, (OC2, C2, 3, 3))
    ref2 = oracle.conv2d(x2, s2, g2, None, (1, 1), (1, 1))
    x2f = Framed(x2.shape, torch.int32, cuda_device, POISON, data=x2)
    cw2, w2f = _cw_framed(s2, g2, cuda_device)
    o2f = Framed(ref2.shape, torch.int32, cuda_device, CANARY)
    f2 = kernels._fuse(_ffi.IN_I32, _ffi.OUT_I32, 4, 12, act_bits=16)
    assert lib.ds_conv2d_noalloc(x2f.t.data_ptr(), cw2.data.data_ptr(), None, o2f.t.data_ptr(), B2, C2, H2, H2, OC2, 3, 3,
                                 1, 1, 1, 1, cw2.bits, cw2.base, f2, st) == 0
    torch.cuda.synchronize(cuda_device)
    assert np.array_equal(o2f.t.cpu().numpy(), ref2)
    assert o2f.intact() and x2f.intact() and w2f.intact() and xf.intact() and bf.intact() and wf.intact()


@pytest.mark.parametrize("M,K,N", [(1, 4096, 33), (5, 1031, 300), (16, 96, 4100), (40, 3000, 70), (64, 515, 130),
                                   (65, 4, 33), (300, 512, 200), (2304, 260, 130), (257, 29, 260)])
@pytest.mark.parametrize("act_bits", [16, 0])
def test_linear_stays_inside_its_buffers(oracle, cuda_device, M, K, N, act_bits):
    from deepshift_b200 import _ffi, kernels
    rng = np.random.default_rng(M + 3 * K + 5 * N)
    x = acts_q16(rng, (M, K))
    shift, sign = weights(rng, (N, K))
    bias = rng.integers(-2000, 2000, N).astype(np.int32)
    ref = oracle.linear(x, shift, sign, bias)
    xf = Framed(x.shape, torch.int32, cuda_device, POISON, data=x)
    bf = Framed(bias.shape, torch.int32, cuda_device, POISON, data=bias)
    cw, wf = _cw_framed(shift, sign, cuda_device)
    for ws_ints in (None, 16384 + (24 << 20)):
        of = Framed(ref.shape, torch.int32, cuda_device, CANARY)
        wsf = Framed((ws_ints,), torch.int32, cuda_device, CANARY) if ws_ints else None
        if wsf is not None:
            wsf.t.zero_()
        f = kernels._fuse(act_bits=act_bits, workspace=wsf.t if wsf is not None else None)
        rc = _ffi.lib().ds_linear_ex(xf.t.data_ptr(), cw.data.data_ptr(), bf.t.data_ptr(), of.t.data_ptr(), M, K, N,
                                     cw.bits, cw.base, f, torch.cuda.current_stream(cuda_device).cuda_stream)
        assert rc == 0
        torch.cuda.synchronize(cuda_device)
        assert np.array_equal(of.t.cpu().numpy(), ref)
        assert of.intact() and (wsf is None or wsf.intact())
    assert xf.intact() and bf.intact() and wf.intact()


@pytest.mark.parametrize("case", [(2, 3, 9, 7, 5, 3, 2, 1, 1), (3, 20, 11, 13, 70, 3, 1, 1, 2), (2, 3, 30, 30, 64, 7, 2, 3, 3),
                                  (49, 32, 28, 28, 100, 3, 1, 1, 1)], ids=str)
def test_staged_convolution_stays_inside_its_buffers(oracle, cuda_device, case):
    """The TMA-fed kernel: the staged input (with its halo) inside a poisoned frame, every output
    form inside canaries.  Tensor-map loads past the last image are zero-filled by the hardware and
    belong to rows that are never stored."""
    from deepshift_b200 import _ffi, staged, utils
    B, C, H, W, OC, k, s, p, halo = case
    rng = np.random.default_rng(sum(case))
    x = acts_q16(rng, (B, C, H, W))
    shift, sign = weights(rng, (OC, C, k, k))
    bias = rng.integers(-2000, 2000, OC).astype(np.int32)
    ref = oracle.conv2d(x, shift, sign, bias, (s, s), (p, p))
    OH, OW = ref.shape[2], ref.shape[3]
    Cs = (C + 3) // 4 * 4
    lib, st = _ffi.lib(), torch.cuda.current_stream(cuda_device).cuda_stream
    xs_f = Framed((B, H + 2 * halo, W + 2 * halo, Cs), torch.float32, cuda_device, 0x4E7FFFFF)   # ~1.07e9 as a float
    xs = _ffi.Staged(xs_f.t.data_ptr(), B, H, W, C, halo)
    assert lib.ds_staged_fill(ctypes.byref(xs), st) == 0
    xin = torch.from_numpy(x).to(cuda_device)
    assert lib.ds_stage_nchw(xin.data_ptr(), _ffi.IN_I32, 4, 12, ctypes.byref(xs), st) == 0
    cw, wf = _cw_framed(shift, sign, cuda_device)
    prepared = staged.prepared_weights(cw, C, OC, k, k, cuda_device)
    pf = Framed(prepared.shape, torch.int32, cuda_device, 0x4E7FFFFF, data=prepared.cpu().numpy())
    codes = Framed((B, OH, OW, OC), torch.int32, cuda_device, CANARY)
    nchw = Framed((B, OC, OH, OW), torch.int32, cuda_device, CANARY)
    nxt_f = Framed((B, OH + 2, OW + 2, (OC + 3) // 4 * 4), torch.float32, cuda_device, CANARY)
    nxt = _ffi.Staged(nxt_f.t.data_ptr(), B, OH, OW, OC, 1)
    assert lib.ds_staged_fill(ctypes.byref(nxt), st) == 0
    bf = Framed(bias.shape, torch.int32, cuda_device, POISON, data=bias)
    wsf = Framed((16384 + (24 << 20),), torch.int32, cuda_device, CANARY)
    wsf.t.zero_()
    o = _ffi.StagedOut()
    o.codes, o.nchw, o.staged = codes.t.data_ptr(), nchw.t.data_ptr(), ctypes.pointer(nxt)
    o.act_integer_bits, o.act_fraction_bits, o.in_act_bits = 4, 12, 16
    for _ in range(2):
        rc = lib.ds_staged_conv2d(ctypes.byref(xs), pf.t.data_ptr(), pf.n * 4, bf.t.data_ptr(), OC, k, k, s, s, p, p,
                                  ctypes.byref(o), wsf.t.data_ptr(), wsf.n * 4, st)
        assert rc == 0
        torch.cuda.synchronize(cuda_device)
        assert np.array_equal(nchw.t.cpu().numpy(), ref)
        assert np.array_equal(codes.t.cpu().numpy(), np.transpose(ref, (0, 2, 3, 1)))
    inner = nxt_f.t[:, 1:1 + OH, 1:1 + OW, :OC].cpu().numpy()
    assert np.array_equal(inner, np.clip(np.transpose(ref, (0, 2, 3, 1)), -32768, 28672).astype(np.float32) + 0.5)
    assert codes.intact() and nchw.intact() and nxt_f.intact() and wsf.intact() and xs_f.intact() and pf.intact()
    assert bf.intact() and wf.intact()
    assert int(wsf.t[:16383].abs().sum()) == 0


def test_bounds_checking_flavour_of_the_library(cuda_device):
    """The library built with -DDS_BOUNDS_CHECK (every global access of the linear / convolution
    kernels tests its address first, skips it if outside and records the kind) in a process of its
    own: all shapes exact with status 0, and the checks are seen to fire when the activations are
    declared shorter than they are.  Nothing traps and nothing leaves a real buffer."""
    import os
    import subprocess
    import sys
    from deepshift_b200 import _build
    if not os.path.exists(_build.CHECKED_LIB_PATH) and _build.nvcc_path() is None:
        pytest.skip("checked flavour not built and no nvcc here")
    env = dict(os.environ, DEEPSHIFT_B200_CHECKED="1")
    script = os.path.join(os.path.dirname(os.path.abspath(__file__)), "checked_build_cases.py")
    res = subprocess.run([sys.executable, script], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                         timeout=1200)
    assert res.returncode == 0 and "checked build: ok" in res.stdout, res.stdout[-3000:]


def test_timing_flavour_prints_cycle_counters_and_computes_the_same(cuda_device):
    """The library built with -DDS_WS_TIMING in a process of its own: one convolution on the
    warp-specialised kernel gives the result of the normal flavour and leaves one "ws_timing" line per
    warp of a CTA (16 consumer and 8 producer warps).  Skipped where that flavour was not built."""
    import os
    import subprocess
    import sys
    from deepshift_b200 import _build, _ffi, kernels
    if not _build.is_current(timing=True):
        pytest.skip("timing flavour not built")
    code = (
        "import numpy as np, torch\n"
        "from deepshift_b200 import kernels, utils, _ffi\n"
        "rng = np.random.default_rng(3)\n"
        "x = torch.from_numpy(rng.integers(-30000, 30000, (40, 16, 28, 28)).astype(np.int32)).cuda()\n"
        "shift = torch.from_numpy(rng.integers(-14, 1, (128, 16, 3, 3)).astype(np.float32))\n"
        "sign = torch.from_numpy(rng.choice([-1., 0., 1.], (128, 16, 3, 3)).astype(np.float32))\n"
        "cw = utils.compress_bits(shift, sign, device=x.device)\n"
        "out = kernels.conv2d_fused(x, (128, 16, 3, 3), None, cw, 1, 1, act_bits=16)\n"
        "torch.cuda.synchronize()\n"
        "print('checksum', int(out.to(torch.int64).sum()), int((out.to(torch.int64) * 7 % 1000003).sum()))\n")
    outs = {}
    for flavour in ("", "1"):
        env = dict(os.environ, DEEPSHIFT_B200_TIMING=flavour, PYTHONPATH=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        res = subprocess.run([sys.executable, "-c", code], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                             text=True, timeout=600)
        assert res.returncode == 0, res.stdout[-3000:]
        outs[flavour] = res.stdout
    checks = {k: [l for l in v.splitlines() if l.startswith("checksum")] for k, v in outs.items()}
    assert checks[""] and checks[""] == checks["1"]
    assert "ws_timing" not in outs[""]
    lines = [l for l in outs["1"].splitlines() if l.startswith("ws_timing")]
    assert sum("consumer warp" in l for l in lines) == 16 and sum("producer warp" in l for l in lines) == 8, outs["1"][-2000:]
