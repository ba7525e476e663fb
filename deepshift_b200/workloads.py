"""The benchmark networks of the use_kernel path, as data, and two ways to run them on the GPU.

A network is a list of shift layers plus a short program of steps (convolution, linear, pooling,
residual bookkeeping).  The same program is run

* by ``ModuleNet``: an ``nn.Module`` built from ``Conv2dShift`` / ``LinearShift`` with the
  reference's fp32 glue between layers (``F.relu``, ``+``, ``F.max_pool2d`` ...) -- the drop-in
  module path, one fused kernel per shift layer;
* by ``IntPipeline``: activations stay int32 fixed point from the first layer to the logits,
  ReLU / residual add / fp32 rounding are fused into the convolution epilogues, pooling runs on
  the int32 codes, all buffers are pre-allocated and the whole forward pass can be replayed as
  one CUDA graph.  Every shift-layer output and the logits are bit-identical to ``ModuleNet``'s.

Global average pooling: fp32 summation order is not fixed by torch (its CPU kernel sums in an
order that depends on the vector width, its CUDA ``adaptive_avg_pool2d`` reduces as a tree and then
multiplies by a rounded 1/(H*W)), so results differ between the two by a few codes of 2^-12 once a
plane's codes sum to more than 2^24 -- which the unclamped residual stream of this synthetic
ResNet-18 does.  Both executors use the order-independent rule: the exact sum, rounded once to
fp32, divided by H*W.  It equals torch's CPU result whenever fp32 addition is exact (sum of codes
below 2^24; pinned by a golden vector).

Topologies: the reference's ``LinearMNIST`` / ``ConvMNIST`` (pytorch/mnist.py:23-57, without the
dropout and log-softmax, which are not part of the kernel path), its CIFAR-10 ``resnet20``
(pytorch/cifar10_models/resnet.py:23-140, option-A shortcuts, BatchNorm folded into a bias) and
the torchvision ResNet-18 the reference converts for ImageNet (pytorch/imagenet.py:199-219).
Weights and inputs are synthetic and seeded; no dataset or checkpoint is read.
"""
from dataclasses import dataclass, field

import numpy as np
import torch
import torch.nn as nn
import torch.nn.functional as F

from . import _ffi, kernels, modules, utils


# ------------------------------------------------------------------------------------------------ nets
@dataclass
class Layer:
    kind: str            # 'conv' or 'linear'
    cin: int
    cout: int
    k: int = 1
    stride: int = 1
    pad: int = 0

    @property
    def weight_shape(self):
        return (self.cout, self.cin, self.k, self.k) if self.kind == 'conv' else (self.cout, self.cin)


@dataclass
class Net:
    name: str
    in_shape: tuple      # (C, H, W)
    layers: list
    steps: list          # tuples, see the executors
    act_integer_bits: int = 4
    act_fraction_bits: int = 12
    weight_bits: int = 5
    seed: int = 20250

    def shift_ops(self, batch=1):
        """(activation, weight) pairs of one forward pass: MACs of the equivalent dense net."""
        shapes, total = _trace_shapes(self), 0
        for li, (cin_hw, out_hw) in shapes.items():
            L = self.layers[li]
            if L.kind == 'conv':
                total += out_hw[0] * out_hw[1] * L.cout * L.cin * L.k * L.k
            else:
                total += L.cin * L.cout
        return total * batch


def _trace_shapes(net):
    """Per shift layer: input (H, W) and output (H, W)."""
    C, H, W = net.in_shape
    cur = {'x': (C, H, W)}
    out = {}
    for st in net.steps:
        op = st[0]
        if op == 'conv':
            li, o = st[1], st[2]
            L = net.layers[li]
            c, h, w = cur[o.get('src', 'x')]
            oh, ow = (h + 2 * L.pad - L.k) // L.stride + 1, (w + 2 * L.pad - L.k) // L.stride + 1
            out[li] = ((h, w), (oh, ow))
            cur[o.get('dst', 'x')] = (L.cout, oh, ow)
        elif op == 'linear':
            li = st[1]
            out[li] = ((1, 1), (1, 1))
            cur['x'] = (net.layers[li].cout, 1, 1)
        elif op == 'maxpool':
            _, k, s, p = st
            c, h, w = cur['x']
            cur['x'] = (c, (h + 2 * p - k) // s + 1, (w + 2 * p - k) // s + 1)
        elif op == 'gap':
            cur['x'] = (cur['x'][0], 1, 1)
        elif op == 'flatten':
            c, h, w = cur['x']
            cur['x'] = (c * h * w, 1, 1)
        elif op == 'copy':
            cur[st[2]] = cur[st[1]]
        elif op == 'shortcutA':
            c, h, w = cur[st[1]]
            cur[st[2]] = (c + 2 * (st[3] // 4), (h + 1) // 2, (w + 1) // 2)
    return out


def mnist_fc():
    L = [Layer('linear', 784, 512), Layer('linear', 512, 512), Layer('linear', 512, 10)]
    S = [('flatten',), ('linear', 0, dict(relu=True)), ('linear', 1, dict(relu=True)), ('linear', 2, dict(relu=False))]
    return Net('mnist_fc', (1, 28, 28), L, S, seed=20250)


def mnist_conv():
    L = [Layer('conv', 1, 20, 5, 1, 0), Layer('conv', 20, 50, 5, 1, 0), Layer('linear', 800, 500),
         Layer('linear', 500, 10)]
    S = [('conv', 0, dict(relu=True)), ('maxpool', 2, 2, 0), ('conv', 1, dict(relu=True)), ('maxpool', 2, 2, 0),
         ('flatten',), ('linear', 2, dict(relu=True)), ('linear', 3, dict(relu=False))]
    return Net('mnist_conv', (1, 28, 28), L, S, seed=20251)


def resnet20():
    L = [Layer('conv', 3, 16, 3, 1, 1)]
    S = [('conv', 0, dict(relu=True))]
    cin = 16
    for planes, stride0 in ((16, 1), (32, 2), (64, 2)):
        for b in range(3):
            stride = stride0 if b == 0 else 1
            a, c = len(L), len(L) + 1
            L += [Layer('conv', cin, planes, 3, stride, 1), Layer('conv', planes, planes, 3, 1, 1)]
            if stride != 1 or cin != planes:
                S.append(('shortcutA', 'x', 'id', planes))
            else:
                S.append(('copy', 'x', 'id'))
            S += [('conv', a, dict(relu=True)), ('conv', c, dict(relu=True, add='id'))]
            cin = planes
    L.append(Layer('linear', 64, 10))
    S += [('gap',), ('linear', len(L) - 1, dict(relu=False))]
    return Net('resnet20', (3, 32, 32), L, S, seed=20252)


def resnet18(num_classes=1000, in_hw=224):
    L = [Layer('conv', 3, 64, 7, 2, 3)]
    S = [('conv', 0, dict(relu=True)), ('maxpool', 3, 2, 1)]
    cin = 64
    for planes, stride0 in ((64, 1), (128, 2), (256, 2), (512, 2)):
        for b in range(2):
            stride = stride0 if b == 0 else 1
            S.append(('copy', 'x', 'id'))
            a = len(L)
            L.append(Layer('conv', cin, planes, 3, stride, 1))
            c = len(L)
            L.append(Layer('conv', planes, planes, 3, 1, 1))
            if stride != 1 or cin != planes:
                d = len(L)
                L.append(Layer('conv', cin, planes, 1, stride, 0))
                S.append(('conv', d, dict(relu=False, src='id', dst='id')))
            S += [('conv', a, dict(relu=True)), ('conv', c, dict(relu=True, add='id'))]
            cin = planes
    L.append(Layer('linear', 512, num_classes))
    S += [('gap',), ('linear', len(L) - 1, dict(relu=False))]
    return Net('resnet18', (3, in_hw, in_hw), L, S, seed=20253)


NETS = {'mnist_fc': mnist_fc, 'mnist_conv': mnist_conv, 'resnet20': resnet20, 'resnet18': resnet18}


# ------------------------------------------------------------------------------------------------ data
def make_weights(net, zero_fraction=0.10):
    """Per layer (shift int32 <= 0, sign int32 in {-1,0,+1}, bias fp32 on the 2^-F grid), seeded:
    sign -1/0/+1 with P = 0.45/0.10/0.45, shift uniform in [-(2^(wb-1)-1), 0], bias N(0, 0.01)
    rounded with round_to_fixed."""
    out = []
    lo = -(2 ** (net.weight_bits - 1) - 1)
    for li, L in enumerate(net.layers):
        g = torch.Generator().manual_seed(net.seed * 1000 + li)
        shape = L.weight_shape
        shift = torch.randint(lo, 1, shape, generator=g, dtype=torch.int32)
        u = torch.rand(shape, generator=g)
        neg = (1.0 - zero_fraction) / 2
        sign = torch.where(u < neg, -1, torch.where(u < neg + zero_fraction, 0, 1)).to(torch.int32)
        bias = torch.randn(L.cout, generator=g) * 0.01
        bias = utils.round_to_fixed(bias, net.act_integer_bits, net.act_fraction_bits)
        out.append(dict(shift=shift, sign=sign, bias=bias))
    return out


def make_input(net, batch, rank=0):
    """Seeded fp32 input already on the fixed-point grid (what round_to_fixed leaves unchanged)."""
    g = torch.Generator().manual_seed(net.seed + 7919 * (rank + 1))
    if net.name.startswith('mnist'):
        x = (torch.rand((batch,) + net.in_shape, generator=g) - 0.1307) / 0.3081
    else:
        x = torch.randn((batch,) + net.in_shape, generator=g)
    return utils.round_to_fixed(x, net.act_integer_bits, net.act_fraction_bits)


# ------------------------------------------------------------------------------------------------ module path
def _shortcut_a(x, planes):
    # cifar10_models/resnet.py:38-40
    return F.pad(x[:, :, ::2, ::2], (0, 0, 0, 0, planes // 4, planes // 4), "constant", 0)


class ModuleNet(nn.Module):
    """The network as the reference would run it with ``use_kernel=True``: shift modules and fp32
    glue.  ``fuse=True`` hands the residual additions and ReLUs that follow a shift layer to that
    layer's ``forward`` as fusion hints and pools with ``kernels.maxpool2d_f32`` (same values, fewer
    and faster passes over the activations)."""

    def __init__(self, net, weights, device='cuda', use_kernel=True, fuse=False):
        super().__init__()
        self.net = net
        self.fuse = fuse
        mods = []
        kw = dict(use_kernel=use_kernel, use_cuda=True, rounding='deterministic', weight_bits=net.weight_bits,
                  act_integer_bits=net.act_integer_bits, act_fraction_bits=net.act_fraction_bits)
        for L, w in zip(net.layers, weights):
            if L.kind == 'conv':
                m = modules.Conv2dShift(L.cin, L.cout, L.k, L.stride, L.pad, bias=True, **kw)
            else:
                m = modules.LinearShift(L.cin, L.cout, bias=True, **kw)
            m.shift.data = w['shift'].float()
            m.sign.data = w['sign'].float()
            m.bias.data = w['bias'].clone()
            mods.append(m)
        self.layers = nn.ModuleList(mods)
        self.to(device)
        if use_kernel:
            for m in self.layers:
                m.conc_weight = utils.compress_bits(m.shift.data, m.sign.data, device=torch.device(device))

    def forward(self, x):
        t = {'x': x}
        for st in self.net.steps:
            op = st[0]
            if op == 'conv':
                li, o = st[1], st[2]
                if self.fuse:
                    y = self.layers[li](t[o.get('src', 'x')], residual=t[o['add']] if o.get('add') else None,
                                        relu=bool(o.get('relu')))
                else:
                    y = self.layers[li](t[o.get('src', 'x')])
                    if o.get('add'):
                        y = y + t[o['add']]
                    if o.get('relu'):
                        y = F.relu(y)
                t[o.get('dst', 'x')] = y
            elif op == 'linear':
                if self.fuse:
                    t['x'] = self.layers[st[1]](t['x'], relu=bool(st[2].get('relu')))
                else:
                    y = self.layers[st[1]](t['x'])
                    t['x'] = F.relu(y) if st[2].get('relu') else y
            elif op == 'maxpool':
                if self.fuse and t['x'].is_cuda and t['x'].dtype == torch.float32:
                    t['x'] = kernels.maxpool2d_f32(t['x'].contiguous(), st[1], st[2], st[3])
                else:
                    t['x'] = F.max_pool2d(t['x'], st[1], st[2], st[3])
            elif op == 'gap':
                # exact sum (float64 holds it), one rounding to fp32, then a true division: by a tensor,
                # because torch's CUDA division by a Python number multiplies by its rounded reciprocal
                x = t['x']
                hw = torch.full((), float(x.shape[2] * x.shape[3]), dtype=torch.float32, device=x.device)
                t['x'] = x.sum((2, 3), dtype=torch.float64).float() / hw
            elif op == 'flatten':
                t['x'] = t['x'].flatten(1)
            elif op == 'copy':
                t[st[2]] = t[st[1]]
            elif op == 'shortcutA':
                t[st[2]] = _shortcut_a(t[st[1]], st[3])
        return t['x']


# ------------------------------------------------------------------------------------------------ integer pipeline
class _Pipeline:
    """What both whole-network executors share: a static input buffer, a list of launches recorded
    once, optional CUDA-graph replay, and the count of library kernels in one pass."""

    @property
    def n_launches(self):
        """Kernels of this library in one pass, counted by the library itself while the pass was
        recorded (a layer call can be several kernels: weight expansion, the convolution)."""
        return len(self.calls) if self._n_launches is None else self._n_launches

    def _capture(self):
        with torch.cuda.device(self.device):
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                self._launch_all()  # warm-up outside capture: kernel attributes, weights expanded once
            torch.cuda.current_stream().wait_stream(s)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            before = _ffi.lib().ds_launch_count()
            with torch.cuda.graph(g):
                self._launch_all()
            self._n_launches = int(_ffi.lib().ds_launch_count() - before)  # kernels of one replay
            self.graph = g

    def run(self, x=None):
        """x: fp32 CUDA tensor [batch, C, H, W] (copied into the static input buffer) or None to
        reuse the buffer's contents.  Returns the static fp32 logits tensor."""
        if x is not None:
            self.x_in.copy_(x, non_blocking=True)
        if self.graph is not None:
            self.graph.replay()
        else:
            before = _ffi.lib().ds_launch_count()
            self._launch_all()
            self._n_launches = int(_ffi.lib().ds_launch_count() - before)
        return self.out


class IntPipeline(_Pipeline):
    """Whole-network fixed-point executor.

    ``run(x)`` takes an fp32 CUDA batch of the fixed size given at construction and returns fp32
    logits.  Activations between layers are int32 codes (value * 2^F).  Every convolution reads
    them with the clamp of the consuming layer's quantiser (DS_IN_I32_CLAMP) and writes
    relu(acc + bias [+ residual]) rounded as the reference's fp32 tensor would hold it.
    """

    def __init__(self, net, weights, batch, device='cuda', use_graph=True):
        self.net, self.batch, self.device = net, batch, torch.device(device)
        self.I, self.F = net.act_integer_bits, net.act_fraction_bits
        self.packed, self.bias = [], []
        for L, w in zip(net.layers, weights):
            self.packed.append(utils.compress_bits(w['shift'].float(), w['sign'].float(), device=self.device))
            self.bias.append((w['bias'] * (2 ** self.F)).int().to(self.device).contiguous())
        self.x_in = torch.empty((batch,) + net.in_shape, dtype=torch.float32, device=self.device)
        self.workspace = kernels.new_workspace(self.device)   # its own: pipelines may run side by side
        self._plan()
        self._n_launches = None
        self.graph = None
        if use_graph:
            self._capture()

    # Builds the list of launches with all output buffers allocated once.
    def _plan(self):
        net, dev = self.net, self.device
        t = {'x': self.x_in}
        fp32 = {'x': True}
        self.calls = []
        n_shift = sum(1 for s in net.steps if s[0] in ('conv', 'linear'))
        seen = 0
        for st in net.steps:
            op = st[0]
            if op in ('conv', 'linear'):
                seen += 1
                lastlayer = seen == n_shift
                li, o = st[1], st[2]
                L = net.layers[li]
                src = o.get('src', 'x')
                xin = t[src]
                in_fp32 = fp32[src]
                if op == 'conv':
                    if in_fp32 and utils.quantise_in_own_pass((L.k, L.k), L.cout):
                        # every input value would be converted many times: quantise it once in a
                        # pass of its own instead of inside the convolution's staging code
                        xq = torch.empty(xin.shape, dtype=torch.int32, device=dev)
                        self.calls.append(('quant', xin, xq))
                        xin, in_fp32 = xq, False
                    in_kind = _ffi.IN_F32_CONV if in_fp32 else _ffi.IN_I32_CLAMP
                    B, C, H, W = xin.shape
                    OH, OW = (H + 2 * L.pad - L.k) // L.stride + 1, (W + 2 * L.pad - L.k) // L.stride + 1
                    out = torch.empty((B, L.cout, OH, OW), device=dev,
                                      dtype=torch.float32 if lastlayer else torch.int32)
                else:
                    in_kind = _ffi.IN_F32_LINEAR if in_fp32 else _ffi.IN_I32
                    xin = xin.reshape(xin.shape[0], -1)
                    out = torch.empty((xin.shape[0], L.cout), device=dev,
                                      dtype=torch.float32 if lastlayer else torch.int32)
                res = t[o['add']] if o.get('add') else None
                fuse = kernels._fuse(in_kind, _ffi.OUT_F32 if lastlayer else _ffi.OUT_I32, self.I, self.F,
                                     relu=bool(o.get('relu')), requant=False, residual=res,
                                     round_f32=not lastlayer, workspace=self.workspace)
                self.calls.append((op, xin, li, L, out, fuse, res))
                dst = o.get('dst', 'x')
                t[dst], fp32[dst] = out, lastlayer
            elif op == 'maxpool':
                _, k, s_, p_ = st
                xin = t['x']
                assert not fp32['x'], "pooling runs on int32 activations"
                B, C, H, W = xin.shape
                out = torch.empty((B, C, (H + 2 * p_ - k) // s_ + 1, (W + 2 * p_ - k) // s_ + 1),
                                  dtype=torch.int32, device=dev)
                self.calls.append(('maxpool', xin, k, s_, p_, out))
                t['x'] = out
            elif op == 'gap':
                xin = t['x']
                out = torch.empty((xin.shape[0], xin.shape[1]), dtype=torch.int32, device=dev)
                self.calls.append(('gap', xin, out))
                t['x'] = out
            elif op == 'flatten':
                t['x'] = t['x'].reshape(t['x'].shape[0], -1)
            elif op == 'copy':
                t[st[2]], fp32[st[2]] = t[st[1]], fp32[st[1]]
            elif op == 'shortcutA':
                xin = t[st[1]]
                pad = st[3] // 4
                B, C, H, W = xin.shape
                out = torch.zeros((B, C + 2 * pad, (H + 1) // 2, (W + 1) // 2), dtype=torch.int32, device=dev)
                self.calls.append(('shortcutA', xin, out, pad))
                t[st[2]], fp32[st[2]] = out, False
        self.out = t['x']

    def _launch_all(self):
        lib = _ffi.lib()
        stream = torch.cuda.current_stream(self.device).cuda_stream
        for c in self.calls:
            op = c[0]
            if op == 'conv':
                _, xin, li, L, out, fuse, _res = c
                B, C, H, W = xin.shape
                cw = self.packed[li]
                if fuse.prepared is None and fuse.prepared_bytes == 0:
                    # first pass (outside graph capture): expand the layer's weights once and for all
                    geometry = (B, C, H, W, L.cout, L.k, L.k, L.stride, L.stride, L.pad, L.pad)
                    prepared = kernels._prepared_weights(cw, geometry, fuse, self.device)
                    if prepared is not None:
                        fuse.prepared, fuse.prepared_bytes = prepared.data_ptr(), prepared.numel() * 4
                    else:
                        fuse.prepared_bytes = -1  # asked: launches of this geometry do not use them
                rc = lib.ds_conv2d_ex(xin.data_ptr(), cw.data.data_ptr(), self.bias[li].data_ptr(), out.data_ptr(),
                                      B, C, H, W, L.cout, L.k, L.k, L.stride, L.stride, L.pad, L.pad, cw.bits,
                                      cw.base, fuse, stream)
                _ffi.check(rc, "conv2d_ex")
            elif op == 'linear':
                _, xin, li, L, out, fuse, _res = c
                cw = self.packed[li]
                rc = lib.ds_linear_ex(xin.data_ptr(), cw.data.data_ptr(), self.bias[li].data_ptr(), out.data_ptr(),
                                      xin.shape[0], xin.shape[1], L.cout, cw.bits, cw.base, fuse, stream)
                _ffi.check(rc, "linear_ex")
            elif op == 'quant':
                _, xin, xq = c
                _ffi.check(lib.ds_quantize_f32(xin.data_ptr(), xq.data_ptr(), xin.numel(), _ffi.IN_F32_CONV, self.I,
                                               self.F, stream), "quantize_f32")
            elif op == 'maxpool':
                _, xin, k, s_, p_, out = c
                B, C, H, W = xin.shape
                _ffi.check(lib.ds_maxpool2d_i32(xin.data_ptr(), out.data_ptr(), B, C, H, W, k, s_, p_, stream),
                           "maxpool2d_i32")
            elif op == 'gap':
                _, xin, out = c
                B, C, H, W = xin.shape
                _ffi.check(lib.ds_avgpool_fix_i32(xin.data_ptr(), out.data_ptr(), B, C, H, W, self.F, stream),
                           "avgpool_fix_i32")
            elif op == 'shortcutA':
                _, xin, out, pad = c
                out[:, pad:pad + xin.shape[1]].copy_(xin[:, :, ::2, ::2])



# ------------------------------------------------------------------------------------------------ staged pipeline
class _Val:
    """One activation tensor of the staged pipeline and the forms its readers need."""

    def __init__(self, C, H, W):
        self.C, self.H, self.W = C, H, W
        self.halo = None        # not None: read by a convolution (needs the staged operand, this halo)
        self.need_codes = False  # read as residual, by a pooling step or by the classifier
        self.flat = False        # the result of global pooling: codes are [B,C]
        self.zero_init = False   # codes are only partly written (option-A shortcut): start from zero
        self.staged = None
        self.codes = None        # int32 NHWC [B,H,W,C]; [B,C] after global pooling


class StagedPipeline(_Pipeline):
    """Whole-network fixed-point executor on staged activations: every convolution is the TMA-fed
    kernel (``staged.conv2d``), activations travel between layers as the fp32 NHWC operand the next
    convolution reads (clamped code + 0.5, physical halo) and, where a residual add, a pooling step
    or the classifier needs them, as int32 NHWC codes.  ReLU, residual add, the fp32 rounding and
    the next layer's quantiser clamp are fused into the convolution epilogues.  Same results as
    ``IntPipeline`` and ``ModuleNet``, bit for bit.

    Supports the steps of the ResNets (conv, maxpool, gap, linear after gap, copy, shortcutA);
    networks that flatten a spatial map into a classifier (the MNIST ones) stay on ``IntPipeline``.
    Needs act_integer_bits + act_fraction_bits <= 18 (the FP32-pipe bound) and right shifts only.
    """

    def __init__(self, net, weights, batch, device='cuda', use_graph=True):
        from . import staged as S
        self.S = S
        self.net, self.batch, self.device = net, batch, torch.device(device)
        self.I, self.F = net.act_integer_bits, net.act_fraction_bits
        if utils.code_bits(self.I, self.F) > 18:
            raise NotImplementedError("staged pipeline: activations wider than 18 bits")
        self.packed, self.bias = [], []
        for L, w in zip(net.layers, weights):
            self.packed.append(utils.compress_bits(w['shift'].float(), w['sign'].float(), device=self.device))
            self.bias.append((w['bias'] * (2 ** self.F)).int().to(self.device).contiguous())
        self.x_in = torch.empty((batch,) + net.in_shape, dtype=torch.float32, device=self.device)
        self.workspace = kernels.new_workspace(self.device)
        self._plan()
        self._n_launches = None
        self.graph = None
        if use_graph:
            self._capture()

    def _plan(self):
        net, dev, B = self.net, self.device, self.batch
        # pass 1: which forms of every tensor are read
        C, H, W = net.in_shape
        env = {'x': _Val(C, H, W)}
        first = env['x']
        vals, prog = [first], []
        after_gap = False
        for st in net.steps:
            op = st[0]
            if op == 'conv':
                li, o = st[1], st[2]
                L = net.layers[li]
                src = env[o.get('src', 'x')]
                src.halo = max(src.halo or 0, L.pad)
                res = env[o['add']] if o.get('add') else None
                if res is not None:
                    res.need_codes = True
                out = _Val(L.cout, (src.H + 2 * L.pad - L.k) // L.stride + 1, (src.W + 2 * L.pad - L.k) // L.stride + 1)
                vals.append(out)
                prog.append(('conv', li, src, res, out, bool(o.get('relu'))))
                env[o.get('dst', 'x')] = out
            elif op == 'maxpool':
                _, k, s_, p_ = st
                src = env['x']
                src.need_codes = True
                out = _Val(src.C, (src.H + 2 * p_ - k) // s_ + 1, (src.W + 2 * p_ - k) // s_ + 1)
                vals.append(out)
                prog.append(('maxpool', src, out, k, s_, p_))
                env['x'] = out
            elif op == 'gap':
                src = env['x']
                src.need_codes = True
                out = _Val(src.C, 1, 1)
                out.need_codes = out.flat = True
                vals.append(out)
                prog.append(('gap', src, out))
                env['x'] = out
                after_gap = True
            elif op == 'linear':
                if not after_gap:
                    raise NotImplementedError("staged pipeline: a classifier on a flattened spatial map")
                li, o = st[1], st[2]
                src = env['x']
                out = _Val(net.layers[li].cout, 1, 1)
                vals.append(out)
                prog.append(('linear', li, src, out, bool(o.get('relu'))))
                env['x'] = out
            elif op == 'copy':
                env[st[2]] = env[st[1]]
            elif op == 'shortcutA':
                src = env[st[1]]
                src.need_codes = True
                pad = st[3] // 4
                out = _Val(src.C + 2 * pad, (src.H + 1) // 2, (src.W + 1) // 2)
                out.need_codes = out.zero_init = True
                vals.append(out)
                prog.append(('shortcutA', src, out, pad))
                env[st[2]] = out
            elif op == 'flatten':
                if not after_gap:
                    raise NotImplementedError("staged pipeline: flatten of a spatial map")
            else:
                raise NotImplementedError(op)
        if first.need_codes or first.halo is None:
            raise NotImplementedError("staged pipeline: the network input must feed a convolution only")
        last = prog[-1]
        if last[0] != 'linear' or sum(1 for q in prog if q[0] == 'linear') != 1:
            raise NotImplementedError("staged pipeline: the last step must be the classifier")
        # pass 2: buffers
        for v in vals:
            if v.halo is not None:
                v.staged = self.S.StagedTensor(B, v.H, v.W, v.C, v.halo, dev)
            if v.need_codes and v is not last[3]:
                shape = (B, v.C) if v.flat else (B, v.H, v.W, v.C)
                v.codes = (torch.zeros if v.zero_init else torch.empty)(shape, dtype=torch.int32, device=dev)
        self.out = torch.empty((B, last[3].C), dtype=torch.float32, device=dev)
        self.first = first
        self.calls = [('stage',)] + prog

    def _launch_all(self):
        S, lib = self.S, _ffi.lib()
        import ctypes
        stream = torch.cuda.current_stream(self.device).cuda_stream
        I, F = self.I, self.F
        for c in self.calls:
            op = c[0]
            if op == 'stage':
                rc = lib.ds_stage_nchw(self.x_in.data_ptr(), _ffi.IN_F32_CONV, I, F, ctypes.byref(self.first.staged.c),
                                       stream)
                _ffi.check(rc, "stage_nchw")
            elif op == 'conv':
                _, li, src, res, out, relu = c
                L = self.net.layers[li]
                S.conv2d(src.staged, L.weight_shape, self.bias[li], self.packed[li], L.stride, L.pad,
                         act_integer_bits=I, act_fraction_bits=F, relu=relu, round_f32=True,
                         residual=res.codes if res is not None else None, out_codes=out.codes, out_staged=out.staged,
                         workspace=self.workspace)
            elif op == 'maxpool':
                _, src, out, k, s_, p_ = c
                rc = lib.ds_maxpool_nhwc(src.codes.data_ptr(), self.batch, src.H, src.W, src.C, k, s_, p_,
                                         out.codes.data_ptr() if out.codes is not None else None,
                                         ctypes.byref(out.staged.c) if out.staged is not None else None, I, F, stream)
                _ffi.check(rc, "maxpool_nhwc")
            elif op == 'gap':
                _, src, out = c
                rc = lib.ds_avgpool_fix_nhwc(src.codes.data_ptr(), out.codes.data_ptr(), self.batch, src.H, src.W, src.C,
                                             F, stream)
                _ffi.check(rc, "avgpool_fix_nhwc")
            elif op == 'linear':
                _, li, src, out, relu = c
                L, cw = self.net.layers[li], self.packed[li]
                fuse = kernels._fuse(_ffi.IN_I32, _ffi.OUT_F32, I, F, relu=relu, workspace=self.workspace)
                rc = lib.ds_linear_ex(src.codes.data_ptr(), cw.data.data_ptr(), self.bias[li].data_ptr(),
                                      self.out.data_ptr(), self.batch, L.cin, L.cout, cw.bits, cw.base, fuse, stream)
                _ffi.check(rc, "linear_ex")
            elif op == 'shortcutA':
                _, src, out, pad = c
                out.codes[..., pad:pad + src.C].copy_(src.codes[:, ::2, ::2, :])
