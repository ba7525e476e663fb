"""CPU evaluation of the benchmark networks with the oracle kernels (TEST INFRASTRUCTURE ONLY).

Follows, step by step, what the reference's modules do with ``use_kernel=True`` on a network
built from ``Conv2dShift`` / ``LinearShift`` (pytorch/deepshift/modules.py:23-31,150-162,312-340)
and fp32 glue: quantise the fp32 input (conv: floor + clamp, linear: truncation), run the integer
kernel (``oracle.conv2d`` / ``oracle.linear``), convert back with ``out.float() / 2**F``, then
ReLU / residual add / pooling in float32 numpy.  The network description is the plain-data
``Net`` of deepshift_b200.workloads (steps and layer shapes only; no product code is executed).
"""
import numpy as np

from . import oracle as O


def _max_pool(x, k, s, p):
    B, C, H, W = x.shape
    OH, OW = (H + 2 * p - k) // s + 1, (W + 2 * p - k) // s + 1
    xp = np.full((B, C, H + 2 * p, W + 2 * p), -np.inf, dtype=np.float32)
    xp[:, :, p:p + H, p:p + W] = x
    out = np.full((B, C, OH, OW), -np.inf, dtype=np.float32)
    for kh in range(k):
        for kw in range(k):
            out = np.maximum(out, xp[:, :, kh:kh + s * OH:s, kw:kw + s * OW:s])
    return out


def forward(net, weights, x):
    """net: workloads.Net; weights: list of dicts with numpy 'shift', 'sign' (int32) and 'bias'
    (float32); x: float32 [B,C,H,W].  Returns float32 logits."""
    I, F = net.act_integer_bits, net.act_fraction_bits
    t = {'x': np.asarray(x, dtype=np.float32)}
    for st in net.steps:
        op = st[0]
        if op == 'conv':
            li, o = st[1], st[2]
            L, w = net.layers[li], weights[li]
            xin = t[o.get('src', 'x')]
            xi = O.to_fixed_conv(xin, I, F)
            bi = O.to_fixed_conv(w['bias'], I, F)
            yi = O.conv2d(xi, w['shift'], w['sign'], bi, (L.stride, L.stride), (L.pad, L.pad))
            y = O.from_fixed(yi, F)
            if o.get('add'):
                y = (y + t[o['add']]).astype(np.float32)
            if o.get('relu'):
                y = np.maximum(y, np.float32(0))
            t[o.get('dst', 'x')] = y
        elif op == 'linear':
            li, o = st[1], st[2]
            w = weights[li]
            xi = O.to_fixed_linear(t['x'].reshape(t['x'].shape[0], -1), F)
            bi = O.to_fixed_linear(w['bias'], F)
            y = O.from_fixed(O.linear(xi, w['shift'], w['sign'], bi), F)
            t['x'] = np.maximum(y, np.float32(0)) if o.get('relu') else y
        elif op == 'maxpool':
            t['x'] = _max_pool(t['x'], st[1], st[2], st[3])
        elif op == 'gap':
            t['x'] = O.global_avg(t['x'])
        elif op == 'flatten':
            t['x'] = t['x'].reshape(t['x'].shape[0], -1)
        elif op == 'copy':
            t[st[2]] = t[st[1]]
        elif op == 'shortcutA':
            xs = t[st[1]][:, :, ::2, ::2]
            p = st[3] // 4
            t[st[2]] = np.pad(xs, ((0, 0), (p, p), (0, 0), (0, 0)))
    return t['x']
