"""Whole networks: module path (shift modules + fp32 glue) and the integer pipeline against the
CPU oracle, on sizes the oracle finishes in seconds; size-independent properties at full size."""
import numpy as np
import pytest
import torch

from helpers import np_weights

pytestmark = pytest.mark.gpu

SMALL = [('mnist_fc', 64, {}), ('mnist_conv', 24, {}), ('resnet20', 6, {}),
         ('resnet18', 3, dict(in_hw=64, num_classes=100))]


@pytest.mark.parametrize("name,batch,kw", SMALL, ids=[s[0] for s in SMALL])
def test_networks_bit_exact_against_oracle(oracle, cuda_device, name, batch, kw):
    from deepshift_b200 import workloads as W
    from oracle import reference_nets as R
    net = W.NETS[name](**kw)
    ws = W.make_weights(net)
    x = W.make_input(net, batch)
    ref = R.forward(net, np_weights(ws), x.numpy())
    with torch.no_grad():
        y_mod = W.ModuleNet(net, ws, cuda_device).eval()(x.to(cuda_device)).cpu().numpy()
        y_fused = W.ModuleNet(net, ws, cuda_device, fuse=True).eval()(x.to(cuda_device)).cpu().numpy()
    assert np.array_equal(y_mod, ref)
    assert np.array_equal(y_fused, ref)
    for graph in (False, True):
        pipe = W.IntPipeline(net, ws, batch, cuda_device, use_graph=graph)
        assert np.array_equal(pipe.run(x.to(cuda_device)).cpu().numpy(), ref), graph


def test_resnet18_full_resolution_sample_against_oracle(oracle, cuda_device):
    """Eight 224x224 images (the benchmark shape) through the CPU oracle against both product paths:
    the drop-in modules with fp32 glue and the integer pipeline, and the two against each other."""
    from deepshift_b200 import workloads as W
    from oracle import reference_nets as R
    net = W.resnet18()
    ws = W.make_weights(net)
    x = W.make_input(net, 8)
    ref = R.forward(net, np_weights(ws), x.numpy())
    pipe = W.IntPipeline(net, ws, 8, cuda_device)
    y_pipe = pipe.run(x.to(cuda_device)).cpu().numpy()
    with torch.no_grad():
        y_mod = W.ModuleNet(net, ws, cuda_device).eval()(x.to(cuda_device)).cpu().numpy()
        y_fused = W.ModuleNet(net, ws, cuda_device, fuse=True).eval()(x.to(cuda_device)).cpu().numpy()
    assert np.array_equal(y_pipe, ref)
    assert np.array_equal(y_mod, ref)
    assert np.array_equal(y_fused, ref)
    assert np.array_equal(y_mod, y_pipe)


def test_resnet18_benchmark_batch_properties(cuda_device):
    """Batch 256 at 224x224 (the benchmark shape): a replay gives identical logits, and every image
    of the batch gets the logits it gets when run in a batch of 8 -- images are independent."""
    from deepshift_b200 import workloads as W
    net = W.resnet18()
    ws = W.make_weights(net)
    x = W.make_input(net, 256).to(cuda_device)
    pipe = W.IntPipeline(net, ws, 256, cuda_device)
    y = pipe.run(x).clone()
    assert torch.equal(pipe.run(x), y)
    assert torch.isfinite(y).all()
    small = W.IntPipeline(net, ws, 8, cuda_device)
    for b0 in (0, 128, 248):
        assert torch.equal(small.run(x[b0:b0 + 8]), y[b0:b0 + 8]), b0


def test_evaluate_entry_point_with_kernels(cuda_device, tmp_path):
    """`-e --use-kernel True` on two batches of MNIST-shaped and one of CIFAR-shaped stand-in data:
    the converted model runs on the CUDA kernels, and agrees with its own fp32 path on nearly every
    prediction (they differ only by the fixed-point rounding of the activations)."""
    from deepshift_b200 import evaluate
    common = ['-s', '100', '-st', 'PS', '-wb', '5', '-ab', '4', '12', '-e', '--out-dir', str(tmp_path)]
    for ds, extra in (('mnist', ['--type', 'conv', '-b', '32', '--synthetic-images', '64']),
                      ('cifar10', ['-a', 'resnet20', '-b', '16', '--synthetic-images', '16'])):
        rows = {}
        for uk in ('True', 'False'):
            lines = []
            rows[uk] = evaluate.main(['--dataset', ds] + extra + common + ['--use-kernel', uk, '--desc', uk],
                                     out=lines.append)
            assert any("dataset unavailable on this box" in l for l in lines)
        assert np.isfinite(rows['True'][0]) and abs(rows['True'][0] - rows['False'][0]) < 0.05 * max(1.0, rows['False'][0])
