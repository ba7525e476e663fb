"""Evaluation entry point of the ``use_kernel`` path: what the reference's three drivers do with
``-e --use-kernel True`` (pytorch/mnist.py:75-91,317-323, pytorch/cifar10.py:594-633,
pytorch/imagenet.py:609-649), in one program.

    python -m deepshift_b200.evaluate --dataset imagenet -a resnet18 -s 1000 -st PS -wb 5 -ab 4 12 \\
        --use-kernel True -e -b 256 [--weights checkpoint.pth] [DIR]

builds the model, converts it with ``convert_to_shift`` (kernel-relevant flags of
imagenet.py:50-136 / mnist.py:99-148 under their own names), runs the validation loop with loss,
top-1 / top-5 meters and batch time, and writes ``test_log.csv`` with the reference's columns
(imagenet.py:469-472) into the run directory.

Data: with ``DIR`` holding the dataset in torchvision's layout the real validation set is read
(MNIST / CIFAR-10 test split, ImageNet ``val/`` folder).  Without it -- there is no dataset on a
box without network -- seeded synthetic tensors of the dataset's shape and normalisation with
random labels stand in, and the program says so: the run then exercises every step of the user
path and measures time, while its accuracy figures mean nothing.  Training is not part of this
package: without ``-e`` the program refuses, as the reference does for ``--use-kernel``
(mnist.py:157-158).
"""
import argparse
import csv
import os
import time

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import convert

DATASETS = {  # name: (input shape, classes, mean, std, default number of synthetic images)
    'mnist': ((1, 28, 28), 10, (0.1307,), (0.3081,), 2048),
    'cifar10': ((3, 32, 32), 10, (0.4914, 0.4822, 0.4465), (0.2023, 0.1994, 0.2010), 2048),
    'imagenet': ((3, 224, 224), 1000, (0.485, 0.456, 0.406), (0.229, 0.224, 0.225), 512),
}


def _flag(v):
    if isinstance(v, bool):
        return v
    if v.lower() in ('y', 'yes', 't', 'true', 'on', '1'):
        return True
    if v.lower() in ('n', 'no', 'f', 'false', 'off', '0'):
        return False
    raise argparse.ArgumentTypeError("expected a truth value, got %r" % v)


def build_parser():
    p = argparse.ArgumentParser(description="DeepShift use_kernel evaluation on the B200 kernels")
    p.add_argument('data', metavar='DIR', nargs='?', default=None, help='path to dataset (optional)')
    p.add_argument('--dataset', default='imagenet', choices=sorted(DATASETS))
    p.add_argument('-a', '--arch', default=None,
                   help='imagenet: a torchvision model name (default resnet18); cifar10: resnet20/32/44/56; '
                        'mnist: linear | conv (also --type)')
    p.add_argument('--type', default=None, choices=['linear', 'conv'], help='mnist model (mnist.py:105)')
    p.add_argument('--weights', default='', metavar='WEIGHTS_PATH', help='state dict (or checkpoint with "state_dict") to load')
    p.add_argument('-s', '--shift-depth', type=int, default=0, help='how many layers to convert to shift')
    p.add_argument('-st', '--shift-type', default='PS', choices=['Q', 'PS'])
    p.add_argument('-r', '--rounding', default='deterministic', choices=['deterministic', 'stochastic'])
    p.add_argument('-wb', '--weight-bits', type=int, default=5)
    p.add_argument('-ab', '--activation-bits', nargs='+', default=[16, 16],
                   help='integer and fraction bits of the fixed-point activations')
    p.add_argument('-b', '--batch-size', '--test-batch-size', dest='batch_size', default=256, type=int)
    p.add_argument('-p', '--print-freq', default=10, type=int)
    p.add_argument('-e', '--evaluate', action='store_true', help='only evaluate (the only mode there is)')
    p.add_argument('--use-kernel', type=_flag, default=False, help='run the shift layers on the custom kernels')
    p.add_argument('--seed', default=1, type=int)
    p.add_argument('--gpu', default=0, type=int)
    p.add_argument('--synthetic-images', default=None, type=int, help='size of the stand-in dataset')
    p.add_argument('--max-batches', default=None, type=int, help='stop after this many batches')
    p.add_argument('--desc', default=None, help='suffix of the run directory')
    p.add_argument('--out-dir', default='models', help='where run directories are made')
    return p


# ------------------------------------------------------------------------------------------------ models
class LinearMNIST(nn.Module):
    """784-512-512-10 perceptron (mnist.py:23-39); log-softmax output."""

    def __init__(self):
        super().__init__()
        self.fc1, self.fc2, self.fc3 = nn.Linear(784, 512), nn.Linear(512, 512), nn.Linear(512, 10)
        self.dropout1, self.dropout2 = nn.Dropout(0.2), nn.Dropout(0.2)

    def forward(self, x):
        x = self.dropout1(F.relu(self.fc1(x.flatten(1))))
        x = self.dropout2(F.relu(self.fc2(x)))
        return F.log_softmax(self.fc3(x), dim=1)


class ConvMNIST(nn.Module):
    """Two 5x5 convolutions with 2x2 pooling, then 800-500-10 (mnist.py:41-57)."""

    def __init__(self):
        super().__init__()
        self.conv1, self.conv2 = nn.Conv2d(1, 20, 5, 1), nn.Conv2d(20, 50, 5, 1)
        self.fc1, self.fc2 = nn.Linear(800, 500), nn.Linear(500, 10)

    def forward(self, x):
        x = F.max_pool2d(F.relu(self.conv1(x)), 2, 2)
        x = F.max_pool2d(F.relu(self.conv2(x)), 2, 2)
        return F.log_softmax(self.fc2(F.relu(self.fc1(x.flatten(1)))), dim=1)


class _BlockA(nn.Module):
    """CIFAR basic block with the parameter-free option-A shortcut (cifar10_models/resnet.py:23-58)."""

    def __init__(self, cin, planes, stride):
        super().__init__()
        self.conv1 = nn.Conv2d(cin, planes, 3, stride, 1, bias=False)
        self.bn1 = nn.BatchNorm2d(planes)
        self.conv2 = nn.Conv2d(planes, planes, 3, 1, 1, bias=False)
        self.bn2 = nn.BatchNorm2d(planes)
        self.pad = planes // 4 if (stride != 1 or cin != planes) else None

    def forward(self, x):
        out = F.relu(self.bn1(self.conv1(x)))
        out = self.bn2(self.conv2(out))
        sc = x if self.pad is None else F.pad(x[:, :, ::2, ::2], (0, 0, 0, 0, self.pad, self.pad))
        return F.relu(out + sc)


class CifarResNet(nn.Module):
    """6n+2-layer CIFAR ResNet (cifar10_models/resnet.py:92-140)."""

    def __init__(self, n, num_classes=10):
        super().__init__()
        self.conv1, self.bn1 = nn.Conv2d(3, 16, 3, 1, 1, bias=False), nn.BatchNorm2d(16)
        blocks, cin = [], 16
        for planes, stride in ((16, 1), (32, 2), (64, 2)):
            for b in range(n):
                blocks.append(_BlockA(cin, planes, stride if b == 0 else 1))
                cin = planes
        self.layers = nn.Sequential(*blocks)
        self.linear = nn.Linear(64, num_classes)

    def forward(self, x):
        x = self.layers(F.relu(self.bn1(self.conv1(x))))
        return self.linear(F.avg_pool2d(x, x.size(3)).flatten(1))


def build_model(args):
    if args.dataset == 'mnist':
        kind = args.type or args.arch or 'linear'
        if kind not in ('linear', 'conv'):
            raise SystemExit("mnist: --type linear | conv")
        return LinearMNIST() if kind == 'linear' else ConvMNIST(), 'mnist_' + kind
    if args.dataset == 'cifar10':
        arch = args.arch or 'resnet20'
        depth = {'resnet20': 3, 'resnet32': 5, 'resnet44': 7, 'resnet56': 9}.get(arch)
        if depth is None:
            raise SystemExit("cifar10: -a resnet20 | resnet32 | resnet44 | resnet56")
        return CifarResNet(depth), arch
    arch = args.arch or 'resnet18'
    import torchvision.models as tvm
    if not hasattr(tvm, arch):
        raise SystemExit("imagenet: unknown torchvision model %r" % arch)
    return getattr(tvm, arch)(weights=None), arch


# ------------------------------------------------------------------------------------------------ data
class SyntheticSet(torch.utils.data.Dataset):
    """Seeded stand-in: uniform [0,1) pixels normalised with the dataset's mean and std, random labels."""

    def __init__(self, name, n, seed):
        shape, classes, mean, std, default_n = DATASETS[name]
        n = n or default_n
        g = torch.Generator().manual_seed(seed)
        x = torch.rand((n,) + shape, generator=g)
        self.x = (x - torch.tensor(mean).view(-1, 1, 1)) / torch.tensor(std).view(-1, 1, 1)
        self.y = torch.randint(0, classes, (n,), generator=g)

    def __len__(self):
        return self.x.shape[0]

    def __getitem__(self, i):
        return self.x[i], self.y[i]


def build_loader(args):
    """(DataLoader, description).  Real data only when DIR holds it; nothing is ever downloaded."""
    shape, classes, mean, std, _ = DATASETS[args.dataset]
    data = None
    if args.data and os.path.isdir(args.data):
        try:
            import torchvision.datasets as tvd
            import torchvision.transforms as T
            norm = T.Normalize(mean, std)
            if args.dataset == 'mnist':
                data = tvd.MNIST(args.data, train=False, download=False, transform=T.Compose([T.ToTensor(), norm]))
            elif args.dataset == 'cifar10':
                data = tvd.CIFAR10(args.data, train=False, download=False, transform=T.Compose([T.ToTensor(), norm]))
            else:
                val = os.path.join(args.data, 'val')
                if os.path.isdir(val):
                    data = tvd.ImageFolder(val, T.Compose([T.Resize(256), T.CenterCrop(224), T.ToTensor(), norm]))
        except (RuntimeError, OSError, ImportError):
            data = None
    if data is not None:
        what = "%s validation data from %s (%d images)" % (args.dataset, args.data, len(data))
    else:
        data = SyntheticSet(args.dataset, args.synthetic_images, args.seed)
        what = ("dataset unavailable on this box: %d seeded synthetic %s-shaped images with random labels stand in "
                "(accuracy figures are meaningless)" % (len(data), args.dataset))
    return torch.utils.data.DataLoader(data, batch_size=args.batch_size, shuffle=False, pin_memory=True), what


# ------------------------------------------------------------------------------------------------ meters
class Meter:
    """Running average of one quantity."""

    def __init__(self):
        self.total, self.count, self.last = 0.0, 0, 0.0

    def add(self, value, n=1):
        self.last = float(value)
        self.total += float(value) * n
        self.count += n

    @property
    def mean(self):
        return self.total / max(self.count, 1)


def topk_correct(output, target, ks=(1, 5)):
    """Number of samples whose label is among the k highest outputs, for each k."""
    kmax = min(max(ks), output.shape[1])
    pred = output.topk(kmax, dim=1).indices
    hit = pred.eq(target.view(-1, 1))
    return [int(hit[:, :min(k, kmax)].any(dim=1).sum()) for k in ks]


def validate(loader, model, device, log_softmax_output, print_freq=10, max_batches=None, out=print):
    """The reference's validation loop (imagenet.py:609-649): returns (loss, top-1 %, top-5 %, mean
    batch time in seconds)."""
    loss_m, top1, top5, time_m = Meter(), Meter(), Meter(), Meter()
    model.eval()
    with torch.no_grad():
        end = time.time()
        for i, (x, y) in enumerate(loader):
            if max_batches is not None and i >= max_batches:
                break
            x, y = x.to(device, non_blocking=True), y.to(device, non_blocking=True)
            output = model(x)
            loss = F.nll_loss(output, y) if log_softmax_output else F.cross_entropy(output, y)
            c1, c5 = topk_correct(output, y)
            n = x.shape[0]
            loss_m.add(loss.item(), n)
            top1.add(100.0 * c1 / n, n)
            top5.add(100.0 * c5 / n, n)
            if device.type == 'cuda':
                torch.cuda.synchronize(device)
            time_m.add(time.time() - end)
            end = time.time()
            if print_freq and i % print_freq == 0:
                out("Test: [%d/%d]  Time %.3f (%.3f)  Loss %.4e (%.4e)  Acc@1 %.2f (%.2f)  Acc@5 %.2f (%.2f)"
                    % (i, len(loader), time_m.last, time_m.mean, loss_m.last, loss_m.mean, top1.last, top1.mean,
                       top5.last, top5.mean))
    out(" * Acc@1 %.3f Acc@5 %.3f" % (top1.mean, top5.mean))
    return loss_m.mean, top1.mean, top5.mean, time_m.mean


def run_dir(args, arch):
    """models/<dataset>/<arch>/shift_<depth>[_<type>_wb<bits>][_<desc>], in the spirit of imagenet.py:296-329."""
    name = "shift_%d" % args.shift_depth if args.shift_depth > 0 else "shift_0"
    if args.shift_depth > 0:
        name += "_%s_wb%d_ab%s.%s" % (args.shift_type, args.weight_bits, args.activation_bits[0], args.activation_bits[1])
    if args.desc:
        name += "_" + args.desc
    d = os.path.join(args.out_dir, args.dataset, arch, name)
    os.makedirs(d, exist_ok=True)
    return d


def main(argv=None, out=print):
    args = build_parser().parse_args(argv)
    if len(args.activation_bits) != 2:
        raise SystemExit("activation-bits needs two values: integer bits and fraction bits, e.g. '4 12'")
    I, Fb = int(args.activation_bits[0]), int(args.activation_bits[1])
    if not args.evaluate:
        raise SystemExit("this package runs inference only: pass -e / --evaluate "
                         "(the custom kernels support inference, not training)")
    torch.manual_seed(args.seed)
    if args.use_kernel and not torch.cuda.is_available():
        raise SystemExit("--use-kernel True needs a CUDA device: the shift kernels have no CPU path")
    device = torch.device('cuda', args.gpu) if torch.cuda.is_available() else torch.device('cpu')
    model, arch = build_model(args)
    if args.weights:
        state = torch.load(args.weights, map_location='cpu')
        model.load_state_dict(state.get('state_dict', state) if isinstance(state, dict) else state)
    converted = 0
    if args.shift_depth > 0:
        model, _ = convert.convert_to_shift(
            model, args.shift_depth, args.shift_type, convert_all_linear=(args.dataset != 'imagenet'),
            convert_weights=True, use_kernel=args.use_kernel, use_cuda=device.type == 'cuda', rounding=args.rounding,
            weight_bits=args.weight_bits, act_integer_bits=I, act_fraction_bits=Fb)
        model = convert.round_shift_weights(model, weight_bits=args.weight_bits, act_integer_bits=I,
                                            act_fraction_bits=Fb)
    from . import modules, modules_q
    converted = sum(convert.count_layer_type(model, t) for t in (modules.LinearShift, modules.Conv2dShift,
                                                                 modules_q.LinearShiftQ, modules_q.Conv2dShiftQ))
    model = model.to(device)
    loader, what = build_loader(args)
    out("%s: %s, %d layer(s) converted to DeepShift-%s, use_kernel=%s, activations %d.%d, %d-bit weights"
        % (args.dataset, arch, converted, args.shift_type, args.use_kernel, I, Fb, args.weight_bits))
    out(what)
    t0 = time.time()
    row = validate(loader, model, device, log_softmax_output=(args.dataset == 'mnist'), print_freq=args.print_freq,
                   max_batches=args.max_batches, out=out)
    d = run_dir(args, arch)
    with open(os.path.join(d, "test_log.csv"), "w", newline='') as fh:
        w = csv.writer(fh)
        w.writerow(['test_loss', 'test_top1_acc', 'test_top5_acc', 'test_time', 'cumulative_time'])
        w.writerow(list(row) + [time.time() - t0])
    out("log: " + os.path.join(d, "test_log.csv"))
    return row


if __name__ == "__main__":
    main()
