"""Host logic that needs no GPU: helpers with the reference's names, conversion, workload
descriptions, and the C ABI's symbol table and argument checks."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch
import torch.nn as nn

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_round_to_fixed_and_shift_sign_match_reference_golden(golden_dir):
    from deepshift_b200 import utils
    g = np.load(os.path.join(golden_dir, "glue_ref.npz"))
    v = torch.from_numpy(g["rtf_in"])
    for I, F in [(4, 12), (16, 16), (8, 8), (1, 7), (2, 3)]:
        assert np.array_equal(utils.round_to_fixed(v, I, F).numpy(), g[f"rtf_{I}_{F}"]), (I, F)
    shift, sign = utils.get_shift_and_sign(torch.from_numpy(g["gss_w"]))
    assert np.array_equal(sign.numpy(), g["gss_sign"])
    nz = g["gss_w"] != 0
    assert np.array_equal(shift.numpy()[nz], g["gss_shift"][nz])


def test_round_accepts_the_reference_spelling():
    from deepshift_b200 import utils
    x = torch.tensor([0.4, 1.5, -2.5])
    assert torch.equal(utils.round(x, 'determinstic'), utils.round(x, 'deterministic'))
    with pytest.raises(AssertionError):
        utils.round(x, 'nearest')


def test_module_signatures_match_reference():
    import inspect
    from deepshift_b200 import convert, kernels, modules
    lin = inspect.signature(modules.LinearShift.__init__)
    assert list(lin.parameters)[1:] == ['in_features', 'out_features', 'bias', 'check_grad', 'freeze_sign', 'use_kernel',
                                        'use_cuda', 'rounding', 'weight_bits', 'act_integer_bits', 'act_fraction_bits']
    conv = inspect.signature(modules.Conv2dShift.__init__)
    assert list(conv.parameters)[1:] == ['in_channels', 'out_channels', 'kernel_size', 'stride', 'padding', 'dilation',
                                         'groups', 'bias', 'padding_mode', 'check_grad', 'freeze_sign', 'use_kernel',
                                         'use_cuda', 'rounding', 'weight_bits', 'act_integer_bits', 'act_fraction_bits']
    assert conv.parameters['rounding'].default == 'determinstic'
    cts = inspect.signature(convert.convert_to_shift)
    assert list(cts.parameters) == ['model', 'shift_depth', 'shift_type', 'convert_all_linear', 'convert_weights',
                                    'freeze_sign', 'use_kernel', 'use_cuda', 'rounding', 'weight_bits',
                                    'act_integer_bits', 'act_fraction_bits']
    assert list(inspect.signature(kernels.linear).parameters)[:6] == ['input', 'shift', 'sign', 'bias', 'conc_weight',
                                                                       'use_cuda']
    assert list(inspect.signature(kernels.conv2d).parameters)[:10] == ['input', 'shift', 'sign', 'bias', 'conc_weight',
                                                                        'stride', 'padding', 'dilation', 'groups',
                                                                        'use_cuda']
    assert list(inspect.signature(kernels.compress_sign_and_shift).parameters) == ['shift', 'sign', 'comp_size', 'base',
                                                                                   'bits', 'row_length', 'num']


def test_convert_to_shift_structure_and_count():
    from deepshift_b200 import convert, modules
    model = nn.Sequential(nn.Conv2d(3, 8, 3, padding=1), nn.ReLU(),
                          nn.Sequential(nn.Conv2d(8, 8, 3, stride=2), nn.ReLU()), nn.Flatten(), nn.Linear(8, 4))
    model, count = convert.convert_to_shift(model, 1000, 'PS', convert_weights=True)
    assert count == 2  # convolutions only, as the reference counts with convert_all_linear=True
    assert convert.count_layer_type(model, modules.Conv2dShift) == 2
    assert convert.count_layer_type(model, modules.LinearShift) == 1
    c = model[0]
    assert c.stride == (1, 1) and c.padding == (1, 1) and c.shift.shape == (8, 3, 3, 3)
    assert c.shift_range == (-14, 0)
    assert torch.all(c.sign.data.abs() <= 1)
    # depth 1 converts the LAST convolution (the reference walks the children backwards)
    m2 = nn.Sequential(nn.Conv2d(3, 8, 3), nn.Conv2d(8, 8, 3))
    m2, n = convert.convert_to_shift(m2, 1, 'PS')
    assert n == 1 and type(m2[1]) is modules.Conv2dShift and type(m2[0]) is nn.Conv2d
    with pytest.raises(ValueError):
        convert.convert_to_shift(nn.Sequential(nn.Linear(2, 2)), 1, 'XYZ')


def test_round_shift_weights_rounds_parameters():
    from deepshift_b200 import convert, modules
    m = nn.Sequential(modules.LinearShift(6, 3, act_integer_bits=4, act_fraction_bits=12))
    m[0].shift.data.fill_(-2.4)
    m[0].sign.data.fill_(0.7)
    m[0].bias.data.fill_(0.12345)
    convert.round_shift_weights(m, act_integer_bits=4, act_fraction_bits=12)
    assert torch.all(m[0].shift.data == -2) and torch.all(m[0].sign.data == 1)
    assert torch.all(m[0].bias.data == np.floor(0.12345 * 4096) / 4096)


def test_float_path_forward_equals_dense_layers():
    """use_kernel=False: the layers are plain conv / linear with weights sign * 2^shift."""
    from deepshift_b200 import modules
    torch.manual_seed(0)
    conv = modules.Conv2dShift(3, 4, 3, padding=1, rounding='deterministic', act_integer_bits=8, act_fraction_bits=8)
    conv.shift.data = torch.randint(-6, 1, conv.shift.shape).float()
    conv.sign.data = torch.randint(-1, 2, conv.sign.shape).float()
    x = torch.randn(2, 3, 5, 5)
    from deepshift_b200 import utils
    w = (2.0 ** conv.shift.data) * conv.sign.data
    ref = torch.nn.functional.conv2d(utils.round_to_fixed(x, 8, 8), w, utils.round_to_fixed(conv.bias.data, 8, 8),
                                     padding=1)
    assert torch.equal(conv(x), ref)
    lin = modules.LinearShift(7, 3)
    lin.shift.data = torch.randint(-6, 1, lin.shift.shape).float()
    lin.sign.data = torch.randint(-1, 2, lin.sign.shape).float()
    x = torch.randn(4, 7)
    assert torch.equal(lin(x), torch.nn.functional.linear(x, (2.0 ** lin.shift.data) * lin.sign.data, lin.bias))


def test_kernel_mode_without_cuda_raises():
    from deepshift_b200 import kernels, modules
    lin = modules.LinearShift(4, 2, use_kernel=True, use_cuda=False)
    with pytest.raises(RuntimeError, match="no CPU kernel path"):
        lin(torch.zeros(1, 4))
    with pytest.raises(RuntimeError, match="no CPU kernel path"):
        kernels.linear(torch.zeros(1, 4, dtype=torch.int32), torch.zeros(2, 4), None, use_cuda=False)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        from deepshift_b200.utils import ConcWeight
        kernels.linear(torch.zeros(1, 4, dtype=torch.int32), torch.zeros(2, 4), None, None,
                       ConcWeight(torch.zeros(2, dtype=torch.int32), 0, 3))


# --------------------------------------------------------------------------- DeepShift-Q modules
def test_q_module_signatures_and_attributes_match_reference():
    import inspect
    from deepshift_b200 import modules_q
    lin = inspect.signature(modules_q.LinearShiftQ.__init__)
    assert list(lin.parameters)[1:] == ['in_features', 'out_features', 'bias', 'check_grad', 'use_kernel', 'use_cuda',
                                        'rounding', 'weight_bits', 'act_integer_bits', 'act_fraction_bits']
    conv = inspect.signature(modules_q.Conv2dShiftQ.__init__)
    assert list(conv.parameters)[1:] == ['in_channels', 'out_channels', 'kernel_size', 'stride', 'padding', 'dilation',
                                         'groups', 'bias', 'padding_mode', 'check_grad', 'use_kernel', 'use_cuda',
                                         'rounding', 'weight_bits', 'act_integer_bits', 'act_fraction_bits']
    m = modules_q.Conv2dShiftQ(3, 4, 3, weight_bits=5)
    assert m.shift_range == (-15, 0) and m.conc_weight is None and tuple(m.weight.shape) == (4, 3, 3, 3)
    assert modules_q.LinearShiftQ(5, 2, weight_bits=4).shift_range == (-7, 0)


def test_q_float_path_uses_clamped_power_of_two_weights():
    from deepshift_b200 import modules_q, utils
    torch.manual_seed(5)
    conv = modules_q.Conv2dShiftQ(3, 4, 3, padding=1, act_integer_bits=4, act_fraction_bits=12)
    conv.weight.data[0, 0, 0, 0] = 3.0       # clamped to 1
    conv.weight.data[0, 0, 0, 1] = -1e-9     # clamped to -2^-15
    conv.weight.data[0, 0, 0, 2] = 0.0       # stays 0
    x = torch.randn(2, 3, 5, 5) * 3
    y = conv(x)
    w = conv.weight.data
    assert w[0, 0, 0, 0] == 1.0 and w[0, 0, 0, 1] == -2.0 ** -15 and w[0, 0, 0, 2] == 0.0
    wq = utils.round_power_of_2(w)
    ref = torch.nn.functional.conv2d(utils.round_to_fixed(x, 4, 12), wq, utils.round_to_fixed(conv.bias.data, 4, 12),
                                     padding=1)
    assert torch.equal(y, ref)
    lin = modules_q.LinearShiftQ(6, 3, act_integer_bits=4, act_fraction_bits=12)
    xl = torch.randn(4, 6)
    refl = utils.round_to_fixed(xl, 4, 12).mm(utils.round_power_of_2(lin.weight.data).t()) + lin.bias.data
    assert torch.allclose(lin(xl), refl, atol=0, rtol=0)


def test_convert_to_shift_q_and_round_shift_weights():
    from deepshift_b200 import convert, modules_q
    torch.manual_seed(6)
    model = nn.Sequential(nn.Conv2d(3, 8, 3, padding=1), nn.ReLU(), nn.Flatten(), nn.Linear(8 * 36, 10))
    w0 = model[0].weight
    model, n = convert.convert_to_shift(model, 10, 'Q', act_integer_bits=4, act_fraction_bits=12)
    assert n == 1 and type(model[0]) is modules_q.Conv2dShiftQ and type(model[3]) is modules_q.LinearShiftQ
    assert model[0].weight is w0
    x = torch.randn(2, 3, 6, 6)
    y = model(x)
    rounded = convert.round_shift_weights(model, clone=True, act_integer_bits=4, act_fraction_bits=12)
    assert torch.equal(torch.log2(rounded[0].weight.data.abs()).frac(), torch.zeros_like(rounded[0].weight.data))
    assert torch.equal(rounded(x), y)
    with pytest.raises(ValueError):
        convert.convert_to_shift(nn.Sequential(nn.Linear(2, 2)), 1, 'X')


def test_q_golden_vectors_of_the_reference_match_the_oracle(oracle, golden_dir):
    """The reference's Conv2dShiftQ forward (use_kernel=True on its CPU kernel) restated: clamp
    |w| into [2^-15, 1], round to a power of two, quantise input and bias, integer convolution."""
    from deepshift_b200 import utils
    g = np.load(os.path.join(golden_dir, "q_ref.npz"))
    for i in range(int(g["n"])):
        w = utils.clampabs(torch.from_numpy(g[f"w{i}"].copy()), 2.0 ** -15, 1.0)
        shift, sign = utils.get_shift_and_sign(w)
        st = int(g[f"stride{i}"])
        ref = oracle.conv2d(oracle.to_fixed_conv(g[f"x{i}"], 4, 12), shift.numpy().astype(np.int32),
                            sign.numpy().astype(np.int32), oracle.to_fixed_conv(g[f"bias{i}"], 4, 12), (st, st), (0, 0))
        assert np.array_equal(oracle.from_fixed(ref, 12), g[f"y{i}"]), i


def test_q_kernel_mode_without_cuda_raises():
    from deepshift_b200 import modules_q
    with pytest.raises(RuntimeError, match="no CPU kernel path"):
        modules_q.LinearShiftQ(4, 2, use_kernel=True, use_cuda=False)(torch.zeros(1, 4))
    with pytest.raises(RuntimeError, match="no CPU kernel path"):
        modules_q.Conv2dShiftQ(1, 2, 3, use_kernel=True, use_cuda=False)(torch.zeros(1, 1, 4, 4))


# --------------------------------------------------------------------------- workloads
def test_workload_shift_op_counts():
    from deepshift_b200 import workloads as W
    assert W.mnist_fc().shift_ops() == 668672
    assert W.mnist_conv().shift_ops() == 2293000
    assert W.resnet20().shift_ops() == 40551040
    r18 = W.resnet18()
    assert r18.shift_ops() == 1814073344
    assert sum(1 for l in r18.layers if l.kind == 'conv') == 20 and sum(1 for l in r18.layers if l.kind == 'linear') == 1


def test_workload_generators_are_seeded_and_in_range():
    from deepshift_b200 import workloads as W
    net = W.mnist_conv()
    a, b = W.make_weights(net), W.make_weights(net)
    for wa, wb in zip(a, b):
        assert torch.equal(wa['shift'], wb['shift']) and torch.equal(wa['sign'], wb['sign'])
        assert int(wa['shift'].min()) >= -15 and int(wa['shift'].max()) <= 0
        assert set(wa['sign'].unique().tolist()) <= {-1, 0, 1}
        assert torch.equal(wa['bias'], torch.floor(wa['bias'] * 4096) / 4096)
    frac0 = float((a[2]['sign'] == 0).float().mean())
    assert 0.08 < frac0 < 0.12
    x0, x1 = W.make_input(net, 4, rank=0), W.make_input(net, 4, rank=1)
    assert x0.shape == (4, 1, 28, 28) and not torch.equal(x0, x1)
    assert float(x0.min()) >= -8.0 and float(x0.max()) <= 7.0


def test_oracle_network_runs_on_cpu(oracle):
    """The oracle executor alone (no GPU): shapes and determinism of a small ResNet-20 pass."""
    from deepshift_b200 import workloads as W
    from helpers import np_weights
    from oracle import reference_nets as R
    net = W.resnet20()
    ws = np_weights(W.make_weights(net))
    x = W.make_input(net, 2).numpy()
    y = R.forward(net, ws, x)
    assert y.shape == (2, 10) and y.dtype == np.float32
    assert np.array_equal(y, R.forward(net, ws, x))
    assert np.array_equal(y[:1], R.forward(net, ws, x[:1]))


# --------------------------------------------------------------------------- C ABI
def _declared_functions():
    text = open(os.path.join(ROOT, "include", "deepshift_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ds_[a-z0-9_]+)\s*\(", text)))


def _library():
    from deepshift_b200 import _build
    if not os.path.exists(_build.LIB_PATH):
        if _build.nvcc_path() is None:
            pytest.skip("CUDA library not built and no nvcc here")
        _build.build()
    return ctypes.CDLL(_build.LIB_PATH)


def test_library_exports_every_declared_symbol():
    lib = _library()
    names = _declared_functions()
    assert {"ds_linear_i32", "ds_conv2d_i32", "ds_compress", "ds_linear_ex", "ds_conv2d_ex", "ds_strerror"} <= set(names)
    for n in names:
        assert hasattr(lib, n), n


def test_argument_checks_need_no_gpu():
    """Bad arguments are rejected before any CUDA call."""
    from deepshift_b200 import _ffi
    lib = _ffi.lib()
    assert lib.ds_linear_i32(None, None, None, None, 4, 4, 4, 3, 0, 0, None) == 1
    assert lib.ds_linear_i32(None, None, None, None, 4, 0, 4, 3, 0, 0, None) == 1
    assert lib.ds_linear_i32(None, None, None, None, 0, 4, 4, 3, 0, 0, None) == 0  # empty batch
    assert lib.ds_conv2d_i32(None, None, None, None, 1, 1, 4, 4, 1, 5, 5, 1, 1, 0, 0, 3, 0, 0, None) == 1
    assert lib.ds_compress(None, None, None, 1, 1, 3, 0, None) == 1
    assert lib.ds_compress(16, 16, 16, 1, 1, 9, 0, None) == 2
    assert b"unsupported" in lib.ds_strerror(2)
    assert lib.ds_version() >= 100
    with pytest.raises(RuntimeError, match="bad argument"):
        _ffi.check(1, "probe")


# --------------------------------------------------------------------------- evaluation entry point
def test_evaluate_flags_follow_the_reference_drivers():
    from deepshift_b200 import evaluate
    a = evaluate.build_parser().parse_args(
        ['--dataset', 'imagenet', '-a', 'resnet18', '-s', '1000', '-st', 'PS', '-wb', '5', '-ab', '4', '12',
         '--use-kernel', 'True', '-e', '-b', '64', '/nonexistent'])
    assert (a.arch, a.shift_depth, a.shift_type, a.weight_bits, a.batch_size) == ('resnet18', 1000, 'PS', 5, 64)
    assert a.use_kernel is True and a.evaluate is True and [int(v) for v in a.activation_bits] == [4, 12]
    assert a.data == '/nonexistent'
    with pytest.raises(SystemExit):
        evaluate.main(['--dataset', 'mnist', '--type', 'linear'])            # no -e: inference only
    with pytest.raises(SystemExit):
        evaluate.main(['--dataset', 'mnist', '-e', '-ab', '4'])              # needs two values


def test_evaluate_runs_on_synthetic_data_and_writes_the_csv(tmp_path):
    """No dataset on the box: the seeded stand-in is announced, the whole user path runs (model, conversion
    to DeepShift-PS, validation loop, meters) on the fp32 path, and test_log.csv has the reference's columns."""
    import csv
    from deepshift_b200 import evaluate, modules
    lines = []
    row = evaluate.main(['--dataset', 'mnist', '--type', 'conv', '-s', '10', '-st', 'PS', '-ab', '4', '12', '-e',
                         '-b', '16', '--synthetic-images', '40', '--out-dir', str(tmp_path), '--desc', 't'],
                        out=lines.append)
    assert any("dataset unavailable on this box" in l for l in lines)
    assert any("4 layer(s) converted" in l for l in lines)
    loss, top1, top5, bt = row
    assert np.isfinite(loss) and 0.0 <= top1 <= top5 <= 100.0 and bt > 0
    path = tmp_path / 'mnist' / 'mnist_conv' / 'shift_10_PS_wb5_ab4.12_t' / 'test_log.csv'
    rows = list(csv.reader(open(path)))
    assert rows[0] == ['test_loss', 'test_top1_acc', 'test_top5_acc', 'test_time', 'cumulative_time']
    assert len(rows) == 2 and len(rows[1]) == 5
    assert evaluate.topk_correct(torch.tensor([[0.1, 0.9, 0.0], [0.5, 0.2, 0.3]]), torch.tensor([1, 2]), ks=(1, 2)) == [1, 2]
    m, _ = evaluate.build_model(evaluate.build_parser().parse_args(['--dataset', 'cifar10', '-a', 'resnet20', '-e']))
    assert sum(1 for x in m.modules() if isinstance(x, torch.nn.Conv2d)) == 19
    assert tuple(m(torch.zeros(2, 3, 32, 32)).shape) == (2, 10)


# --------------------------------------------------------------------------- the binding inside the reference tree
def test_reference_tree_calls_the_stub_with_the_right_arguments(monkeypatch):
    """The reference's own Python dispatcher (deepshift/kernels/kernels.py:10-74), imported from the
    reference checkout, driven over deepshift_b200/reference_binding/deepshift_cuda.py: a recording
    stand-in for the C library shows that every call reaches the C ABI with the argument list
    include/deepshift_b200.h declares.  (No GPU here: the same stub against the real library is a
    GPU test.)  Skipped where the reference checkout is not mounted."""
    import importlib
    import sys
    import types
    root = os.environ.get("DEEPSHIFT_REFERENCE") or os.path.join(os.path.dirname(ROOT), "reference")
    if not os.path.isdir(os.path.join(root, "pytorch", "deepshift")):
        pytest.skip("reference checkout not mounted")
    binding = os.path.join(ROOT, "deepshift_b200", "reference_binding")
    monkeypatch.syspath_prepend(os.path.join(root, "pytorch"))
    monkeypatch.syspath_prepend(binding)
    for name in [n for n in sys.modules if n == "deepshift" or n.startswith("deepshift.") or n in ("deepshift_cuda", "deepshift_cpu")]:
        monkeypatch.delitem(sys.modules, name)
    monkeypatch.setitem(sys.modules, "deepshift_cpu", types.ModuleType("deepshift_cpu"))
    stub = importlib.import_module("deepshift_cuda")
    assert os.path.dirname(stub.__file__) == binding
    calls = []

    class FakeLib:
        def __getattr__(self, name):
            def fn(*args):
                calls.append((name, args))
                return 0
            return fn
    monkeypatch.setattr(stub, "_lib", FakeLib())
    ref_kernels = importlib.import_module("deepshift.kernels.kernels")
    ref_utils = importlib.import_module("deepshift.utils")
    assert ref_kernels.deepshift_cuda is stub
    x = torch.zeros((3, 20), dtype=torch.int32)
    shift, bias = torch.zeros((7, 20)), torch.zeros(7, dtype=torch.int32)
    cw = ref_utils.ConcWeight(torch.zeros((7, 5), dtype=torch.int32), base=0, bits=6)
    out = ref_kernels.linear(x, shift, None, bias, cw, use_cuda=True)
    name, a = calls[-1]
    assert name == "ds_linear_i32" and tuple(out.shape) == (3, 7)
    assert a[:4] == (x.data_ptr(), cw.data.data_ptr(), bias.data_ptr(), out.data_ptr())
    assert a[4:] == (3, 20, 7, 6, 0, 0, None)          # M, K, N, bits, base, act_bits, stream
    xi = torch.zeros((2, 3, 8, 8), dtype=torch.int32)
    shift = torch.zeros((5, 3, 3, 3))
    cw = ref_utils.ConcWeight(torch.zeros((5, 7), dtype=torch.int32), base=0, bits=6)
    bias = torch.zeros(5, dtype=torch.int32)
    out = ref_kernels.conv2d(xi, shift, None, bias, cw, stride=(2, 2), padding=(1, 1), use_cuda=True)
    name, a = calls[-1]
    assert name == "ds_conv2d_i32" and tuple(out.shape) == (2, 5, 4, 4)
    # B, C, H, W of the tensor kernels.py has already padded; OC; window; strides; no padding; bits, base, act_bits
    assert a[4:] == (2, 3, 10, 10, 5, 3, 3, 2, 2, 0, 0, 6, 0, 0, None)
    assert a[1:4] == (cw.data.data_ptr(), bias.data_ptr(), out.data_ptr())


def test_library_flavours_have_their_own_files_and_flags():
    """The normal, bounds-checking and timing flavours are three libraries with three stamps; only the
    two diagnostic ones get an extra macro."""
    from deepshift_b200 import _build
    normal, checked, timing = _build._flavour(False, False), _build._flavour(True, False), _build._flavour(False, True)
    assert len({normal[0], checked[0], timing[0]}) == 3 and len({normal[1], checked[1], timing[1]}) == 3
    assert normal[2] == () and checked[2] == ("-DDS_BOUNDS_CHECK",) and timing[2] == ("-DDS_WS_TIMING",)
    assert len({normal[3], checked[3], timing[3]}) == 3
