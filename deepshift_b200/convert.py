"""Model conversion with the reference's signatures (pytorch/deepshift/convert.py:11,83,107).

Both branches are implemented: ``shift_type='PS'`` (the path under acceleration) and
``shift_type='Q'``, whose modules round their fp32 weights to powers of two on the fly and pack
them on first use (modules_q.py).  Unlike the reference, a converted LinearShift gets its packed weights whenever
``use_kernel`` is set (convert.py:39-40 packs them only under ``convert_weights``), and
``round_shift_weights`` re-packs after rounding so that ``conc_weight`` always matches the
module's parameters.
"""
import copy

import torch.nn as nn

from . import modules, modules_q, utils


def _pack(module):
    module.conc_weight = utils.compress_bits(module.shift.data.round(), module.sign.data.round().sign())


def convert_to_shift(model, shift_depth, shift_type, convert_all_linear=True, convert_weights=False,
                     freeze_sign=False, use_kernel=False, use_cuda=True, rounding='deterministic',
                     weight_bits=5, act_integer_bits=16, act_fraction_bits=16):
    if shift_type not in ('PS', 'Q'):
        raise ValueError('Unsupported shift_type argument: ', shift_type)
    conversion_count = 0
    # The reference walks the children from the last one backwards (convert.py:13).
    for name, module in reversed(model._modules.items()):
        if len(list(module.children())) > 0:
            model._modules[name], num_converted = convert_to_shift(
                model=module, shift_depth=shift_depth - conversion_count, shift_type=shift_type,
                convert_all_linear=convert_all_linear, convert_weights=convert_weights,
                freeze_sign=freeze_sign, use_kernel=use_kernel, use_cuda=use_cuda, rounding=rounding,
                weight_bits=weight_bits, act_integer_bits=act_integer_bits,
                act_fraction_bits=act_fraction_bits)
            conversion_count += num_converted
        if shift_type == 'Q' and type(module) == nn.Linear and (convert_all_linear == True or
                                                                 conversion_count < shift_depth):
            # convert.py:22-30; the weights are packed by the module on first use, after its clamp
            shift_linear = modules_q.LinearShiftQ(
                module.in_features, module.out_features, module.bias is not None, use_kernel=use_kernel,
                use_cuda=use_cuda, rounding=rounding, weight_bits=weight_bits,
                act_integer_bits=act_integer_bits, act_fraction_bits=act_fraction_bits)
            shift_linear.weight = module.weight
            if module.bias is not None:
                shift_linear.bias.data = utils.round_to_fixed(module.bias.data, integer_bits=act_integer_bits,
                                                              fraction_bits=act_fraction_bits)
            model._modules[name] = shift_linear
            if convert_all_linear == False:
                conversion_count += 1
        elif shift_type == 'Q' and type(module) == nn.Conv2d and conversion_count < shift_depth:
            # convert.py:51-62
            shift_conv2d = modules_q.Conv2dShiftQ(
                module.in_channels, module.out_channels, module.kernel_size, module.stride, module.padding,
                module.dilation, module.groups, module.bias is not None, module.padding_mode,
                use_kernel=use_kernel, use_cuda=use_cuda, rounding=rounding, weight_bits=weight_bits,
                act_integer_bits=act_integer_bits, act_fraction_bits=act_fraction_bits)
            shift_conv2d.weight = module.weight
            if module.bias is not None:
                shift_conv2d.bias.data = utils.round_to_fixed(module.bias.data, integer_bits=act_integer_bits,
                                                              fraction_bits=act_fraction_bits)
            model._modules[name] = shift_conv2d
            conversion_count += 1
        if shift_type == 'Q':
            continue

        if type(module) == nn.Linear and (convert_all_linear == True or conversion_count < shift_depth):
            linear = module
            shift_linear = modules.LinearShift(
                module.in_features, module.out_features, module.bias is not None, freeze_sign=freeze_sign,
                use_kernel=use_kernel, use_cuda=use_cuda, rounding=rounding, weight_bits=weight_bits,
                act_integer_bits=act_integer_bits, act_fraction_bits=act_fraction_bits)
            if convert_weights == True:
                shift_linear.shift.data, shift_linear.sign.data = utils.get_shift_and_sign(linear.weight)
                shift_linear.bias = linear.bias
            if use_cuda == True and use_kernel == True:
                _pack(shift_linear)
            model._modules[name] = shift_linear
            if convert_all_linear == False:
                conversion_count += 1

        if type(module) == nn.Conv2d and conversion_count < shift_depth:
            conv2d = module
            shift_conv2d = modules.Conv2dShift(
                module.in_channels, module.out_channels, module.kernel_size, module.stride, module.padding,
                module.dilation, module.groups, module.bias is not None, module.padding_mode,
                freeze_sign=freeze_sign, use_kernel=use_kernel, use_cuda=use_cuda, rounding=rounding,
                weight_bits=weight_bits, act_integer_bits=act_integer_bits,
                act_fraction_bits=act_fraction_bits)
            if convert_weights == True:
                shift_conv2d.shift.data, shift_conv2d.sign.data = utils.get_shift_and_sign(conv2d.weight)
                shift_conv2d.bias = conv2d.bias
            if use_cuda == True and use_kernel == True:
                _pack(shift_conv2d)
            model._modules[name] = shift_conv2d
            conversion_count += 1

    return model, conversion_count


def round_shift_weights(model, clone=False, weight_bits=5, act_integer_bits=16, act_fraction_bits=16):
    if clone:
        model = copy.deepcopy(model)
    for name, module in reversed(model._modules.items()):
        if len(list(module.children())) > 0:
            model._modules[name] = round_shift_weights(model=module, weight_bits=weight_bits,
                                                       act_integer_bits=act_integer_bits,
                                                       act_fraction_bits=act_fraction_bits)
        if type(module) == modules.LinearShift or type(module) == modules.Conv2dShift:
            module.shift.data = module.shift.round()
            module.sign.data = module.sign.round().sign()
            if module.bias is not None:
                module.bias.data = utils.round_to_fixed(module.bias, integer_bits=act_integer_bits,
                                                        fraction_bits=act_fraction_bits)
            if module.use_kernel and module.use_cuda and module.conc_weight is not None:
                _pack(module)
        elif type(module) == modules_q.LinearShiftQ or type(module) == modules_q.Conv2dShiftQ:
            # convert.py:98-104; the module re-packs when it next runs (its cache is dropped here)
            module.weight.data = utils.clampabs(module.weight.data, 2 ** module.shift_range[0],
                                                2 ** module.shift_range[1])
            module.weight.data = utils.round_power_of_2(module.weight.data)
            if module.bias is not None:
                module.bias.data = utils.round_to_fixed(module.bias.data, integer_bits=act_integer_bits,
                                                        fraction_bits=act_fraction_bits)
            module.conc_weight = None
    return model


def count_layer_type(model, layer_type):
    count = 0
    for name, module in model._modules.items():
        if len(list(module.children())) > 0:
            count += count_layer_type(model=module, layer_type=layer_type)
        if type(module) == layer_type:
            count += 1
    return count
