"""deepshift_b200: DeepShift's ``use_kernel`` inference path on NVIDIA B200 (sm_100a).

Public surface mirrors the reference package ``deepshift``: ``modules`` (LinearShift,
Conv2dShift), ``convert`` (convert_to_shift, round_shift_weights, count_layer_type),
``modules_q`` (LinearShiftQ, Conv2dShiftQ), ``utils`` (round_to_fixed, ConcWeight, compress_bits, ...) and ``kernels`` (linear, conv2d,
compress_sign_and_shift).  Submodules are imported on first use so that importing the
package does not need a GPU.
"""
__all__ = ["kernels", "utils", "modules", "modules_q", "convert", "ste"]
__version__ = "0.1.0"
