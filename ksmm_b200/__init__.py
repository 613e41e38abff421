"""ksmm_b200: Kronecker-sparse matrix multiplication for NVIDIA B200 (sm_100a).

A drop-in for the ``algo='kernel'`` path of the reference project: the same
``KSLinear`` / ``Kernel.forward`` Python surface over a C-ABI CUDA library
(``libksmm_cu.so``, declared in ``include/ksmm_cu.h``).
"""
from ._lib import KsmmError, LIB_PATH  # noqa: F401
from .interface import (KSLinear, KSLinearGroup, from_kernel_format_to_abcd,  # noqa: F401
                        from_kernel_format_to_dense, generate_factor)
from .kernel import (FactorFunction, Kernel, alloc_count, backward_input, backward_weights, chain_forward, check_device, default_choice, forward,  # noqa: F401
                     forward_ex, forward_fp8, grouped_chain_forward, launch_count, quantize_e4m3)

# the tuned table shipped with the package (choices that beat the heuristic on a B200); needs no device
from . import tuner as _tuner  # noqa: E402

_tuner.load_default()

__all__ = [
    "KSLinear", "KSLinearGroup", "grouped_chain_forward", "alloc_count", "Kernel", "FactorFunction",
    "backward_input", "backward_weights", "forward", "forward_ex", "forward_fp8", "chain_forward",
    "quantize_e4m3", "check_device", "launch_count", "default_choice", "generate_factor",
    "from_kernel_format_to_dense", "from_kernel_format_to_abcd", "KsmmError", "LIB_PATH",
]
