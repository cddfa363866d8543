"""lib_b200 — B200-native fused dequantize-and-multiply over GGUF block-quantized
weights (Q8_0, Q4_0, Q4_K, and the Q2_K / IQ2_XXS super-block formats), behind the Go-facing API of the reference's
lm/quant and lm/moe packages.

The product is `libqmatmul.so` (C ABI in include/qmatmul.h) with its sm_100a
cubins. This Python package is the harness-side binding of that ABI: it loads
the library with ctypes and mirrors the reference's function names. It has no
CPU implementation of any operation; on a machine without a B200 the library
still loads (symbols can be inspected) but `Context()` raises.
"""
from . import _capi  # noqa: F401
from ._capi import Context, QmError, lib, Q4_0, Q8_0, Q2_K, Q4_K, IQ2_XXS  # noqa: F401
