"""Host-side mirror of the reference's lm/quant API over the CUDA library.

Names, argument meaning and error cases follow lm/quant/quant.go and
lm/quant/kquant.go; the work is done by libqmatmul.so on the GPU. MatVec is
the new entry point of this path (the reference package only dequantizes); it
keeps the package's voice: GGUF block bytes in, float32 out, `quant:` errors.
"""
import numpy as np

from . import _capi
from ._capi import Q4_0, Q8_0, Q2_K, Q4_K, IQ2_XXS, QmError  # noqa: F401

BlockSize = 32          # lm/quant/quant.go:12
SuperBlockSize = 256    # lm/quant/kquant.go:12
FormatQ4_0, FormatQ8_0, FormatQ2_K, FormatQ4_K, FormatIQ2_XXS = "Q4_0", "Q8_0", "Q2_K", "Q4_K", "IQ2_XXS"
_FMT = {FormatQ4_0: Q4_0, FormatQ8_0: Q8_0, FormatQ2_K: Q2_K, FormatQ4_K: Q4_K, FormatIQ2_XXS: IQ2_XXS}

_default_ctx = None


def default_context():
    global _default_ctx
    if _default_ctx is None:
        _default_ctx = _capi.Context(0)
    return _default_ctx


def DequantizeQ4_0(data, numElements, ctx=None):
    """quant.DequantizeQ4_0 (lm/quant/quant.go:44)."""
    return (ctx or default_context()).dequantize_host(Q4_0, data, numElements)


def DequantizeQ8_0(data, numElements, ctx=None):
    """quant.DequantizeQ8_0 (lm/quant/quant.go:72)."""
    return (ctx or default_context()).dequantize_host(Q8_0, data, numElements)


def DequantizeQ2_K(data, numElements, ctx=None):
    """quant.DequantizeQ2_K (lm/quant/kquant.go:49)."""
    return (ctx or default_context()).dequantize_host(Q2_K, data, numElements)


def DequantizeIQ2_XXS(data, numElements, ctx=None):
    """quant.DequantizeIQ2_XXS (lm/quant/kquant.go:87)."""
    return (ctx or default_context()).dequantize_host(IQ2_XXS, data, numElements)


def DequantizeQ4_K(data, numElements, ctx=None):
    """GGUF type 12 (gguf/gguf.go:276), arithmetic form of lm/quant/kquant.go:73."""
    return (ctx or default_context()).dequantize_host(Q4_K, data, numElements)


def MatVec(format, data, rows, cols, x, ctx=None):
    """y = x . W^T over GGUF block bytes `data` holding `rows` x `cols` weights.
    x is [cols] or [m][cols] float32 with m <= 8."""
    ctx = ctx or default_context()
    w = ctx.store_upload(_FMT[format] if isinstance(format, str) else format, rows, cols, data)
    try:
        return ctx.matvec_host(w, np.asarray(x, dtype=np.float32))
    finally:
        w.free()
