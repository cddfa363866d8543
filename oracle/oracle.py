"""ctypes front end of oracle/qm_oracle.c (test infrastructure only).

The shared object is built by `make -C oracle` (also run by
`__graft_entry__.build()`). Function names follow the reference's Go API
(lm/quant/quant.go, lm/quant/kquant.go, lm/moe/moe.go) so that tests read like
the reference's own.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libqm_oracle.so")

Q4_0, Q8_0, Q2_K, Q4_K, IQ2_XXS = 2, 8, 10, 12, 16
BLOCK = {Q4_0: (32, 18), Q8_0: (32, 34), Q2_K: (256, 84), Q4_K: (256, 144), IQ2_XXS: (256, 66)}


class OracleError(ValueError):
    pass


def _load():
    if not os.path.exists(_SO) or os.path.getmtime(_SO) < max(
            os.path.getmtime(os.path.join(_HERE, f)) for f in ("qm_oracle.c", "iq2xxs_grid.h")):
        subprocess.check_call(["make", "-C", _HERE, "libqm_oracle.so"],
                              stdout=subprocess.DEVNULL)
    lib = ctypes.CDLL(_SO)
    i64, i32, p = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p
    lib.qo_f16_to_f32_bits.restype = ctypes.c_uint32
    lib.qo_f16_to_f32_bits.argtypes = [ctypes.c_uint16]
    lib.qo_dequantize.argtypes = [i32, p, i64, i64, p]
    lib.qo_tensor_bytes.argtypes = [ctypes.c_uint32, p, i32, p]
    lib.qo_route.argtypes = [p, i32, i32, i32, p, p, p]
    lib.qo_matvec.argtypes = [i32, p, i64, i64, i64, p, i32, i64, p, i64]
    lib.qo_matvec_f32_threaded.argtypes = [i32, p, i64, i64, i64, p, i32, i64, p, i64, i32]
    lib.qo_matvec_faithful.argtypes = [i32, p, i64, i64, i64, p, i32, i64, p, i64]
    lib.qo_rmsnorm.argtypes = [p, i64, ctypes.c_float, p]
    lib.qo_rmsnorm.restype = None
    lib.qo_f32_to_f16.argtypes = [ctypes.c_float]
    lib.qo_f32_to_f16.restype = ctypes.c_uint16
    lib.qo_rmsnorm_q8_1.argtypes = [p, i64, p, i64, i64, i64, ctypes.c_float, i32, p]
    lib.qo_swiglu_q8_1.argtypes = [p, p, p, i32, i32, p]
    lib.qo_swiglu_q8_1.restype = None
    lib.qo_q8_1_dequantize.argtypes = [p, i64, p]
    lib.qo_q8_1_dequantize.restype = None
    return lib


_lib = _load()

_MSG = {-1: "quant: element count is not a non-negative multiple of the block",
        -2: "quant: buffer length insufficient", -3: "quant: unknown format",
        -4: "gguf: unsupported tensor type", -5: "gguf: tensor row is not block aligned",
        -6: "gguf: tensor byte count overflow",
        -10: "cudaquant: invalid RMSNorm dimensions or epsilon", -11: "cudaquant: input length mismatch",
        -12: "cudaquant: weight length mismatch", -13: "cudaquant: nonfinite input",
        -14: "cudaquant: nonfinite weight", -15: "cudaquant: zero normalization denominator",
        -16: "cudaquant: normalized value is nonfinite"}


def _raise(rc):
    if rc:
        raise OracleError(_MSG.get(rc, "oracle error %d" % rc))


def _u8(data):
    a = np.frombuffer(bytes(data), dtype=np.uint8) if not isinstance(data, np.ndarray) else data
    return np.ascontiguousarray(a, dtype=np.uint8)


def Float16ToFloat32Bits(h):
    """lm/quant/quant.go:94 — returns the float32 bit pattern."""
    return int(_lib.qo_f16_to_f32_bits(int(h) & 0xFFFF))


def Float16ToFloat32(h):
    return np.array([Float16ToFloat32Bits(h)], dtype=np.uint32).view(np.float32)[0]


def Dequantize(fmt, data, num_elements):
    a = _u8(data)
    out = np.empty(max(int(num_elements), 0), dtype=np.float32)
    _raise(_lib.qo_dequantize(fmt, a.ctypes.data, a.size, int(num_elements), out.ctypes.data))
    return out


def DequantizeQ4_0(data, n):
    return Dequantize(Q4_0, data, n)


def DequantizeQ8_0(data, n):
    return Dequantize(Q8_0, data, n)


def DequantizeQ2_K(data, n):
    return Dequantize(Q2_K, data, n)


def DequantizeQ4_K(data, n):
    return Dequantize(Q4_K, data, n)


def DequantizeIQ2_XXS(data, n):
    """lm/quant/kquant.go:87."""
    return Dequantize(IQ2_XXS, data, n)


def TensorBytes(type_id, dims):
    """gguf/gguf.go:285 Tensor.Bytes."""
    d = np.asarray(dims, dtype=np.uint64)
    out = ctypes.c_uint64(0)
    _raise(_lib.qo_tensor_bytes(int(type_id), d.ctypes.data, d.size, ctypes.byref(out)))
    return out.value


def Route(logits, num_experts, topk, biases=None):
    """lm/moe/moe.go:73 GroupedTopKRouter.Route for one token -> (ids, weights)."""
    lg = np.ascontiguousarray(logits, dtype=np.float32)
    b = None if biases is None else np.ascontiguousarray(biases, dtype=np.float32)
    cap = max(min(int(topk), lg.size, int(num_experts)), 0)
    ids = np.zeros(max(cap, 1), dtype=np.int32)
    w = np.zeros(max(cap, 1), dtype=np.float32)
    k = _lib.qo_route(lg.ctypes.data, lg.size, int(num_experts), int(topk),
                      None if b is None else b.ctypes.data, ids.ctypes.data, w.ctypes.data)
    return ids[:k].copy(), w[:k].copy()


def MatVec(fmt, data, rows, cols, x, threads=0):
    """y[m][r] = sum_c x[m][c]*W[r][c]; float64 accumulation when threads == 0,
    float32 arithmetic split over `threads` threads otherwise (timed baseline)."""
    a = _u8(data)
    x = np.ascontiguousarray(x, dtype=np.float32)
    x2 = x.reshape(1, -1) if x.ndim == 1 else x
    m = x2.shape[0]
    y = np.empty((m, rows), dtype=np.float32)
    if threads:
        rc = _lib.qo_matvec_f32_threaded(fmt, a.ctypes.data, a.size, rows, cols, x2.ctypes.data,
                                         m, x2.shape[1], y.ctypes.data, rows, int(threads))
    else:
        rc = _lib.qo_matvec(fmt, a.ctypes.data, a.size, rows, cols, x2.ctypes.data, m,
                            x2.shape[1], y.ctypes.data, rows)
    _raise(rc)
    return y[0] if x.ndim == 1 else y


def MatVecFaithful(fmt, data, rows, cols, x):
    """Timed single-thread baseline: dequantize the whole matrix to float32, then dot in float32."""
    a = _u8(data)
    x = np.ascontiguousarray(x, dtype=np.float32)
    x2 = x.reshape(1, -1) if x.ndim == 1 else x
    y = np.empty((x2.shape[0], rows), dtype=np.float32)
    _raise(_lib.qo_matvec_faithful(fmt, a.ctypes.data, a.size, rows, cols, x2.ctypes.data, x2.shape[0],
                                   x2.shape[1], y.ctypes.data, rows))
    return y[0] if x.ndim == 1 else y


def RMSNorm(x, eps=1e-6):
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty_like(x)
    if x.ndim == 1:
        _lib.qo_rmsnorm(x.ctypes.data, x.size, eps, out.ctypes.data)
    else:
        for i in range(x.shape[0]):
            _lib.qo_rmsnorm(x[i].ctypes.data, x.shape[1], eps, out[i].ctypes.data)
    return out


def Float32ToFloat16(f):
    """nvidia/x/cudaquant/quant.go:325 float32ToFloat16 (bits)."""
    return int(_lib.qo_f32_to_f16(float(np.float32(f))))


def RMSNormQ8_1(input, weight, rows, cols, epsilon, weighted):
    """nvidia/x/cudaquant/quant.go:46 RMSNormQ8_1 -> bytes of rows*cols/32 blocks (d, s, 32 quants)."""
    x = np.ascontiguousarray(input, dtype=np.float32).reshape(-1)
    w = np.zeros(0, dtype=np.float32) if weight is None else np.ascontiguousarray(weight, dtype=np.float32).reshape(-1)
    # the output is sized by the input actually given: the length checks run before anything is written
    nblk = x.size // 32 if rows > 0 and cols > 0 and int(rows) * int(cols) == x.size else 0
    out = np.zeros(max(nblk, 1) * 36, dtype=np.uint8)
    _raise(_lib.qo_rmsnorm_q8_1(x.ctypes.data, x.size, w.ctypes.data if w.size else None, w.size, int(rows), int(cols),
                                float(epsilon), 1 if weighted else 0, out.ctypes.data))
    return out[:nblk * 36].tobytes()


def SwiGLUQ8_1(gate, up, weights, width, slots):
    """fused_swiglu_q8_1 (nvidia/x/egraph/codegen.go:513-552) -> bytes of ceil(width*slots/32) blocks."""
    g = np.ascontiguousarray(gate, dtype=np.float32).reshape(-1)
    u = np.ascontiguousarray(up, dtype=np.float32).reshape(-1)
    w = np.ascontiguousarray(weights, dtype=np.float32).reshape(-1)
    assert g.size == u.size == width * slots and w.size == slots
    nblk = (width * slots + 31) // 32
    out = np.zeros(max(nblk, 1) * 36, dtype=np.uint8)
    _lib.qo_swiglu_q8_1(g.ctypes.data, u.ctypes.data, w.ctypes.data, int(width), int(slots), out.ctypes.data)
    return out[:nblk * 36].tobytes()


def DequantizeQ8_1(blocks, n):
    """q8_1_at (nvidia/x/egraph/codegen.go:125-128) for elements 0..n-1."""
    b = _u8(blocks)
    assert b.size >= (n + 31) // 32 * 36
    out = np.empty(n, dtype=np.float32)
    _lib.qo_q8_1_dequantize(b.ctypes.data, int(n), out.ctypes.data)
    return out


def SelectedMatVecQ8_1(fmt, data, experts, rows, cols, ids, xq):
    """The *_selected_matvec_q8_1 kernels (nvidia/x/egraph/codegen.go:554-616): weights laid out
    [expert][row][block], one Q8_1 vector x for all slots, y[slot][row]; a negative id gives NaN."""
    a = _u8(data)
    row_bytes = a.size // (experts * rows)
    x = DequantizeQ8_1(xq, cols)
    y = np.empty((len(ids), rows), dtype=np.float32)
    for s, e in enumerate(ids):
        if e < 0:
            y[s] = np.nan
        else:
            y[s] = MatVec(fmt, a[e * rows * row_bytes:(e + 1) * rows * row_bytes], rows, cols, x)
    return y
