"""ctypes binding of include/qmatmul.h. Every call goes through the C ABI."""
import ctypes
import os
import re

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.environ.get("QMATMUL_LIB", os.path.join(_HERE, "libqmatmul.so"))
_HEADER = os.path.join(_HERE, "..", "include", "qmatmul.h")

Q4_0, Q8_0, Q2_K, Q4_K, IQ2_XXS = 2, 8, 10, 12, 16
XOP_NONE, XOP_RMSNORM, XOP_ADD_RMSNORM, XOP_SWIGLU = 0, 1, 2, 3
FLAG_PDL = 0x100
FLAG_X_Q8_1 = 0x200


class QmError(RuntimeError):
    def __init__(self, code, what=""):
        self.code = code
        msg = lib.qm_error_string(code).decode() if lib is not None else "status %d" % code
        super().__init__("%s%s (status %d)" % (what + ": " if what else "", msg, code))


def _load():
    if not os.path.exists(_LIB_PATH):
        raise ImportError(
            "libqmatmul.so is not built (%s); run `python lib_b200/build.py`. There is no "
            "fallback implementation." % _LIB_PATH)
    L = ctypes.CDLL(_LIB_PATH)
    i32, i64, u32, u64, p = ctypes.c_int32, ctypes.c_int64, ctypes.c_uint32, ctypes.c_uint64, ctypes.c_void_p
    sig = {
        "qm_version": (i32, []),
        "qm_error_string": (ctypes.c_char_p, [i32]),
        "qm_init": (i32, [i32, ctypes.POINTER(p)]),
        "qm_destroy": (i32, [p]),
        "qm_set_stream": (i32, [p, u64]),
        "qm_sync": (i32, [p]),
        "qm_last_status": (i32, [p, ctypes.POINTER(u32)]),
        "qm_launch_count": (i64, [p]),
        "qm_malloc": (i32, [p, i64, ctypes.POINTER(u64)]),
        "qm_free": (i32, [p, u64]),
        "qm_memcpy_h2d": (i32, [p, u64, p, i64]),
        "qm_memcpy_d2h": (i32, [p, p, u64, i64]),
        "qm_store_upload": (i32, [p, i32, i64, i64, p, i64, i64, i64, ctypes.POINTER(u64)]),
        "qm_store_create": (i32, [p, i32, i64, i64, ctypes.POINTER(u64)]),
        "qm_store_write_rows": (i32, [p, u64, i64, i64, p, i64]),
        "qm_store_write_rows_device": (i32, [p, u64, i64, i64, u64, i64]),
        "qm_store_free": (i32, [p, u64]),
        "qm_store_info": (i32, [p, u64, ctypes.POINTER(i64)]),
        "qm_dequantize": (i32, [p, u64, u64]),
        "qm_dequantize_host": (i32, [p, i32, p, i64, i64, p]),
        "qm_matvec": (i32, [p, u64, u64, u64, i32, i64, u64, i64, u32]),
        "qm_matvec_host": (i32, [p, u64, p, i32, i64, p, i64, u32]),
        "qm_matmul_bf16": (i32, [p, u64, u64, i32, i64, u64, i64]),
        "qm_moe_route": (i32, [p, u64, i32, i64, i32, i32, u64, u64, u64]),
        "qm_moe_grouped": (i32, [p, p, p, i32, u64, i32, i64, u64, u64, i32, u64, i64]),
        "qm_moe_dispatch": (i32, [p, u64, i32, i32, i32, u64, i64, i32, u64, u64, p]),
        "qm_moe_experts": (i32, [p, p, p, i32, u64, p, u64]),
        "qm_moe_combine": (i32, [p, u64, u64, u64, i32, i32, i32, u64, i64]),
        "qm_matvec_noalloc": (i32, [u64, u64, i32, i64, u64, i64, u64]),
        "qm_expert_pool_create": (i32, [p, p, i32, i64, i64, i32, ctypes.POINTER(p)]),
        "qm_expert_pool_get": (i32, [p, p, i64, ctypes.POINTER(u64)]),
        "qm_expert_pool_info": (i32, [p, ctypes.POINTER(i64)]),
        "qm_expert_pool_evict": (i32, [p, i64]),
        "qm_expert_pool_close": (i32, [p, p]),
        "qm_ep_create": (i32, [p, p, p, i32, i32, i32, i32, i32, i32, ctypes.POINTER(p)]),
        "qm_ep_arena": (i32, [p, p, ctypes.POINTER(u64), ctypes.POINTER(i64)]),
        "qm_ep_ipc_handle": (i32, [p, p, p]),
        "qm_ep_set_peers": (i32, [p, p, p]),
        "qm_ep_set_peer_pointers": (i32, [p, p, ctypes.POINTER(u64)]),
        "qm_ep_moe": (i32, [p, p, u64, i32, i64, u64, u64, u64, i64]),
        "qm_ep_begin": (i32, [p, p, u64, i32, i64, u64, u64, u64, i64]),
        "qm_ep_run": (i32, [p, p]),
        "qm_ep_end": (i32, [p, p]),
        "qm_ep_destroy": (i32, [p, p]),
        "qm_moe_decode_create": (i32, [p, p, p, i32, i32, i32, ctypes.POINTER(p)]),
        "qm_moe_decode_run": (i32, [p, p, u64, i32, i64, u64, u64, u64, i64]),
        "qm_moe_decode_destroy": (i32, [p, p]),
        "qm_rmsnorm_q8_1": (i32, [p, u64, i64, u64, i64, i64, ctypes.c_float, u64]),
        "qm_rmsnorm_q8_1_host": (i32, [p, p, i64, p, i64, i64, i64, ctypes.c_float, i32, p]),
        "qm_swiglu_q8_1": (i32, [p, u64, u64, u64, i32, i32, u64]),
        "qm_q8_1_dequantize": (i32, [p, u64, i32, i64, i64, u64, i64]),
        "qm_matvec_q8_1": (i32, [p, u64, u64, i32, i64, u64, i64, u32]),
        "qm_matvec_selected": (i32, [p, u64, i32, u64, i32, u64, i64, u64, u32]),
        "qm_noalloc_status": (i32, [ctypes.POINTER(u32)]),
        "qm_stack_create": (i32, [p, i32, i32, i32, i32, i32, ctypes.POINTER(p)]),
        "qm_stack_destroy": (i32, [p, p]),
        "qm_stack_set_layer": (i32, [p, p, i32, u64, u64, u64, u64]),
        "qm_stack_step": (i32, [p, p, u64, i32, i64, u64, i64]),
        "qm_stack_step_host": (i32, [p, p, p, i32, p, p]),
        "qm_stack_buffers": (i32, [p, p, ctypes.POINTER(u64)]),
        "qm_stack_parts": (i32, [p, p, ctypes.POINTER(i64)]),
        "qm_stack_use_graph": (i32, [p, p, i32]),
        "qm_stack_create_tp": (i32, [p, i32, i32, i32, i32, i32, i32, i32, ctypes.POINTER(p)]),
        "qm_stack_create_tp_paired": (i32, [p, i32, i32, i32, i32, i32, i32, i32, ctypes.POINTER(p)]),
        "qm_stack_ipc_handle": (i32, [p, p, p]),
        "qm_stack_set_peers": (i32, [p, p, p]),
        "qm_stack_arena": (i32, [p, p, ctypes.POINTER(u64), ctypes.POINTER(i64)]),
        "qm_stack_set_peer_pointers": (i32, [p, p, ctypes.POINTER(u64)]),
        "qm_gguf_open": (i32, [ctypes.c_char_p, ctypes.POINTER(p)]),
        "qm_gguf_close": (i32, [p]),
        "qm_gguf_tensor_count": (i32, [p]),
        "qm_gguf_tensor_info": (i32, [p, i32, ctypes.c_char_p, i32, ctypes.POINTER(i64), ctypes.POINTER(i64)]),
        "qm_gguf_find": (i32, [p, ctypes.c_char_p]),
        "qm_gguf_load_tensor": (i32, [p, p, i32, i64, i64, ctypes.POINTER(u64)]),
        "qm_gguf_load_rows": (i32, [p, p, i32, i64, i64, u64, i64]),
        "qm_expert_cache_create": (i32, [ctypes.c_char_p, i32, ctypes.POINTER(p)]),
        "qm_expert_cache_register": (i32, [p, i64, p, i64]),
        "qm_expert_cache_get": (i32, [p, i64, p, i64, ctypes.POINTER(i64)]),
        "qm_expert_cache_hot": (i32, [p]),
        "qm_expert_cache_evict": (i32, [p, i64]),
        "qm_expert_cache_close": (i32, [p]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype, fn.argtypes = res, args
    return L


lib = _load()


def declared_symbols():
    """Names of every entry point include/qmatmul.h declares."""
    return re.findall(r"QM_API\s+[\w \*]+?\b(qm_\w+)\(", open(_HEADER).read())


def _check(rc, what=""):
    if rc != 0:
        raise QmError(rc, what)


def _u8(data):
    if isinstance(data, np.ndarray):
        return np.ascontiguousarray(data.view(np.uint8).reshape(-1))
    return np.frombuffer(bytes(data), dtype=np.uint8)


class GgufFile:
    """qm_gguf: the tensor directory of a GGUF file, and its tensors streamed into the store."""

    def __init__(self, path):
        h = ctypes.c_void_p()
        _check(lib.qm_gguf_open(os.fsencode(path), ctypes.byref(h)), "gguf_open")
        self._h = h

    def tensor_count(self):
        return int(lib.qm_gguf_tensor_count(self._h))

    def tensor_info(self, index):
        """(name, type id, dimensions, file offset of the bytes, byte count)."""
        name = ctypes.create_string_buffer(80)
        info, offs = (ctypes.c_int64 * 6)(), (ctypes.c_int64 * 2)()
        _check(lib.qm_gguf_tensor_info(self._h, index, name, 80, info, offs), "gguf_tensor_info")
        return name.value.decode(), int(info[0]), [int(v) for v in info[2:2 + info[1]]], int(offs[0]), int(offs[1])

    def find(self, name):
        rc = lib.qm_gguf_find(self._h, name.encode())
        if rc < 0:
            raise QmError(rc, "gguf_find")
        return rc

    def load_tensor(self, ctx, index, row_lo=0, row_hi=0):
        h = ctypes.c_uint64(0)
        _check(lib.qm_gguf_load_tensor(ctx._h, self._h, index, row_lo, row_hi, ctypes.byref(h)), "gguf_load_tensor")
        return Weight(ctx, h.value)

    def load_rows(self, ctx, index, row_lo, row_hi, weight, dst_row):
        _check(lib.qm_gguf_load_rows(ctx._h, self._h, index, row_lo, row_hi, weight.handle, dst_row), "gguf_load_rows")

    def close(self):
        if self._h:
            lib.qm_gguf_close(self._h)
            self._h = None


class Weight:
    """A device-resident weight matrix of the store (qm_weight)."""

    def __init__(self, ctx, handle):
        self.ctx, self.handle = ctx, handle
        info = (ctypes.c_int64 * 5)()
        _check(lib.qm_store_info(ctx._h, handle, info))
        self.fmt, self.rows, self.cols, self.device_bytes, self.gguf_bytes = [int(v) for v in info]

    def write_rows(self, row_offset, nrows, data):
        a = _u8(data)
        _check(lib.qm_store_write_rows(self.ctx._h, self.handle, row_offset, nrows, a.ctypes.data, a.size),
               "store_write_rows")

    def write_rows_device(self, row_offset, nrows, dev_ptr, nbytes):
        _check(lib.qm_store_write_rows_device(self.ctx._h, self.handle, row_offset, nrows, dev_ptr, nbytes),
               "store_write_rows_device")

    def free(self):
        if self.handle:
            _check(lib.qm_store_free(self.ctx._h, self.handle))
            self.handle = 0


class Context:
    """qm_ctx: one device, its kernels and a stream. Raises if the CUDA driver
    or the sm_100a kernel images cannot be loaded — there is no other path."""

    def __init__(self, device=0):
        h = ctypes.c_void_p()
        _check(lib.qm_init(device, ctypes.byref(h)), "qm_init")
        self._h = h
        self.device = device

    def close(self):
        if self._h:
            lib.qm_destroy(self._h)
            self._h = None

    def set_stream(self, cu_stream):
        _check(lib.qm_set_stream(self._h, int(cu_stream)))

    def sync(self):
        _check(lib.qm_sync(self._h), "qm_sync")

    def last_status(self):
        s = ctypes.c_uint32(0)
        rc = lib.qm_last_status(self._h, ctypes.byref(s))
        return rc, s.value

    def launch_count(self):
        return int(lib.qm_launch_count(self._h))

    # -- memory -------------------------------------------------------------
    def malloc(self, nbytes):
        d = ctypes.c_uint64(0)
        _check(lib.qm_malloc(self._h, nbytes, ctypes.byref(d)), "qm_malloc")
        return d.value

    def free(self, dptr):
        _check(lib.qm_free(self._h, dptr))

    def h2d(self, dptr, arr):
        a = np.ascontiguousarray(arr)
        _check(lib.qm_memcpy_h2d(self._h, dptr, a.ctypes.data, a.nbytes), "h2d")

    def d2h(self, arr, dptr):
        assert arr.flags["C_CONTIGUOUS"]
        _check(lib.qm_memcpy_d2h(self._h, arr.ctypes.data, dptr, arr.nbytes), "d2h")

    # -- store --------------------------------------------------------------
    def store_upload(self, fmt, rows, cols, data, row_lo=0, row_hi=None):
        a = _u8(data)
        h = ctypes.c_uint64(0)
        _check(lib.qm_store_upload(self._h, fmt, rows, cols, a.ctypes.data, a.size, row_lo,
                                   rows if row_hi is None else row_hi, ctypes.byref(h)), "store_upload")
        return Weight(self, h.value)

    def store_create(self, fmt, rows, cols):
        h = ctypes.c_uint64(0)
        _check(lib.qm_store_create(self._h, fmt, rows, cols, ctypes.byref(h)), "store_create")
        return Weight(self, h.value)

    # -- operations -----------------------------------------------------------
    def dequantize(self, w, out_dev):
        _check(lib.qm_dequantize(self._h, w.handle, out_dev), "dequantize")

    def dequantize_host(self, fmt, data, num_elements):
        a = _u8(data)
        out = np.empty(max(int(num_elements), 0), dtype=np.float32)
        _check(lib.qm_dequantize_host(self._h, fmt, a.ctypes.data, a.size, int(num_elements),
                                      out.ctypes.data), "dequantize")
        return out

    def matvec(self, w, x_dev, m, ldx, y_dev, ldy, flags=0, x2_dev=0):
        _check(lib.qm_matvec(self._h, w.handle, x_dev, x2_dev, m, ldx, y_dev, ldy, flags), "matvec")

    def matmul_bf16(self, w, a_dev, m, lda, c_dev, ldc):
        """qm_matmul_bf16: c[m][rows] = a[m][cols] (bf16) x W^T on tcgen05, fp32 out."""
        _check(lib.qm_matmul_bf16(self._h, w.handle, a_dev, m, lda, c_dev, ldc), "matmul_bf16")

    def moe_route(self, logits_dev, tokens, ld, experts, topk, ids_dev, weights_dev, bias_dev=0):
        _check(lib.qm_moe_route(self._h, logits_dev, tokens, ld, experts, topk, bias_dev, ids_dev, weights_dev),
               "moe_route")

    def moe_grouped(self, gate_up, down, x_dev, tokens, ldx, ids_dev, weights_dev, topk, out_dev, ldo):
        n = len(gate_up)
        ga = (ctypes.c_uint64 * n)(*[w.handle for w in gate_up])
        da = (ctypes.c_uint64 * n)(*[w.handle for w in down])
        _check(lib.qm_moe_grouped(self._h, ga, da, n, x_dev, tokens, ldx, ids_dev, weights_dev, topk, out_dev, ldo),
               "moe_grouped")

    def moe_dispatch(self, ids_dev, tokens, topk, experts, x_dev, ldx, hidden, rows_dev, pos_dev):
        """qm_moe_dispatch: rows grouped by expert + pos; returns the per-expert counts (list)."""
        counts = (ctypes.c_int32 * experts)()
        _check(lib.qm_moe_dispatch(self._h, ids_dev, tokens, topk, experts, x_dev, ldx, hidden, rows_dev, pos_dev,
                                   counts), "moe_dispatch")
        return list(counts)

    def moe_experts(self, gate_up, down, rows_dev, counts, y_dev):
        n = len(gate_up)
        ga = (ctypes.c_uint64 * n)(*[w.handle for w in gate_up])
        da = (ctypes.c_uint64 * n)(*[w.handle for w in down])
        ca = (ctypes.c_int32 * n)(*[int(v) for v in counts])
        _check(lib.qm_moe_experts(self._h, ga, da, n, rows_dev, ca, y_dev), "moe_experts")

    def moe_combine(self, y_dev, pos_dev, weights_dev, tokens, topk, hidden, out_dev, ldo):
        _check(lib.qm_moe_combine(self._h, y_dev, pos_dev, weights_dev, tokens, topk, hidden, out_dev, ldo),
               "moe_combine")

    def moe_decode_create(self, gate_up, down, topk, max_tokens):
        """qm_moe_decode_create -> opaque handle for moe_decode_run / moe_decode_destroy."""
        n = len(gate_up)
        ga = (ctypes.c_uint64 * n)(*[w.handle for w in gate_up])
        da = (ctypes.c_uint64 * n)(*[w.handle for w in down])
        h = ctypes.c_void_p()
        _check(lib.qm_moe_decode_create(self._h, ga, da, n, topk, max_tokens, ctypes.byref(h)), "moe_decode_create")
        return h

    def moe_decode_run(self, md, x_dev, tokens, ldx, ids_dev, weights_dev, out_dev, ldo):
        _check(lib.qm_moe_decode_run(self._h, md, x_dev, tokens, ldx, ids_dev, weights_dev, out_dev, ldo), "moe_decode_run")

    def moe_decode_destroy(self, md):
        _check(lib.qm_moe_decode_destroy(self._h, md), "moe_decode_destroy")

    def matvec_noalloc(self, w, x_dev, m, ldx, y_dev, ldy, cu_stream=0):
        """qm_matvec_noalloc: Q4_0/Q8_0 matvec that allocates nothing (fixed scratch array)."""
        _check(lib.qm_matvec_noalloc(w.handle, x_dev, m, ldx, y_dev, ldy, cu_stream), "matvec_noalloc")

    def noalloc_status(self):
        """qm_noalloc_status: (return code, status word) of the last qm_matvec_noalloc on this device."""
        s = ctypes.c_uint32(0)
        rc = lib.qm_noalloc_status(ctypes.byref(s))
        return rc, s.value

    # ---- Q8_1 activation ABI -----------------------------------------------------------------
    def rmsnorm_q8_1(self, x_dev, ldx, weight_dev, rows, cols, eps, out_dev):
        _check(lib.qm_rmsnorm_q8_1(self._h, x_dev, ldx, weight_dev, rows, cols, eps, out_dev), "rmsnorm_q8_1")

    def RMSNormQ8_1(self, input, weight, rows, cols, epsilon, weighted):
        """cudaquant.RMSNormQ8_1 (nvidia/x/cudaquant/quant.go:46) on the GPU over host arrays -> block bytes;
        raises QmError where the reference returns an error."""
        x = np.ascontiguousarray(input, dtype=np.float32).reshape(-1)
        w = None if weight is None else np.ascontiguousarray(weight, dtype=np.float32).reshape(-1)
        ok = rows > 0 and cols > 0 and int(rows) * int(cols) == x.size
        out = np.zeros((x.size // 32 if ok else 0) * 36 + 4, dtype=np.uint8)
        _check(lib.qm_rmsnorm_q8_1_host(self._h, x.ctypes.data, x.size, None if w is None else w.ctypes.data,
                                        0 if w is None else w.size, int(rows), int(cols), float(epsilon),
                                        1 if weighted else 0, out.ctypes.data), "RMSNormQ8_1")
        return out[:-4].tobytes()

    def swiglu_q8_1(self, gate_dev, up_dev, weights_dev, width, slots, out_dev):
        _check(lib.qm_swiglu_q8_1(self._h, gate_dev, up_dev, weights_dev, width, slots, out_dev), "swiglu_q8_1")

    def q8_1_dequantize(self, xq_dev, m, ldx_blocks, cols, out_dev, ld_out):
        _check(lib.qm_q8_1_dequantize(self._h, xq_dev, m, ldx_blocks, cols, out_dev, ld_out), "q8_1_dequantize")

    def matvec_q8_1(self, w, xq_dev, m, ldx_blocks, y_dev, ldy, flags=0):
        _check(lib.qm_matvec_q8_1(self._h, w.handle, xq_dev, m, ldx_blocks, y_dev, ldy, flags), "matvec_q8_1")

    def matvec_selected(self, w, experts, ids_dev, slots, x_dev, x_slot_stride, y_dev, flags=0):
        _check(lib.qm_matvec_selected(self._h, w.handle, experts, ids_dev, slots, x_dev, x_slot_stride, y_dev, flags),
               "matvec_selected")

    def matvec_host(self, w, x, flags=0, out=None):
        x = np.ascontiguousarray(x, dtype=np.float32)
        x2 = x.reshape(1, -1) if x.ndim == 1 else x
        m = x2.shape[0]
        y = out if out is not None else np.empty((m, w.rows), dtype=np.float32)
        _check(lib.qm_matvec_host(self._h, w.handle, x2.ctypes.data, m, x2.shape[1], y.ctypes.data,
                                  y.shape[-1], flags), "matvec")
        return y[0] if (x.ndim == 1 and out is None) else y


class ExpertParallel:
    """qm_ep: one rank's share of an expert-parallel MoE layer, the exchange over peer memory."""

    def __init__(self, ctx, gate_up, down, experts_total, topk, max_tokens, rank=0, world=1):
        self.ctx, self.rank, self.world = ctx, rank, world
        n = len(gate_up)
        ga = (ctypes.c_uint64 * n)(*[w.handle for w in gate_up])
        da = (ctypes.c_uint64 * n)(*[w.handle for w in down])
        h = ctypes.c_void_p()
        _check(lib.qm_ep_create(ctx._h, ga, da, n, experts_total, topk, max_tokens, rank, world, ctypes.byref(h)), "ep_create")
        self._h = h

    def arena(self):
        base, nbytes = ctypes.c_uint64(0), ctypes.c_int64(0)
        _check(lib.qm_ep_arena(self.ctx._h, self._h, ctypes.byref(base), ctypes.byref(nbytes)), "ep_arena")
        return base.value, nbytes.value

    def ipc_handle(self):
        buf = ctypes.create_string_buffer(64)
        _check(lib.qm_ep_ipc_handle(self.ctx._h, self._h, buf), "ep_ipc_handle")
        return buf.raw

    def set_peers(self, handles):
        blob = b"".join(handles)
        _check(lib.qm_ep_set_peers(self.ctx._h, self._h, blob), "ep_set_peers")

    def set_peer_pointers(self, bases):
        arr = (ctypes.c_uint64 * len(bases))(*bases)
        _check(lib.qm_ep_set_peer_pointers(self.ctx._h, self._h, arr), "ep_set_peer_pointers")

    def moe(self, x_dev, tokens, ldx, ids_dev, weights_dev, out_dev, ldo):
        _check(lib.qm_ep_moe(self.ctx._h, self._h, x_dev, tokens, ldx, ids_dev, weights_dev, out_dev, ldo), "ep_moe")

    def begin(self, x_dev, tokens, ldx, ids_dev, weights_dev, out_dev, ldo):
        _check(lib.qm_ep_begin(self.ctx._h, self._h, x_dev, tokens, ldx, ids_dev, weights_dev, out_dev, ldo), "ep_begin")

    def run(self):
        _check(lib.qm_ep_run(self.ctx._h, self._h), "ep_run")

    def end(self):
        _check(lib.qm_ep_end(self.ctx._h, self._h), "ep_end")

    def close(self):
        if self._h:
            lib.qm_ep_destroy(self.ctx._h, self._h)
            self._h = None


class Stack:
    """qm_stack: a decode step over `layers` quantized transformer-shaped layers."""

    def __init__(self, ctx, layers, hidden, kv_dim, ffn, m_max=8, rank=0, world=1, paired=False):
        self.ctx, self.layers, self.hidden, self.kv_dim, self.ffn, self.m_max = ctx, layers, hidden, kv_dim, ffn, m_max
        self.rank, self.world, self.paired = rank, world, paired
        h = ctypes.c_void_p()
        if world == 1:
            _check(lib.qm_stack_create(ctx._h, layers, hidden, kv_dim, ffn, m_max, ctypes.byref(h)), "stack_create")
        elif paired:
            _check(lib.qm_stack_create_tp_paired(ctx._h, layers, hidden, kv_dim, ffn, m_max, rank, world, ctypes.byref(h)),
                   "stack_create_tp_paired")
        else:
            _check(lib.qm_stack_create_tp(ctx._h, layers, hidden, kv_dim, ffn, m_max, rank, world, ctypes.byref(h)),
                   "stack_create_tp")
        self._h = h
        self.weights = []

    def ipc_handle(self):
        """64-byte CUDA IPC handle of the tensor-parallel activation arena."""
        buf = (ctypes.c_ubyte * 64)()
        _check(lib.qm_stack_ipc_handle(self.ctx._h, self._h, buf), "stack_ipc_handle")
        return bytes(buf)

    def set_peers(self, handles):
        """handles: the `world` 64-byte handles in rank order."""
        blob = b"".join(handles)
        assert len(blob) == 64 * self.world
        buf = (ctypes.c_ubyte * len(blob)).from_buffer_copy(blob)
        _check(lib.qm_stack_set_peers(self.ctx._h, self._h, buf), "stack_set_peers")

    def arena(self):
        """(base device address, bytes) of the tensor-parallel activation arena."""
        base, nbytes = ctypes.c_uint64(0), ctypes.c_int64(0)
        _check(lib.qm_stack_arena(self.ctx._h, self._h, ctypes.byref(base), ctypes.byref(nbytes)), "stack_arena")
        return base.value, nbytes.value

    def set_peer_pointers(self, bases):
        """bases: the `world` arena base addresses as this process addresses them."""
        arr = (ctypes.c_uint64 * self.world)(*[int(b) for b in bases])
        _check(lib.qm_stack_set_peer_pointers(self.ctx._h, self._h, arr), "stack_set_peer_pointers")

    def set_layer(self, layer, qkv, o, gate_up, down):
        _check(lib.qm_stack_set_layer(self.ctx._h, self._h, layer, qkv.handle, o.handle, gate_up.handle,
                                      down.handle), "stack_set_layer")
        self.weights.append((qkv, o, gate_up, down))

    def use_graph(self, on):
        _check(lib.qm_stack_use_graph(self.ctx._h, self._h, int(on)))

    def step(self, x_dev, m, ldx, h_out_dev=0, ldh=0):
        _check(lib.qm_stack_step(self.ctx._h, self._h, x_dev, m, ldx, h_out_dev, ldh), "stack_step")

    def step_host(self, x, want_kv=False, h_out=None, kv_out=None):
        x = np.ascontiguousarray(x, dtype=np.float32)
        m = x.shape[0]
        h = h_out if h_out is not None else np.empty((m, self.hidden), dtype=np.float32)
        kv = kv_out
        if want_kv and kv is None:
            kv = np.empty((self.layers, m, 2 * self.kv_dim), dtype=np.float32)
        _check(lib.qm_stack_step_host(self.ctx._h, self._h, x.ctypes.data, m, h.ctypes.data,
                                      kv.ctypes.data if kv is not None else None), "stack_step_host")
        return (h, kv) if want_kv else h

    def buffers(self):
        ptrs = (ctypes.c_uint64 * 5)()
        _check(lib.qm_stack_buffers(self.ctx._h, self._h, ptrs))
        return [int(v) for v in ptrs]

    def parts(self):
        """(K parts of the o projection in the most recent step, floats between its partial vectors)."""
        info = (ctypes.c_int64 * 2)()
        _check(lib.qm_stack_parts(self.ctx._h, self._h, info))
        return int(info[0]), int(info[1])

    def close(self):
        if self._h:
            lib.qm_stack_destroy(self.ctx._h, self._h)
            self._h = None
