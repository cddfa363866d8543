"""Second, independently written Q4_K / Q4_0 / Q8_0 decoder in numpy.

Test infrastructure only. The reference pins nothing about GGUF type 12 beyond
its 144-byte / 256-element geometry (gguf/gguf.go:276), so the C oracle's
Q4_K decoder is cross-checked against this vectorised restatement of the same
public field table; the two share no code.
"""
import numpy as np


def _f16(raw_u8_pairs):
    return raw_u8_pairs.copy().view("<f2").astype(np.float32)


def dequantize_q4_k(data, n):
    nb = n // 256
    blk = np.frombuffer(bytes(data), dtype=np.uint8)[: nb * 144].reshape(nb, 144)
    d = _f16(blk[:, 0:2]).reshape(nb)
    dmin = _f16(blk[:, 2:4]).reshape(nb)
    S = blk[:, 4:16].astype(np.uint32)
    sc = np.empty((nb, 8), dtype=np.uint32)
    mn = np.empty((nb, 8), dtype=np.uint32)
    sc[:, 0:4] = S[:, 0:4] & 63
    mn[:, 0:4] = S[:, 4:8] & 63
    sc[:, 4:8] = (S[:, 8:12] & 15) | ((S[:, 0:4] >> 6) << 4)
    mn[:, 4:8] = (S[:, 8:12] >> 4) | ((S[:, 4:8] >> 6) << 4)
    qs = blk[:, 16:144].reshape(nb, 4, 32)
    q = np.empty((nb, 8, 32), dtype=np.float32)
    q[:, 0::2, :] = (qs & 15).astype(np.float32)
    q[:, 1::2, :] = (qs >> 4).astype(np.float32)
    t1 = (d[:, None] * sc.astype(np.float32)).astype(np.float32)
    t3 = (dmin[:, None] * mn.astype(np.float32)).astype(np.float32)
    out = (t1[:, :, None] * q).astype(np.float32) - t3[:, :, None]
    return out.astype(np.float32).reshape(-1)


def dequantize_q4_0(data, n):
    nb = n // 32
    blk = np.frombuffer(bytes(data), dtype=np.uint8)[: nb * 18].reshape(nb, 18)
    d = _f16(blk[:, 0:2]).reshape(nb, 1)
    lo = (blk[:, 2:] & 15).astype(np.int32) - 8
    hi = (blk[:, 2:] >> 4).astype(np.int32) - 8
    return (np.concatenate([lo, hi], axis=1).astype(np.float32) * d).reshape(-1)


def dequantize_q8_0(data, n):
    nb = n // 32
    blk = np.frombuffer(bytes(data), dtype=np.uint8)[: nb * 34].reshape(nb, 34)
    d = _f16(blk[:, 0:2]).reshape(nb, 1)
    return (blk[:, 2:].view(np.int8).astype(np.float32) * d).reshape(-1)
