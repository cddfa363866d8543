"""Seeded synthetic tensors with the shapes and value distributions of the
benchmark configurations. They stand in for model weights: no model file or
dataset is read anywhere.

Distributions (all drawn from numpy's Philox generator keyed by `seed`):
  Q8_0: d = fp16(|N(0,1)|*0.002) per 32 elements, int8 codes uniform [-127,127]
  Q4_0: d = fp16(|N(0,1)|*0.004), 4-bit codes uniform [0,15]
  Q4_K: d, dmin = fp16(|N(0,1)|*0.003) per 256 elements, 6-bit scales and mins
        uniform [0,63], 4-bit codes uniform [0,15]
  Q2_K: d, dmin = fp16(|N(0,1)|*0.01) per 256 elements (bytes 80..83), 4-bit scales and
        mins and 2-bit codes uniform
  IQ2_XXS: d = fp16(|N(0,1)|*0.01) per 256 elements, codebook indices, sign indices and
        4-bit group scales uniform
Bytes are laid out exactly as a GGUF file stores the tensor (row-major blocks).
"""
import numpy as np

Q4_0, Q8_0, Q2_K, Q4_K, IQ2_XXS = 2, 8, 10, 12, 16
BLOCK = {Q4_0: (32, 18), Q8_0: (32, 34), Q4_K: (256, 144), Q2_K: (256, 84), IQ2_XXS: (256, 66)}


def _rng(seed):
    return np.random.Generator(np.random.Philox(key=int(seed)))


def gguf_bytes(fmt, rows, cols):
    be, bb = BLOCK[fmt]
    return rows * (cols // be) * bb


def _random_bytes(g, shape):
    n = int(np.prod(shape))
    raw = g.bit_generator.random_raw((n + 7) // 8)  # uniform 64-bit words -> uniform bytes
    return raw.view(np.uint8)[:n].reshape(shape)


def weights(fmt, rows, cols, seed):
    """GGUF bytes (uint8 array) of a rows x cols tensor of format `fmt`."""
    be, bb = BLOCK[fmt]
    assert cols % be == 0
    nb = rows * (cols // be)
    g = _rng(seed)
    # uniform bytes: uniform nibbles (4-bit codes), uniform 6-bit scale/min fields in any packing
    out = _random_bytes(g, (nb, bb)).copy()
    if fmt == Q8_0:
        # int8 codes uniform in [-127, 127]: redraw the (rare) -128 patterns
        q = out[:, 2:]
        bad = q == 0x80
        q[bad] = g.integers(-127, 128, size=int(bad.sum()), dtype=np.int8).view(np.uint8)
        scale = 0.002
    elif fmt == Q4_0:
        scale = 0.004
    elif fmt == Q4_K:
        scale = 0.003
    else:
        scale = 0.01
    nd = 2 if fmt in (Q4_K, Q2_K) else 1
    at = 80 if fmt == Q2_K else 0   # Q2_K keeps d | dmin at the end of the block
    d = (np.abs(g.standard_normal((nb, nd), dtype=np.float32)) * np.float32(scale)).astype(np.float16)
    out[:, at:at + 2 * nd] = d.view(np.uint8).reshape(nb, 2 * nd)
    return out.reshape(-1)


def activations(m, cols, seed, dtype=np.float32):
    return _rng(seed).standard_normal((m, cols), dtype=np.float32).astype(dtype)
