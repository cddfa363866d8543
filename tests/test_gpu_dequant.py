"""GPU parity: device dequantization through the C ABI, bit for bit against the
oracle and the reference's vectors (lm/quant/quant_test.go, kquant_test.go)."""
import numpy as np
import pytest

import lib_b200
from lib_b200 import quant as gq
from oracle import oracle

pytestmark = pytest.mark.gpu

FMTS = {2: (32, 18), 8: (32, 34), 10: (256, 84), 12: (256, 144), 16: (256, 66)}


def _same_bits(a, b):
    return bool(((a.view(np.uint32) == b.view(np.uint32)) | (np.isnan(a) & np.isnan(b))).all())


def test_known_answers(ctx, ds4_golden):
    d = bytearray(18)
    d[0:2] = (0x3C00).to_bytes(2, "little")
    d[2] = 0x98
    out = gq.DequantizeQ4_0(d, 32, ctx)
    assert out[0] == 0.0 and out[16] == 1.0
    d = bytearray(34)
    d[0:2] = (0x3C00).to_bytes(2, "little")
    d[2] = 42
    assert gq.DequantizeQ8_0(d, 32, ctx)[0] == 42.0
    d[0:2] = (0x7BFF).to_bytes(2, "little")
    d[2] = 1
    assert gq.DequantizeQ8_0(d, 32, ctx)[0] == 65504.0
    got = gq.DequantizeQ2_K(ds4_golden["q2k_raw"], 256, ctx)
    assert np.array_equal(got.view(np.uint32), ds4_golden["q2k"].view(np.uint32))
    # lm/quant/kquant_test.go:95-108 (1e-6 there; the device values are bit-equal) and :151-179
    got = gq.DequantizeIQ2_XXS(ds4_golden["iq2_raw"], 256, ctx)
    assert np.array_equal(got.view(np.uint32), ds4_golden["iq2"].view(np.uint32))
    blk = bytearray(66)
    blk[0:2] = b"\x00\x3c"
    assert np.all(gq.DequantizeIQ2_XXS(blk, 256, ctx) == np.float32(1.0))
    blk[2 + 7] = 0xF0
    got = gq.DequantizeIQ2_XXS(blk, 256, ctx)
    assert got[0] == np.float32(0.125 * 31 * 8) and got[32] == np.float32(1.0)


@pytest.mark.parametrize("fmt", [2, 8, 10, 12, 16])
def test_random_bytes_bit_exact(ctx, fmt):
    """Uniform random bytes reach every scale pattern: subnormal, inf and NaN
    fp16 scales included."""
    be, bb = FMTS[fmt]
    g = np.random.Generator(np.random.Philox(key=100 + fmt))
    for nblocks in (1, 3, 257, 4096):
        raw = g.integers(0, 256, nblocks * bb, dtype=np.uint8)
        got = ctx.dequantize_host(fmt, raw, nblocks * be)
        with np.errstate(all="ignore"):
            want = oracle.Dequantize(fmt, raw, nblocks * be)
        assert _same_bits(got, want)


@pytest.mark.parametrize("fmt", [2, 8, 12])
def test_store_dequantize_matrix(ctx, devbuf, fmt):
    """A stored matrix (ragged row count, K not a whole 256 unit for the
    32-element formats) dequantizes to the oracle's values."""
    from lib_b200 import synth
    rows, cols = 37, (768 if fmt == 12 else 736)
    raw = synth.weights(fmt, rows, cols, seed=5)
    w = ctx.store_upload(fmt, rows, cols, raw)
    out = devbuf(nbytes=rows * cols * 4)
    ctx.dequantize(w, out.ptr)
    ctx.sync()
    got = out.get((rows * cols,))
    assert _same_bits(got, oracle.Dequantize(fmt, raw, rows * cols))
    # row shard [5, 20) holds exactly those rows
    ws = ctx.store_upload(fmt, rows, cols, raw, 5, 20)
    ctx.dequantize(ws, out.ptr)
    ctx.sync()
    got = out.get((15 * cols,))
    assert _same_bits(got, oracle.Dequantize(fmt, raw, rows * cols).reshape(rows, cols)[5:20].reshape(-1))
    w.free()
    ws.free()


@pytest.mark.parametrize("fmt", [2, 8, 10, 12, 16])
def test_error_paths(ctx, fmt):
    be, bb = FMTS[fmt]
    for data, n, code in [(bytes(bb), be // 2, -1), (bytes(bb), -be, -1), (bytes(bb - 1), be, -2)]:
        with pytest.raises(lib_b200.QmError) as e:
            ctx.dequantize_host(fmt, data, n)
        assert e.value.code == code
    assert ctx.dequantize_host(fmt, bytes(bb + 7), be).shape == (be,)
    assert ctx.dequantize_host(fmt, b"", 0).shape == (0,)
    with pytest.raises(lib_b200.QmError) as e:
        ctx.dequantize_host(99, bytes(64), 32)
    assert e.value.code == -3


def test_ggufpy_vectors_on_device(ctx):
    """The committed vectors of the GGUF format's upstream Python decoder, decoded on the device."""
    import json
    import os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    fx = json.load(open(os.path.join(root, "tests/golden/ggufpy_vectors.json")))["formats"]
    ids = {"Q4_0": 2, "Q8_0": 8, "Q2_K": 10, "Q4_K": 12, "IQ2_XXS": 16}
    for name, cases in fx.items():
        be, bb = FMTS[ids[name]]
        for case, v in cases.items():
            raw = bytes.fromhex(v["raw"])
            want = np.array(v["bits"], dtype=np.uint32).view(np.float32)
            got = ctx.dequantize_host(ids[name], raw, len(raw) // bb * be)
            assert _same_bits(got, want), (name, case)


def test_full_size_q8_0_bit_exact(ctx):
    """Config 1 at full size: 4096 x 4096 Q8_0, all 16.7M values bit-equal."""
    from lib_b200 import synth
    raw = synth.weights(8, 4096, 4096, seed=1)
    got = ctx.dequantize_host(8, raw, 4096 * 4096)
    assert _same_bits(got, oracle.DequantizeQ8_0(raw, 4096 * 4096))
