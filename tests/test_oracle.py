"""CPU tests: the oracle against every golden vector and known-answer test the
reference holds for this path. Structured after lm/quant/quant_test.go,
lm/quant/kquant_test.go, lm/moe/moe_test.go, lm/moe/routing_test.go and
gguf/gguf_test.go."""
import json
import math
import os

import numpy as np
import pytest

from oracle import npref, oracle as quant

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_dequantize_q4_0_known_answer():
    # lm/quant/quant_test.go:12-28
    data = bytearray(18)
    data[0:2] = (0x3C00).to_bytes(2, "little")
    data[2] = 0x98
    out = quant.DequantizeQ4_0(data, 32)
    assert out[0] == 0.0 and out[16] == 1.0


def test_dequantize_q8_0_known_answer():
    # lm/quant/quant_test.go:30-43
    data = bytearray(34)
    data[0:2] = (0x3C00).to_bytes(2, "little")
    data[2] = 42
    assert quant.DequantizeQ8_0(data, 32)[0] == 42.0


def test_q8_0_max_finite_scale():
    # nvidia/x/cudaquant/contract_test.go:58-67
    data = bytearray(34)
    data[0:2] = (0x7BFF).to_bytes(2, "little")
    data[2] = 1
    assert quant.DequantizeQ8_0(data, 32)[0] == 65504.0


def test_nibble_order():
    # apple/x/metal/metalquant/roundtrip_test.go:197-212: element i in the low
    # nibble of byte i, element i+16 in the high nibble
    data = bytearray(18)
    data[0:2] = (0x3C00).to_bytes(2, "little")
    for i in range(16):
        data[2 + i] = i | ((15 - i) << 4)
    out = quant.DequantizeQ4_0(data, 32)
    assert list(out[:16]) == [i - 8 for i in range(16)]
    assert list(out[16:]) == [15 - i - 8 for i in range(16)]


def test_q2_k_golden_bit_exact(ds4_golden):
    # lm/quant/kquant_test.go:80-91
    got = quant.DequantizeQ2_K(ds4_golden["q2k_raw"], 256)
    assert np.array_equal(got.view(np.uint32), ds4_golden["q2k"].view(np.uint32))


def test_q2_k_layout():
    # lm/quant/kquant_test.go:112-146
    block = bytearray(84)
    for i in range(16):
        block[i] = 0x21
    block[80:82] = b"\x00\x3c"
    block[82:84] = b"\x00\x3c"
    block[16] = 0b11100100
    got = quant.DequantizeQ2_K(block, 256)
    for idx, want in [(0, -2.0), (32, -1.0), (64, 0.0), (96, 1.0), (1, -2.0)]:
        assert got[idx] == want


@pytest.mark.parametrize("fn,blk,n_partial", [
    (quant.DequantizeQ2_K, 84, 128), (quant.DequantizeQ4_K, 144, 128), (quant.DequantizeIQ2_XXS, 66, 128),
    (quant.DequantizeQ4_0, 18, 16), (quant.DequantizeQ8_0, 34, 16)])
def test_error_paths(fn, blk, n_partial):
    # lm/quant/kquant_test.go:181-202
    full = 256 if blk in (84, 144, 66) else 32
    with pytest.raises(quant.OracleError):
        fn(bytes(blk), n_partial)
    with pytest.raises(quant.OracleError):
        fn(bytes(blk), -full)
    with pytest.raises(quant.OracleError):
        fn(bytes(blk - 1), full)
    assert fn(bytes(blk + 5), full).shape == (full,)  # trailing bytes are accepted
    assert fn(b"", 0).shape == (0,)


def test_float16_known_values_and_exhaustive():
    # apple/x/metal/metalquant/roundtrip_test.go:12-65 (values) + every pattern
    for h, want in [(0x0000, 0.0), (0x3C00, 1.0), (0xBC00, -1.0), (0x4000, 2.0), (0x3800, 0.5),
                    (0x7BFF, 65504.0), (0x0001, 2.0 ** -24), (0x0400, 2.0 ** -14),
                    (0x03FF, 1023 * 2.0 ** -24)]:
        assert float(quant.Float16ToFloat32(h)) == want
    assert quant.Float16ToFloat32Bits(0x8000) == 0x80000000
    assert quant.Float16ToFloat32Bits(0x7C00) == 0x7F800000
    assert quant.Float16ToFloat32Bits(0x7D01) == 0x7F800000 | (0x101 << 13)  # payload kept, not quieted
    allh = np.arange(65536, dtype=np.uint16)
    ref = allh.view(np.float16).astype(np.float32)
    got = np.array([quant.Float16ToFloat32Bits(int(h)) for h in allh], dtype=np.uint32).view(np.float32)
    finite = np.isfinite(ref)
    assert np.array_equal(got[finite].view(np.uint32), ref[finite].view(np.uint32))
    assert np.all(np.isnan(got[np.isnan(ref)]))


def test_iq2_xxs_golden(ds4_golden):
    # lm/quant/kquant_test.go:95-108 (tolerance 1e-6*(1+|want|) there; the values agree bit for bit)
    got = quant.DequantizeIQ2_XXS(ds4_golden["iq2_raw"], 256)
    want = ds4_golden["iq2"]
    assert np.all(np.abs(got.astype(np.float64) - want) <= 1e-6 * (1 + np.abs(want.astype(np.float64))))
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_iq2_xxs_layout():
    # lm/quant/kquant_test.go:151-179
    block = bytearray(66)
    block[0:2] = b"\x00\x3c"
    plain = quant.DequantizeIQ2_XXS(block, 256)
    assert np.all(plain == np.float32(0.125 * 8))
    block[2 + 7] = 0xF0
    got = quant.DequantizeIQ2_XXS(block, 256)
    assert got[0] == np.float32(0.125 * 31 * 8)
    assert got[32] == np.float32(0.125 * 8)
    # sign index 1 negates element 0 and, through the parity bit, element 7
    block = bytearray(66)
    block[0:2] = b"\x00\x3c"
    block[2 + 4] = 0x01
    got = quant.DequantizeIQ2_XXS(block, 256)
    assert list(got[:8]) == [-1.0, 1.0, 1.0, 1.0, 1.0, 1.0, 1.0, -1.0]


GGUFPY = {"Q4_0": (2, 32, 18), "Q8_0": (8, 32, 34), "Q2_K": (10, 256, 84), "Q4_K": (12, 256, 144),
          "IQ2_XXS": (16, 256, 66)}


def _same_bits(a, b):
    return bool(((a.view(np.uint32) == b.view(np.uint32)) | (np.isnan(a) & np.isnan(b))).all())


@pytest.mark.parametrize("name", sorted(GGUFPY))
def test_oracle_matches_ggufpy_fixture(name):
    """The committed vectors of the GGUF format's upstream Python decoder (gguf-py): this is what
    pins Q4_K, for which the reference holds no vector. Bit for bit (NaNs as NaNs)."""
    fmt, be, bb = GGUFPY[name]
    fx = json.load(open(os.path.join(ROOT, "tests/golden/ggufpy_vectors.json")))["formats"][name]
    assert fx
    for case, v in fx.items():
        raw = bytes.fromhex(v["raw"])
        want = np.array(v["bits"], dtype=np.uint32).view(np.float32)
        with np.errstate(all="ignore"):
            got = quant.Dequantize(fmt, raw, len(raw) // bb * be)
        assert _same_bits(got, want), (name, case)


@pytest.mark.parametrize("name", sorted(GGUFPY))
def test_oracle_matches_ggufpy_live(name):
    """Same comparison against the installed package, on more data: random bytes, the benchmark's
    seeded tensors (config 3: 4096-wide Q4_K rows) and a patterned block."""
    gguf = pytest.importorskip("gguf", reason="gguf-py is not installed; the committed fixture still pins the oracle")
    from gguf import quants
    from lib_b200 import synth
    fmt, be, bb = GGUFPY[name]
    qtype = getattr(gguf.GGMLQuantizationType, name)
    g = np.random.Generator(np.random.Philox(key=31))
    raws = [g.integers(0, 256, bb * 256, dtype=np.uint8), (np.arange(bb * 3, dtype=np.uint32) * 37 + 11).astype(np.uint8)]
    if fmt in synth.BLOCK:
        raws.append(synth.weights(fmt, 16, 4096, seed=3))
    for raw in raws:
        n = raw.size // bb * be
        with np.errstate(all="ignore"):
            want = quants.dequantize(raw.reshape(1, -1), qtype).reshape(-1)
            got = quant.Dequantize(fmt, raw, n)
        assert _same_bits(got, want), name


def test_q4_k_two_decoders_agree():
    # a second, independently written numpy decoder must agree bit for bit (the pin itself is the
    # gguf-py comparison above)
    g = np.random.Generator(np.random.Philox(key=7))
    raw = g.integers(0, 256, 144 * 512, dtype=np.uint8)
    a = quant.DequantizeQ4_K(raw, 256 * 512)
    with np.errstate(all="ignore"):
        b = npref.dequantize_q4_k(raw, 256 * 512)
    same = (a.view(np.uint32) == b.view(np.uint32)) | (np.isnan(a) & np.isnan(b))
    assert same.all()
    fx = json.load(open(os.path.join(ROOT, "tests/golden/q4k_selfcheck.json")))
    got = quant.DequantizeQ4_K(bytes.fromhex(fx["raw"]), 1024)
    want = np.array(fx["bits"], dtype=np.uint32)
    ok = (got.view(np.uint32) == want) | np.isnan(got)
    assert ok.all()


def test_q4_k_hand_built_block():
    # d = 1, dmin = 1; sub-block 0: scale 3 min 2; sub-block 5: scale 33 min 44 (uses the split bits)
    blk = bytearray(144)
    blk[0:2] = b"\x00\x3c"
    blk[2:4] = b"\x00\x3c"
    S = [0] * 12
    S[0] = 3
    S[4] = 2
    sc5, m5 = 33, 44
    S[9] = (sc5 & 15) | ((m5 & 15) << 4)
    S[1] |= (sc5 >> 4) << 6
    S[5] |= (m5 >> 4) << 6
    blk[4:16] = bytes(S)
    blk[16 + 0] = 0x07          # element 0 of sub-block 0 = 7 ; element 0 of sub-block 1 = 0
    blk[16 + 64 + 3] = 0xA0     # bytes 64..95 hold sub-blocks 4 (low) and 5 (high): element 3 of sub-block 5 = 10
    out = quant.DequantizeQ4_K(blk, 256)
    assert out[0] == 3 * 7 - 2
    assert out[1] == -2.0
    assert out[5 * 32 + 3] == 33 * 10 - 44
    assert out[5 * 32 + 4] == -44.0
    assert out[4 * 32 + 3] == 0.0


def test_small_decoders_agree():
    g = np.random.Generator(np.random.Philox(key=9))
    raw = g.integers(0, 256, 18 * 64, dtype=np.uint8)
    with np.errstate(all="ignore"):
        a, b = quant.DequantizeQ4_0(raw, 32 * 64), npref.dequantize_q4_0(raw, 32 * 64)
    assert ((a.view(np.uint32) == b.view(np.uint32)) | (np.isnan(a) & np.isnan(b))).all()
    raw = g.integers(0, 256, 34 * 64, dtype=np.uint8)
    with np.errstate(all="ignore"):
        a, b = quant.DequantizeQ8_0(raw, 32 * 64), npref.dequantize_q8_0(raw, 32 * 64)
    assert ((a.view(np.uint32) == b.view(np.uint32)) | (np.isnan(a) & np.isnan(b))).all()


# ---- router: lm/moe/moe_test.go, lm/moe/routing_test.go -------------------------------
LOGITS8 = [0.1, 2.5, 0.3, 0.4, 5.0, 1.2, 0.8, 0.2]


def test_route_top2():
    ids, w = quant.Route(LOGITS8, 8, 2)
    assert list(ids) == [4, 1]


def test_route_weights_are_a_softmax():
    ids, w = quant.Route(LOGITS8, 8, 3)
    assert list(ids) == [4, 1, 5]
    den = sum(math.exp(float(np.float32(LOGITS8[i]) - np.float32(5.0))) for i in ids)
    for i, e in enumerate(ids):
        assert abs(float(w[i]) - math.exp(float(np.float32(LOGITS8[e]) - np.float32(5.0))) / den) < 1e-6
    assert abs(float(w.sum()) - 1) < 1e-6


def test_route_bias_selects_without_reweighting():
    logits = [1.0, 0.9, 0.2, 0.1]
    ids, _ = quant.Route(logits, 4, 2)
    assert list(ids) == [0, 1]
    ids, w = quant.Route(logits, 4, 2, biases=[0, 0, 5, 0])
    assert list(ids) == [2, 0]
    assert abs(float(w[1] / w[0]) - math.exp(0.8)) < 1e-5
    assert abs(float(w.sum()) - 1) < 1e-6


def test_route_ties_and_degenerate():
    ids, w = quant.Route([0.0] * 16, 16, 4)
    assert list(ids) == [0, 1, 2, 3] and np.allclose(w, 0.25, atol=1e-6)
    ids, w = quant.Route([1, 2], 2, 8)
    assert len(ids) == 2 and len(w) == 2
    ids, w = quant.Route([1], 8, 2)
    assert len(ids) == 1
    ids, w = quant.Route([1, 2, 3, 4], 4, 0)
    assert len(ids) == 0 and len(w) == 0


# ---- gguf sizes: gguf/gguf_test.go:125-160 ----------------------------------------------
def test_tensor_bytes():
    assert quant.TensorBytes(16, [256, 2]) == 132
    assert quant.TensorBytes(12, [4096, 4096]) == 9437184
    assert quant.TensorBytes(8, [4096, 4096]) == 17825792
    assert quant.TensorBytes(2, [4096, 14336]) == 33030144
    with pytest.raises(quant.OracleError):
        quant.TensorBytes(16, [128, 2])
    with pytest.raises(quant.OracleError):
        quant.TensorBytes(4242, [32])
    with pytest.raises(quant.OracleError):
        quant.TensorBytes(0, [2 ** 62, 16])


def test_matvec_oracle_matches_numpy():
    from lib_b200 import synth
    for fmt, dec in [(2, npref.dequantize_q4_0), (8, npref.dequantize_q8_0), (12, npref.dequantize_q4_k)]:
        raw = synth.weights(fmt, 8, 512, seed=3)
        x = synth.activations(2, 512, seed=4)
        W = dec(raw, 8 * 512).reshape(8, 512).astype(np.float64)
        want = (x.astype(np.float64) @ W.T).astype(np.float32)
        assert np.array_equal(quant.MatVec(fmt, raw, 8, 512, x), want)
        got32 = quant.MatVec(fmt, raw, 8, 512, x, threads=3)
        assert np.allclose(got32, want, rtol=1e-4, atol=1e-5)
