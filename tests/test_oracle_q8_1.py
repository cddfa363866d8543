"""The oracle's Q8_1 producers against the reference's analytic fixtures and contract tests
(nvidia/x/cudaquant/norm_source_test.go, norm_contract_test.go, quant_test.go)."""
import struct

import numpy as np
import pytest

from oracle import oracle
from tests import q8_1_cases as cases


@pytest.mark.parametrize("fx", cases.norm_fixtures(), ids=lambda f: f[0])
def test_norm_analytic_fixtures(fx):
    name, rows, cols, eps, weighted, x, w, want = fx
    assert oracle.RMSNormQ8_1(x, w, rows, cols, eps, weighted) == want


def test_known_q8_1_layout():
    # norm_contract_test.go:8-29: d = 1/127 and s = d * sum(q) = 32 in binary16, every quant 127
    got = oracle.RMSNormQ8_1(np.ones(32, dtype=np.float32), None, 1, 32, 0.0, False)
    assert struct.unpack_from("<HH", got) == (0x2008, 0x5000) and got[4:] == bytes([127] * 32)


@pytest.mark.parametrize("rows,cols,eps,value", [(2 ** 63 - 1, 32, 1.0, 0.0), (1, 32, float("inf"), 0.0),
                                                 (1, 32, 1.0, float("nan")), (1, 32, 0.0, 0.0)],
                         ids=["overflow", "infinite epsilon", "nan input", "zero denominator"])
def test_invalid_inputs(rows, cols, eps, value):
    x = np.zeros(32, dtype=np.float32)
    x[0] = value
    with pytest.raises(oracle.OracleError):
        oracle.RMSNormQ8_1(x, None, rows, cols, eps, False)


def test_more_refusals():
    with pytest.raises(oracle.OracleError, match="weight length"):   # quant_test.go:20-25
        oracle.RMSNormQ8_1(np.zeros(32, dtype=np.float32), np.zeros(31, dtype=np.float32), 1, 32, 1e-5, True)
    with pytest.raises(oracle.OracleError, match="input length"):
        oracle.RMSNormQ8_1(np.zeros(33, dtype=np.float32), None, 1, 32, 1e-5, False)
    with pytest.raises(oracle.OracleError, match="dimensions"):
        oracle.RMSNormQ8_1(np.zeros(48, dtype=np.float32), None, 1, 48, 1e-5, False)
    with pytest.raises(oracle.OracleError, match="dimensions"):
        oracle.RMSNormQ8_1(np.zeros(32, dtype=np.float32), None, 1, 32, -1.0, False)
    w = np.ones(32, dtype=np.float32)
    w[3] = np.inf
    with pytest.raises(oracle.OracleError, match="nonfinite weight"):
        oracle.RMSNormQ8_1(np.ones(32, dtype=np.float32), w, 1, 32, 0.0, True)
    w[3] = 3e38                                                       # finite inputs, infinite product
    with pytest.raises(oracle.OracleError, match="normalized value"):
        oracle.RMSNormQ8_1(np.eye(1, 32, 3, dtype=np.float32), w, 1, 32, 0.0, True)   # sqrt(32) * 3e38


def test_rounding_and_saturation():
    # quant_test.go:26-34: one large value -> quant 127, the rest 0
    x = np.zeros(32, dtype=np.float32)
    x[0] = 100
    got = oracle.RMSNormQ8_1(x, None, 1, 32, 0.0, False)
    assert got[4] == 127 and got[5:] == bytes(31)
    got = oracle.RMSNormQ8_1(np.arange(32, dtype=np.float32), None, 1, 32, 1e-5, False)   # quant_test.go:10-18
    assert len(got) == 36 and got[4 + 31] == 127


@pytest.mark.parametrize("value,bits", cases.BINARY16_CASES)
def test_binary16_rounding(value, bits):
    assert oracle.Float32ToFloat16(value) == bits


def test_binary16_matches_numpy_everywhere_it_matters():
    rng = np.random.default_rng(5)
    v = np.concatenate([rng.standard_normal(20000).astype(np.float32) * np.float32(10.0) ** rng.integers(-9, 5, 20000),
                        np.array([65519.9, 65520.0, 1e6, -1e6, 2.0 ** -25, 2.0 ** -25 * 1.0001, 6.1e-5, 5.96e-8], dtype=np.float32)])
    with np.errstate(over="ignore"):
        want = v.astype(np.float16).view(np.uint16)
    got = np.array([oracle.Float32ToFloat16(x) for x in v], dtype=np.uint16)
    assert np.array_equal(got, want)


def test_norm_blocks_decode_back():
    """d * q reproduces the normalised row to half a quantization step (plus the binary16 rounding of d,
    up to 127 * 2^-11 of a step); s = fp16(qscale * sum q)."""
    x, w = cases.random_rows(3, 256, 11)
    raw = oracle.RMSNormQ8_1(x, w, 3, 256, 1e-6, True)
    back = oracle.DequantizeQ8_1(raw, 3 * 256).reshape(3, 256)
    want = x / np.sqrt((x.astype(np.float64) ** 2).mean(axis=1, keepdims=True) + 1e-6).astype(np.float32) * w
    blocks = np.frombuffer(raw, dtype=np.uint8).reshape(-1, 36)
    d = blocks[:, :2].copy().view(np.float16).astype(np.float32).reshape(3, 8, 1)
    assert np.all(np.abs(back.reshape(3, 8, 32) - want.reshape(3, 8, 32)) <= 0.57 * d + 1e-7)
    q = blocks[:, 4:].view(np.int8).astype(np.int32)
    qscale = np.abs(want.reshape(-1, 32)).max(axis=1) / np.float32(127)
    s = (q.sum(axis=1).astype(np.float32) * qscale).astype(np.float16)
    assert np.array_equal(s.view(np.uint16), blocks[:, 2:4].copy().view(np.uint16).reshape(-1))


def test_swiglu_q8_1_blocks():
    """fused_swiglu_q8_1: clamps, per-slot weight, partial last block, fields as the kernel text sets them."""
    rng = np.random.default_rng(3)
    width, slots = 80, 3      # 240 values: 7 full blocks and one of 16
    gate = (rng.standard_normal(width * slots) * 6).astype(np.float32)
    up = (rng.standard_normal(width * slots) * 6).astype(np.float32)
    gate[5], up[6], up[7] = 50.0, 40.0, -40.0
    wts = np.array([1.0, 0.5, -2.0], dtype=np.float32)
    raw = oracle.SwiGLUQ8_1(gate, up, wts, width, slots)
    assert len(raw) == 8 * 36
    g = np.minimum(gate, np.float32(10))
    u = np.clip(up, np.float32(-10), np.float32(10))
    v = (g / (np.float32(1) + np.exp(-g, dtype=np.float32))) * u * np.repeat(wts, width)
    blocks = np.frombuffer(raw, dtype=np.uint8).reshape(8, 36)
    d = blocks[:, :2].copy().view(np.float16).astype(np.float32).reshape(-1)
    vp = np.concatenate([v, np.zeros(16, dtype=np.float32)]).reshape(8, 32)
    assert np.allclose(d, np.abs(vp).max(axis=1) / 127, rtol=2e-3)
    ssum = blocks[:, 2:4].copy().view(np.float16).astype(np.float32).reshape(-1)
    assert np.allclose(ssum, vp.sum(axis=1), rtol=2e-3, atol=1e-3)
    q = blocks[:, 4:].view(np.int8).astype(np.float32)
    assert np.all(np.abs(q * d[:, None] - vp) <= 0.57 * d[:, None] + 1e-6)
    assert np.all(blocks[7, 4 + 16:] == 0)            # the partial block's tail is never written
    assert abs(vp[0, 5]) <= 10 * 10 + 1e-3             # gate 50 acted as 10


def test_selected_matvec_oracle():
    from lib_b200 import synth
    experts, rows, cols = 4, 8, 512
    raw = synth.weights(10, experts * rows, cols, seed=2)
    x, _ = cases.random_rows(1, cols, 4)
    xq = oracle.RMSNormQ8_1(x, None, 1, cols, 1e-6, False)
    y = oracle.SelectedMatVecQ8_1(10, raw, experts, rows, cols, [2, -1, 0], xq)
    row_bytes = len(raw) // (experts * rows)
    want = oracle.MatVec(10, raw[2 * rows * row_bytes:3 * rows * row_bytes], rows, cols, oracle.DequantizeQ8_1(xq, cols))
    assert np.array_equal(y[0], want) and np.all(np.isnan(y[1])) and not np.any(np.isnan(y[2]))
