"""The analytic RMSNorm -> Q8_1 fixtures and contract cases of the reference's tests
(nvidia/x/cudaquant/norm_source_test.go:24-66 normFixtures, norm_contract_test.go:8-52,
quant_test.go:10-34), shared by the oracle's CPU tests and the device tests."""
import struct

import numpy as np


def block_bytes(d, s, quants):
    """One 36-byte block as norm_source_test.go:68-78 normBytes lays it out."""
    return struct.pack("<HH", d, s) + bytes((q & 0xFF) for q in quants)


def norm_fixtures():
    """[(name, rows, cols, epsilon, weighted, input, weight, expected bytes)]: constant rows normalise to 1
    (or 1/2 with epsilon 3); the weighted case has scale exactly 1 and rounding ties of both signs."""
    out = []
    weight = np.array([[127, 0.5, -0.5, 1.5, -1.5, 0, 0, 0][i % 8] for i in range(64)], dtype=np.float32)
    ones = np.ones(128, dtype=np.float32)
    out.append(("unweighted", 2, 64, 0.0, False, ones, weight, block_bytes(0x2008, 0x5000, [127] * 32) * 4))
    out.append(("epsilon", 2, 64, 3.0, False, ones, weight, block_bytes(0x1c08, 0x4c00, [127] * 32) * 4))
    ties = [[127, 1, -1, 2, -2, 0, 0, 0][i % 8] for i in range(32)]
    out.append(("weighted_ties", 2, 64, 0.0, True, ones, weight, block_bytes(0x3c00, 0x5ff0, ties) * 4))
    out.append(("zero", 2, 64, 1.0, False, np.zeros(128, dtype=np.float32), weight, bytes(36 * 4)))
    return out


# (value, binary16 bits) of norm_contract_test.go:54-66 TestBinary16Rounding
BINARY16_CASES = [(0.0, 0), (1.0, 0x3c00), (-2.0, 0xc000), (65504.0, 0x7bff), (2.0 ** -24, 1),
                  (1 + 1.0 / 2048, 0x3c00), (1 + 3.0 / 2048, 0x3c02)]


def random_rows(rows, cols, seed, scale=1.0):
    rng = np.random.default_rng(seed)
    x = (rng.standard_normal((rows, cols)) * scale).astype(np.float32)
    w = (1.0 + 0.25 * rng.standard_normal(cols)).astype(np.float32)
    return x, w
