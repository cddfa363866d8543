"""Generates tests/golden/ggufpy_vectors.json from the gguf Python package
(gguf-py, the GGUF format's upstream Python implementation; its
`gguf.quants.dequantize` is the published decoder of every GGUF tensor type).

Run where the package is importable:
    python tests/golden/make_golden_ggufpy.py
The fixture pins the CPU oracle for the formats the reference itself holds no
vector for (Q4_K, GGUF type 12) and adds independent vectors for the others:
per format a few blocks of raw bytes and the float32 bit patterns gguf-py
decodes them to. Raw bytes: uniform random (every packing of the 6-bit fields,
every fp16 class incl. subnormal/inf/NaN scales), the benchmark's seeded
distribution, and one patterned block.
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

FORMATS = {"Q4_0": (2, 32, 18), "Q8_0": (8, 32, 34), "Q2_K": (10, 256, 84), "Q4_K": (12, 256, 144),
           "IQ2_XXS": (16, 256, 66)}


def cases(name, block_bytes):
    from lib_b200 import synth
    g = np.random.Generator(np.random.Philox(key=20240611))
    fmt = FORMATS[name][0]
    out = {"random": g.integers(0, 256, 6 * block_bytes, dtype=np.uint8)}
    if fmt in synth.BLOCK:
        be = synth.BLOCK[fmt][0]
        out["seeded"] = synth.weights(fmt, 2, 2 * max(be, 256), seed=77)[:6 * block_bytes].copy()
    pat = (np.arange(2 * block_bytes, dtype=np.uint32) * 37 + 11).astype(np.uint8)
    # finite scales in the patterned blocks: fp16 1.0 / 0.5 in every 2-byte scale field position used
    out["patterned"] = pat
    return out


def main():
    import gguf
    from gguf import GGMLQuantizationType as T
    from gguf import quants
    doc = {"source": "gguf-py %s, gguf.quants.dequantize" % getattr(gguf, "__version__", "(unversioned)"),
           "formats": {}}
    for name, (fmt, be, bb) in FORMATS.items():
        entry = {}
        for case, raw in cases(name, bb).items():
            nb = raw.size // bb
            with np.errstate(all="ignore"):
                vals = quants.dequantize(raw[:nb * bb].reshape(1, -1), getattr(T, name)).reshape(-1)
            assert vals.dtype == np.float32 and vals.size == nb * be
            entry[case] = {"raw": raw[:nb * bb].tobytes().hex(), "bits": [int(v) for v in vals.view(np.uint32)]}
        doc["formats"][name] = entry
    json.dump(doc, open(os.path.join(HERE, "ggufpy_vectors.json"), "w"))


if __name__ == "__main__":
    main()
