"""Generates the committed fixtures of tests/golden/ from the reference checkout.

Run in a container that has the reference mounted:
    python tests/golden/make_golden.py <path of the reference checkout>
Writes
  ds4_superblocks.json  the two pseudorandom super-blocks and the 2x256 expected
                        values of lm/quant/testdata/ds4_golden.txt, after checking
                        that the reference's own generator (built from
                        lm/quant/testdata/ds4_golden.c by oracle/Makefile) still
                        reproduces that file;
  q4k_selfcheck.json    four Q4_K super-blocks with the values on which the C
                        oracle and the numpy decoder agree bit for bit. NOT a
                        reference vector: the reference has none for Q4_K.
"""
import json
import os
import subprocess
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)


def parse(text):
    out = {"q2k_raw": None, "iq2_raw": None, "q2k": [None] * 256, "iq2": [None] * 256}
    for line in text.splitlines():
        if not line or line.startswith("#"):
            continue
        f = line.split()
        if f[0] in ("q2k_raw", "iq2_raw"):
            out[f[0]] = f[1]
        else:
            out[f[0]][int(f[1])] = f[2]
    return out


def main():
    if len(sys.argv) < 2:
        sys.exit(__doc__)
    ref = sys.argv[1]
    txt = open(os.path.join(ref, "lm/quant/testdata/ds4_golden.txt")).read()
    gold = parse(txt)
    subprocess.check_call(["make", "-C", os.path.join(ROOT, "oracle"), "ref", "REFERENCE=" + ref],
                          stdout=subprocess.DEVNULL)
    regenerated = subprocess.check_output([os.path.join(ROOT, "oracle/_ref/ds4_golden")], text=True)
    assert parse(regenerated) == gold, "the reference generator no longer reproduces its golden file"
    gold["source"] = "lm/quant/testdata/ds4_golden.txt (values as decimal strings, parsed as float32)"
    json.dump(gold, open(os.path.join(HERE, "ds4_superblocks.json"), "w"), indent=0)

    from oracle import npref, oracle
    raw = np.random.Generator(np.random.Philox(key=412)).integers(0, 256, 4 * 144, dtype=np.uint8)
    raw[0:4] = np.array([0.0123, 0.0045], dtype=np.float16).view(np.uint8)  # finite scales in block 0
    a = oracle.DequantizeQ4_K(raw, 1024)
    b = npref.dequantize_q4_k(raw, 1024)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    json.dump({"note": "self-check only: no reference vector exists for Q4_K", "raw": raw.tobytes().hex(),
               "bits": [int(v) for v in a.view(np.uint32)]},
              open(os.path.join(HERE, "q4k_selfcheck.json"), "w"))


if __name__ == "__main__":
    main()
