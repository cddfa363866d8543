import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200; run with -m gpu on the GPU box")


def _have_gpu():
    return os.path.exists("/dev/nvidia0") or os.path.exists("/dev/nvidiactl")


def pytest_collection_modifyitems(config, items):
    if _have_gpu():
        return
    skip = pytest.mark.skip(reason="no GPU on this machine")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def ctx():
    """One qm_ctx for the whole session. Creation fails loudly when the CUDA
    library cannot run; the GPU tests never fall back to anything else."""
    import lib_b200
    c = lib_b200.Context(0)
    yield c
    c.close()


@pytest.fixture(scope="session")
def ds4_golden():
    g = json.load(open(os.path.join(ROOT, "tests/golden/ds4_superblocks.json")))
    return {
        "q2k_raw": bytes.fromhex(g["q2k_raw"]),
        "iq2_raw": bytes.fromhex(g["iq2_raw"]),
        "q2k": np.array([np.float32(v) for v in g["q2k"]], dtype=np.float32),
        "iq2": np.array([np.float32(v) for v in g["iq2"]], dtype=np.float32),
    }


class DevBuf:
    """Device buffer helper over the C ABI (qm_malloc / qm_memcpy_*)."""

    def __init__(self, ctx, arr=None, nbytes=None):
        self.ctx = ctx
        if arr is not None:
            arr = np.ascontiguousarray(arr)
            nbytes = arr.nbytes
        self.nbytes = nbytes
        self.ptr = ctx.malloc(nbytes)
        if arr is not None:
            ctx.h2d(self.ptr, arr)

    def get(self, shape, dtype=np.float32):
        out = np.empty(shape, dtype=dtype)
        self.ctx.d2h(out, self.ptr)
        return out

    def free(self):
        if self.ptr:
            self.ctx.free(self.ptr)
            self.ptr = 0


@pytest.fixture
def devbuf(ctx):
    made = []

    def make(arr=None, nbytes=None):
        b = DevBuf(ctx, arr, nbytes)
        made.append(b)
        return b
    yield make
    for b in made:
        b.free()
