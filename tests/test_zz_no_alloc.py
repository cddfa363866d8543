"""GPU test of qm_matvec_noalloc, the matvec for callers that cannot allocate device memory
where they call it (frozen memory plan, latency-critical loop, allocator owned by the host
framework). It keeps its split-K scratch in a fixed array inside the library instead of
allocated buffers, so its results must match qm_matvec's on the same inputs — checked here
on two calls in a row, because the second call starts from whatever the first left in the
shared array. The file name sorts last on purpose: a run that stops at the first failure has
then already run every other test."""
import numpy as np
import pytest

import lib_b200
from lib_b200 import synth

pytestmark = pytest.mark.gpu
# normwise; the bounds the other matvec tests hold these formats to: qm_matvec quantizes three and more
# activation rows into two 7-bit limbs, qm_matvec_noalloc keeps fp16 pairs for every batch
def tol(m):
    return 3e-4 if m > 2 else 2e-5


def nre(got, want):
    return float(np.linalg.norm(got.astype(np.float64) - want.astype(np.float64)) / max(np.linalg.norm(want), 1e-30))


def device_sync():
    import torch
    torch.cuda.synchronize()


@pytest.mark.parametrize("fmt,rows,cols,m", [
    (2, 4096, 14336, 8),   # split over K slices: partial sums and tickets in the fixed array
    (8, 1000, 4128, 3),    # ragged rows, K ending inside a 256-column unit
    (2, 320, 1024, 1),
])
def test_noalloc_matches_matvec_twice(ctx, devbuf, fmt, rows, cols, m):
    raw = synth.weights(fmt, rows, cols, seed=700 + fmt + m)
    w = ctx.store_upload(fmt, rows, cols, raw)
    xs = [synth.activations(m, cols, seed=800 + i) for i in range(2)]
    for x in xs:   # two calls in a row, different inputs
        xd = devbuf(x)
        y_ref = devbuf(np.zeros((m, rows), np.float32))
        y_new = devbuf(np.full((m, rows), np.nan, np.float32))
        ctx.matvec(w, xd.ptr, m, cols, y_ref.ptr, rows)
        ctx.sync()
        ctx.matvec_noalloc(w, xd.ptr, m, cols, y_new.ptr, rows)
        device_sync()
        assert ctx.noalloc_status() == (0, 0)   # no bounded wait of the kernel ran out
        want, got = y_ref.get((m, rows)), y_new.get((m, rows))
        assert np.isfinite(got).all()
        assert nre(got, want) <= tol(m)
    w.free()


def test_noalloc_rejects_what_it_cannot_hold(ctx, devbuf):
    xd, yd = devbuf(nbytes=8 * 4096 * 4), devbuf(nbytes=8 * 4096 * 4)
    wk = ctx.store_upload(12, 64, 256, synth.weights(12, 64, 256, 1))
    with pytest.raises(lib_b200.QmError) as e:
        ctx.matvec_noalloc(wk, xd.ptr, 1, 256, yd.ptr, 64)
    assert e.value.code == -3          # only Q4_0 / Q8_0
    wk.free()
    # 200000 rows x 8192 columns at m = 8 needs far more than 4 MiB of partial sums; the store
    # entry is created empty (zero blocks) just to carry the shape
    big = ctx.store_create(2, 200000, 8192)
    xb, yb = devbuf(nbytes=8 * 8192 * 4), devbuf(nbytes=8 * 200000 * 4)
    with pytest.raises(lib_b200.QmError) as e:
        ctx.matvec_noalloc(big, xb.ptr, 8, 8192, yb.ptr, 200000)
    assert e.value.code == -11         # QM_ERR_LIMIT: beyond the fixed scratch array
    big.free()
