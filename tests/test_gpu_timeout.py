"""A bounded device-side wait that runs out, without faulting anything: a tensor-parallel stack of
world size 2 runs on ONE GPU as rank 0 while nobody plays rank 1. Its "peer" arena is a second
buffer on the same GPU, so rank 0's stores go somewhere harmless, and the words rank 1 would
have written stay "not yet written". With a short wait limit (QM_WAIT_LIMIT, SM clock cycles)
every warp gives up at its first wait, sets the status word and runs to the end of the launch;
the host reads QM_ERR_TIMEOUT, and the context is as usable afterwards as before.

The same construction as the status word of the reference's bounded worker
(nvidia/x/cudamega/cudasrc/finite_worker.cu:1-10): a wait that ends by a limit, reported to the
host, instead of a trap or an endless loop."""
import os

import numpy as np
import pytest

import lib_b200
from lib_b200 import _capi, decode, synth
from oracle import oracle

pytestmark = pytest.mark.gpu


def test_wait_runs_out_and_context_stays_usable(ctx, devbuf, monkeypatch):
    layers, hidden, kv, ffn, fmt, seed = 2, 512, 128, 768, 12, 91
    monkeypatch.setenv("QM_WAIT_LIMIT", "20000000")   # ~10 ms of SM clock per wait instead of ~2 s
    st = _capi.Stack(ctx, layers, hidden, kv, ffn, 2, rank=0, world=2)
    weights = []
    for L in range(layers):
        ws = []
        for rows, cols, parts in decode.stacked(decode.layer_tensors(fmt, hidden, kv, ffn, seed, L)):
            lo, hi = decode.shard_range(rows, 0, 2)
            ws.append(decode.upload_rows(ctx, fmt, rows, cols, parts, lo, hi))
        st.set_layer(L, *ws)
        weights += ws
    base, nbytes = st.arena()
    fake_peer = devbuf(nbytes=nbytes)            # where rank 0's slices for "rank 1" land; nobody reads it
    st.set_peer_pointers([base, fake_peer.ptr])
    x = synth.activations(1, hidden, 5)
    st.step_host(x)                               # returns: every wait is bounded
    rc, status = ctx.last_status()
    assert rc == -8 and (status & 1) == 1         # QM_ERR_TIMEOUT, QM_STATUS_TIMEOUT
    assert ctx.last_status() == (0, 0)            # reading the status cleared it
    st.close()
    for w in weights:
        w.free()
    # the context is intact: an ordinary matvec and an ordinary step run clean and match the oracle
    monkeypatch.delenv("QM_WAIT_LIMIT")
    raw = synth.weights(fmt, 256, 512, 3)
    w = ctx.store_upload(fmt, 256, 512, raw)
    y = ctx.matvec_host(w, x)
    want = oracle.MatVec(fmt, raw, 256, 512, x)
    assert float(np.linalg.norm(y - want) / np.linalg.norm(want)) <= 2e-5
    w.free()
    one = decode.SingleGpuDecode(ctx, layers, hidden, kv, ffn, fmt, seed, m_max=2)
    h = one.stack.step_host(x)
    assert np.isfinite(h).all()
    assert ctx.last_status() == (0, 0)
    one.close()
