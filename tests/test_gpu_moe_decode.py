"""Decode-time MoE over selected Q4_K experts (qm_moe_decode_*): one launch of the decode GEMV kernels for all
(token, slot) pairs, against the oracle chain gate|up -> silu(gate)*up -> down -> weighted sum on the same
seeded inputs. Tolerance: normwise 1e-4 (float32 activations, three-limb quantization, fast exponential in the
SwiGLU staging)."""
import numpy as np
import pytest

import lib_b200
from lib_b200 import synth
from oracle import oracle

pytestmark = pytest.mark.gpu


def chain(gu_raw, dn_raw, hidden, ffn, x, ids, wts):
    out = np.zeros((x.shape[0], hidden), np.float64)
    for t in range(x.shape[0]):
        for s in range(ids.shape[1]):
            e = int(ids[t, s])
            gu = oracle.MatVec(12, gu_raw[e], 2 * ffn, hidden, x[t]).astype(np.float64)
            h = (gu[:ffn] / (1 + np.exp(-gu[:ffn])) * gu[ffn:]).astype(np.float32)
            out[t] += float(wts[t, s]) * oracle.MatVec(12, dn_raw[e], hidden, ffn, h).astype(np.float64)
    return out


@pytest.mark.parametrize("experts,hidden,ffn,tokens,topk", [(4, 512, 768, 1, 2), (8, 1024, 1792, 3, 2), (6, 256, 512, 4, 3)])
def test_decode_moe_matches_oracle_chain(ctx, devbuf, experts, hidden, ffn, tokens, topk):
    gu_raw = [synth.weights(12, 2 * ffn, hidden, 40 + e) for e in range(experts)]
    dn_raw = [synth.weights(12, hidden, ffn, 140 + e) for e in range(experts)]
    gu = [ctx.store_upload(12, 2 * ffn, hidden, r) for r in gu_raw]
    dn = [ctx.store_upload(12, hidden, ffn, r) for r in dn_raw]
    md = ctx.moe_decode_create(gu, dn, topk, 4)
    x = synth.activations(tokens, hidden, 7)
    logits = synth.activations(tokens, experts, 8)
    ld, xd = devbuf(logits), devbuf(x)
    ids_d, wts_d = devbuf(nbytes=tokens * topk * 4), devbuf(nbytes=tokens * topk * 4)
    out_d = devbuf(nbytes=tokens * hidden * 4)
    launches = ctx.launch_count()
    ctx.moe_route(ld.ptr, tokens, experts, experts, topk, ids_d.ptr, wts_d.ptr)
    ctx.moe_decode_run(md, xd.ptr, tokens, hidden, ids_d.ptr, wts_d.ptr, out_d.ptr, hidden)
    assert ctx.launch_count() - launches == 3          # route, all matvecs of all pairs, combine
    got = out_d.get((tokens, hidden))
    assert ctx.last_status() == (0, 0)
    ids, wts = ids_d.get((tokens, topk), np.int32), wts_d.get((tokens, topk))
    want = chain(gu_raw, dn_raw, hidden, ffn, x, ids, wts)
    assert np.linalg.norm(got - want) <= 1e-4 * np.linalg.norm(want)
    # a second run on the same buffers (no rebuild) with other experts chosen
    ids2 = ((ids + 1) % experts).astype(np.int32)
    ctx.h2d(ids_d.ptr, ids2)
    ctx.moe_decode_run(md, xd.ptr, tokens, hidden, ids_d.ptr, wts_d.ptr, out_d.ptr, hidden)
    got2 = out_d.get((tokens, hidden))
    want2 = chain(gu_raw, dn_raw, hidden, ffn, x, ids2, wts)
    assert np.linalg.norm(got2 - want2) <= 1e-4 * np.linalg.norm(want2)
    # an id that names no expert: that token's outputs are NaN, the others are untouched by it
    ids3 = ids.copy()
    ids3[0, 0] = experts + 3
    ctx.h2d(ids_d.ptr, ids3)
    ctx.moe_decode_run(md, xd.ptr, tokens, hidden, ids_d.ptr, wts_d.ptr, out_d.ptr, hidden)
    got3 = out_d.get((tokens, hidden))
    assert np.all(got3[0].view(np.uint32) == 0x7fffffff)
    if tokens > 1:
        assert np.array_equal(got3[1:], got[1:])
    assert ctx.last_status() == (0, 0)
    ctx.moe_decode_destroy(md)
    for w in gu + dn:
        w.free()


def test_decode_moe_refusals(ctx, devbuf):
    gu = [ctx.store_upload(12, 512, 256, synth.weights(12, 512, 256, 1)) for _ in range(2)]
    dn = [ctx.store_upload(12, 256, 256, synth.weights(12, 256, 256, 2)) for _ in range(2)]
    with pytest.raises(lib_b200.QmError) as e:
        ctx.moe_decode_create(gu, dn, 2, 17)             # 34 pairs
    assert e.value.code == -4
    bad = [ctx.store_upload(12, 256, 512, synth.weights(12, 256, 512, 3)), dn[1]]
    with pytest.raises(lib_b200.QmError) as e:
        ctx.moe_decode_create(gu, bad, 2, 1)             # a down matrix of another shape
    assert e.value.code == -4
    md = ctx.moe_decode_create(gu, dn, 2, 2)
    b = devbuf(nbytes=4096)
    with pytest.raises(lib_b200.QmError) as e:
        ctx.moe_decode_run(md, b.ptr, 3, 256, b.ptr, b.ptr, b.ptr, 256)   # more tokens than created for
    assert e.value.code == -4
    ctx.moe_decode_destroy(md)
    for w in gu + dn + bad[:1]:
        w.free()
