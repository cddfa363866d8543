"""GPU parity of the mixture-of-experts path: routing against the oracle's restatement of
GroupedTopKRouter.Route (lm/moe/moe.go:73-141, tests lm/moe/moe_test.go and routing_test.go),
and the grouped expert matmul against the oracle chain on the same seeded inputs.

Tolerance of the grouped matmul: normwise 3e-3 (bf16 activations on the tensor cores)."""
import numpy as np
import pytest

from lib_b200 import synth
from oracle import oracle

pytestmark = pytest.mark.gpu
TOL = 3e-3


def to_bf16_bits(x):
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def bf16_to_f32(b):
    return (b.astype(np.uint32) << 16).view(np.float32)


def route_gpu(ctx, devbuf, logits, experts, topk, bias=None):
    tokens = logits.shape[0]
    ld = devbuf(logits)
    ids = devbuf(np.full((tokens, topk), -7, np.int32))
    wts = devbuf(np.full((tokens, topk), np.nan, np.float32))
    bd = devbuf(np.asarray(bias, np.float32)) if bias is not None else None
    ctx.moe_route(ld.ptr, tokens, logits.shape[1], experts, topk, ids.ptr, wts.ptr, bd.ptr if bd else 0)
    ctx.sync()
    return ids.get((tokens, topk), np.int32), wts.get((tokens, topk)), ids, wts


def test_router_reference_cases(ctx, devbuf):
    lg = np.array([[0.1, 2.5, 0.3, 0.4, 5.0, 1.2, 0.8, 0.2]], np.float32)
    ids, w, *_ = route_gpu(ctx, devbuf, lg, 8, 2)
    assert list(ids[0]) == [4, 1]                                    # lm/moe/moe_test.go:20-27
    ids, w, *_ = route_gpu(ctx, devbuf, lg, 8, 3)
    assert list(ids[0]) == [4, 1, 5] and abs(float(w.sum()) - 1) < 1e-6   # routing_test.go:21-46
    lg4 = np.array([[1.0, 0.9, 0.2, 0.1]], np.float32)
    ids, w, *_ = route_gpu(ctx, devbuf, lg4, 4, 2, bias=[0, 0, 5, 0])
    assert list(ids[0]) == [2, 0] and abs(float(w[0, 1] / w[0, 0]) - np.exp(0.8)) < 1e-5   # :52-83
    ids, w, *_ = route_gpu(ctx, devbuf, np.zeros((1, 16), np.float32), 16, 4)
    assert list(ids[0]) == [0, 1, 2, 3] and np.allclose(w, 0.25, atol=1e-6)   # :87-106


def test_router_matches_oracle_bit_for_bit(ctx, devbuf):
    g = np.random.Generator(np.random.Philox(key=5))
    lg = g.standard_normal((512, 8), dtype=np.float32)
    lg[::7, 3] = lg[::7, 5]          # exact ties
    bias = (g.standard_normal(8) * 0.5).astype(np.float32)
    for b in (None, bias):
        ids, w, *_ = route_gpu(ctx, devbuf, lg, 8, 2, bias=b)
        for t in range(512):
            oi, ow = oracle.Route(lg[t], 8, 2, b)
            assert list(ids[t]) == list(oi)
            assert np.array_equal(w[t].view(np.uint32), ow.view(np.uint32))


def moe_oracle(gu_raw, dn_raw, hidden, ffn, x_bf, ids, wts, tokens):
    out = np.zeros((len(tokens), hidden), np.float64)
    for i, t in enumerate(tokens):
        xt = bf16_to_f32(x_bf[t:t + 1])
        for s in range(ids.shape[1]):
            e = int(ids[t, s])
            gu = oracle.MatVec(12, gu_raw[e], 2 * ffn, hidden, xt)[0].astype(np.float64)
            h = gu[:ffn] / (1 + np.exp(-gu[:ffn])) * gu[ffn:]
            hb = bf16_to_f32(to_bf16_bits(h.astype(np.float32)))      # the kernel feeds the down matmul bf16
            y = oracle.MatVec(12, dn_raw[e], hidden, ffn, hb.reshape(1, -1))[0]
            out[i] += float(wts[t, s]) * y.astype(np.float64)
    return out


def run_moe(ctx, devbuf, experts, hidden, ffn, tokens, topk, seed, check_tokens):
    gu_raw = [synth.weights(12, 2 * ffn, hidden, seed + e) for e in range(experts)]
    dn_raw = [synth.weights(12, hidden, ffn, seed + 100 + e) for e in range(experts)]
    gu = [ctx.store_upload(12, 2 * ffn, hidden, r) for r in gu_raw]
    dn = [ctx.store_upload(12, hidden, ffn, r) for r in dn_raw]
    x_bf = to_bf16_bits(synth.activations(tokens, hidden, seed + 200))
    lg = synth.activations(tokens, experts, seed + 201)
    ids, wts, ids_d, wts_d = route_gpu(ctx, devbuf, lg, experts, topk)
    xd = devbuf(x_bf)
    od = devbuf(np.full((tokens, hidden), np.nan, np.float32))
    ctx.moe_grouped(gu, dn, xd.ptr, tokens, hidden, ids_d.ptr, wts_d.ptr, topk, od.ptr, hidden)
    ctx.sync()
    rc, status = ctx.last_status()
    assert rc == 0 and status == 0
    out = od.get((tokens, hidden))
    assert np.isfinite(out).all()
    want = moe_oracle(gu_raw, dn_raw, hidden, ffn, x_bf, ids, wts, check_tokens)
    err = float(np.linalg.norm(out[check_tokens].astype(np.float64) - want) / np.linalg.norm(want))
    for w in gu + dn:
        w.free()
    return err


def test_small_moe(ctx, devbuf):
    assert run_moe(ctx, devbuf, 4, 512, 1024, 70, 2, 11, list(range(70))) <= TOL


def test_mixtral_shape_sampled_tokens(ctx, devbuf):
    """Config 5: 8 experts, top-2, hidden 4096, ffn 14336, 512 tokens; three tokens checked
    against the oracle (all 512 go through the kernels)."""
    assert run_moe(ctx, devbuf, 8, 4096, 14336, 512, 2, 500, [0, 255, 511]) <= TOL


def test_gather_folded_into_the_matmul_gives_the_same_bits(ctx, devbuf, monkeypatch):
    """The gate|up matmul fetching the tokens' rows by the dispatch list itself (the default) against the
    separate gather pass (the reference's order of work, nvidia/x/cudamoe/moe.go:72-96): same rows in the same
    order, so equal bits; also with the list lengths kept on the device, and with a padded row pitch."""
    experts, hidden, ffn, tokens, topk, seed, ldx = 4, 512, 768, 333, 2, 77, 520
    gu_raw = [synth.weights(12, 2 * ffn, hidden, seed + e) for e in range(experts)]
    dn_raw = [synth.weights(12, hidden, ffn, seed + 100 + e) for e in range(experts)]
    gu = [ctx.store_upload(12, 2 * ffn, hidden, r) for r in gu_raw]
    dn = [ctx.store_upload(12, hidden, ffn, r) for r in dn_raw]
    x_bf = np.zeros((tokens, ldx), np.uint16)
    x_bf[:, :hidden] = to_bf16_bits(synth.activations(tokens, hidden, seed + 200))
    lg = synth.activations(tokens, experts, seed + 201)
    ids, wts, ids_d, wts_d = route_gpu(ctx, devbuf, lg, experts, topk)
    xd = devbuf(x_bf)
    outs = {}
    for fold in ("1", "0"):
        for nosync in ("0", "1"):
            monkeypatch.setenv("QM_MOE_FOLD", fold)
            monkeypatch.setenv("QM_MOE_NOSYNC", nosync)
            od = devbuf(np.full((tokens, hidden), np.nan, np.float32))
            ctx.moe_grouped(gu, dn, xd.ptr, tokens, ldx, ids_d.ptr, wts_d.ptr, topk, od.ptr, hidden)
            ctx.sync()
            rc, status = ctx.last_status()
            assert rc == 0 and status == 0
            outs[fold, nosync] = od.get((tokens, hidden))
    base = outs["0", "0"]
    assert np.isfinite(base).all()
    for k, v in outs.items():
        assert np.array_equal(v.view(np.uint32), base.view(np.uint32)), k
    want = moe_oracle(gu_raw, dn_raw, hidden, ffn, x_bf[:, :hidden], ids, wts, [0, 100, 332])
    got = outs["1", "0"][[0, 100, 332]].astype(np.float64)
    assert float(np.linalg.norm(got - want) / np.linalg.norm(want)) <= TOL
    for w in gu + dn:
        w.free()


def test_grouped_down_matmul_with_split_k(ctx, devbuf, monkeypatch):
    """Few experts leave SMs idle in the grouped down launch, so it splits K over CTAs (shares through
    the scratch, added in a fixed order): same bits run after run, the oracle's values within the layer's
    tolerance, and the unsplit launch's values to rounding."""
    experts, hidden, ffn, tokens, topk, seed = 2, 512, 2048, 150, 2, 91
    gu_raw = [synth.weights(12, 2 * ffn, hidden, seed + e) for e in range(experts)]
    dn_raw = [synth.weights(12, hidden, ffn, seed + 100 + e) for e in range(experts)]
    gu = [ctx.store_upload(12, 2 * ffn, hidden, r) for r in gu_raw]
    dn = [ctx.store_upload(12, hidden, ffn, r) for r in dn_raw]
    x_bf = to_bf16_bits(synth.activations(tokens, hidden, seed + 200))
    lg = synth.activations(tokens, experts, seed + 201)
    ids, wts, ids_d, wts_d = route_gpu(ctx, devbuf, lg, experts, topk)
    xd = devbuf(x_bf)
    outs = []
    for split in ("1", "1", "0"):
        monkeypatch.setenv("QM_GEMM_GROUPED_SPLITK", split)
        od = devbuf(np.full((tokens, hidden), np.nan, np.float32))
        ctx.moe_grouped(gu, dn, xd.ptr, tokens, hidden, ids_d.ptr, wts_d.ptr, topk, od.ptr, hidden)
        ctx.sync()
        rc, status = ctx.last_status()
        assert rc == 0 and status == 0
        outs.append(od.get((tokens, hidden)))
    assert np.isfinite(outs[0]).all()
    assert np.array_equal(outs[0].view(np.uint32), outs[1].view(np.uint32))
    ref = outs[2].astype(np.float64)
    assert float(np.linalg.norm(outs[0] - ref) / np.linalg.norm(ref)) <= 1e-5   # another order of float32 additions
    want = moe_oracle(gu_raw, dn_raw, hidden, ffn, x_bf, ids, wts, [0, 77, 149])
    got = outs[0][[0, 77, 149]].astype(np.float64)
    assert float(np.linalg.norm(got - want) / np.linalg.norm(want)) <= TOL
    for w in gu + dn:
        w.free()


def test_layer_stages_match_oracle(ctx):
    """lib_b200.moe.MoELayer on one GPU (route -> dispatch -> experts -> combine through the
    staged entry points) against the oracle chain."""
    import torch
    from lib_b200 import moe
    experts, topk, hidden, ffn, tokens, seed = 4, 2, 512, 768, 45, 3
    layer = moe.MoELayer(ctx, experts, topk, hidden, ffn, seed)
    dev = torch.device("cuda:0")
    x_bits = to_bf16_bits(synth.activations(tokens, hidden, 900))
    lg = synth.activations(tokens, experts, 901)
    x = torch.from_numpy(x_bits.view(np.int16)).to(dev).view(torch.bfloat16)
    out = layer.forward(x, torch.from_numpy(lg).to(dev))
    ids, wts = layer.route(torch.from_numpy(lg).to(dev))
    torch.cuda.synchronize()
    rc, status = ctx.last_status()
    assert rc == 0 and status == 0
    raws = [moe.expert_weights(hidden, ffn, e, seed) for e in range(experts)]
    want = moe_oracle([r[0] for r in raws], [r[1] for r in raws], hidden, ffn, x_bits, ids.cpu().numpy(),
                      wts.cpu().numpy(), list(range(tokens)))
    got = out.cpu().numpy().astype(np.float64)
    assert float(np.linalg.norm(got - want) / np.linalg.norm(want)) <= TOL
    layer.close()


def test_router_and_dispatch_with_256_experts(ctx, devbuf):
    """The reference's MoEConfig names 256 routed experts with 8 active: routing bit for bit against the oracle,
    the per-expert lists against a stable sort of the pairs."""
    g = np.random.Generator(np.random.Philox(key=11))
    tokens, experts, topk, hidden = 96, 256, 8, 64
    lg = g.standard_normal((tokens, experts), dtype=np.float32)
    lg[::5, 200] = lg[::5, 17]          # exact ties across the 64-expert words of the taken mask
    bias = (g.standard_normal(experts) * 0.3).astype(np.float32)
    ids, w, ids_d, wts_d = route_gpu(ctx, devbuf, lg, experts, topk, bias=bias)
    for t in range(tokens):
        oi, ow = oracle.Route(lg[t], experts, topk, bias)
        assert list(ids[t]) == list(oi)
        assert np.array_equal(w[t].view(np.uint32), ow.view(np.uint32))
    x = to_bf16_bits(synth.activations(tokens, hidden, 3))
    rows_d, pos_d = devbuf(nbytes=tokens * topk * hidden * 2), devbuf(nbytes=tokens * topk * 4)
    counts = ctx.moe_dispatch(ids_d.ptr, tokens, topk, experts, devbuf(x).ptr, hidden, hidden, rows_d.ptr, pos_d.ptr)
    flat = ids.reshape(-1)
    assert counts == [int((flat == e).sum()) for e in range(experts)]
    order = np.argsort(flat, kind="stable")               # pairs grouped by expert, token order inside a group
    rows = rows_d.get((tokens * topk, hidden), np.uint16)
    assert np.array_equal(rows, x[order // topk])
    pos = pos_d.get((tokens * topk,), np.int32)
    assert np.array_equal(pos[order], np.arange(tokens * topk))
