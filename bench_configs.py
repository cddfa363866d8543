"""Single-op measurements for the benchmark configurations that are not the full decode step:

  1  Q8_0 GEMV 4096x4096, batch 1
  2  Q4_0 decode GEMV at Llama-3-8B FFN shapes (14336x4096 and 4096x14336), batch 1 and 8
  3  Q4_K prefill matmul 4096x4096, M in {64, 256, 2048}, bf16 activations (tcgen05)
  5  Mixtral-8x7B-shaped MoE layer: 8 experts, top-2, 512 tokens, Q4_K, bf16 activations
     (under `python -m torch.distributed.run --nproc-per-node N ...` the experts are sharded
     over the N GPUs and the tokens exchanged by NCCL all-to-all)
  7  Q4_K decode GEMV at the Llama-3-8B matrix shapes, one matrix at a time, batch 1 and 8
  8  decode-time MoE: Mixtral-8x7B-shaped layer (8 Q4_K experts, top-2) at 1, 2 and 4 tokens through
     qm_moe_decode (one launch for all (token, slot) matvecs); Q2_K / IQ2_XXS matvecs over selected
     experts with Q8_1 activations; the Q8_1 producers

Run as `python bench_configs.py --config 3 [--m 2048] [--copies 4] [--iters 10]`; bench.py runs
short versions of the same cases for its `other_configs` block.
Each case prints one JSON line.  Every case cycles through enough copies of the weights to
exceed the 126 MB L2 (or `--copies`), records the launches in a CUDA graph, and is timed with
CUDA events on the launching stream after three warm-up replays.  Rooflines are against the
measured peaks in MEASURED_PEAKS.json beside this file (fallback 6650 GB/s, 1590 TFLOP/s)."""
import argparse
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

import lib_b200  # noqa: E402
from lib_b200 import _capi, synth  # noqa: E402

Q4_0, Q8_0, Q4_K = 2, 8, 12
PDL = _capi.FLAG_PDL


def peaks():
    try:
        p = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured"
    except Exception:
        return 6650.0, 1590.0, "fallback"


def timed_graph(ctx, enqueue, iters):
    """Mean milliseconds of one `enqueue()` pass, replayed from a CUDA graph."""
    s = torch.cuda.Stream()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(s):
        ctx.set_stream(s.cuda_stream)
        enqueue()
        s.synchronize()
        with torch.cuda.graph(g, stream=s):
            ctx.set_stream(torch.cuda.current_stream().cuda_stream)
            enqueue()
        ctx.set_stream(s.cuda_stream)
        for _ in range(3):
            g.replay()
        s.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(s)
        for _ in range(iters):
            g.replay()
        e1.record(s)
        s.synchronize()
    return e0.elapsed_time(e1) / iters


def timed_eager(ctx, enqueue, iters):
    """Mean milliseconds of one `enqueue()` pass issued call by call (for paths that read
    back from the device in the middle and so cannot be captured)."""
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        ctx.set_stream(s.cuda_stream)
        for _ in range(3):
            enqueue()
        s.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(s)
        for _ in range(iters):
            enqueue()
        e1.record(s)
        s.synchronize()
    return e0.elapsed_time(e1) / iters


def gemv_case(ctx, fmt, rows, cols, m, copies, iters, flags):
    dev = torch.device("cuda", torch.cuda.current_device())
    nbytes = synth.gguf_bytes(fmt, rows, cols)
    copies = copies or max(2, int(400e6 // nbytes))
    raw = synth.weights(fmt, rows, cols, 1)
    ws = [ctx.store_upload(fmt, rows, cols, raw) for _ in range(copies)]
    x = torch.randn(m, cols, device=dev)
    y = torch.empty(m, rows, device=dev)

    def enqueue():
        for w in ws:
            ctx.matvec(w, x.data_ptr(), m, cols, y.data_ptr(), rows, flags)

    ms = timed_graph(ctx, enqueue, iters) / copies
    for w in ws:
        w.free()
    hbm, _, which = peaks()
    gbs = nbytes / (ms * 1e-3) / 1e9
    return {"op": "gemv", "format": {2: "Q4_0", 8: "Q8_0", 12: "Q4_K"}[fmt], "rows": rows, "cols": cols, "m": m,
            "us": round(ms * 1e3, 2), "weight_GBps": round(gbs, 1), "frac_hbm": round(gbs / hbm, 3),
            "peak": which, "copies": copies, "pdl": bool(flags & _capi.FLAG_PDL)}


def gemm_case(ctx, m, copies, iters, n=4096, k=4096):
    dev = torch.device("cuda", torch.cuda.current_device())
    copies = copies or 16
    raw = synth.weights(Q4_K, n, k, 1)
    ws = [ctx.store_upload(Q4_K, n, k, raw) for _ in range(copies)]
    a = torch.randn(m, k, device=dev).to(torch.bfloat16)
    c = torch.empty(m, n, device=dev)

    def enqueue():
        for w in ws:
            ctx.matmul_bf16(w, a.data_ptr(), m, k, c.data_ptr(), n)

    ms = timed_graph(ctx, enqueue, iters) / copies
    for w in ws:
        w.free()
    hbm, tf, which = peaks()
    tflops = 2.0 * m * n * k / (ms * 1e-3) / 1e12
    gbs = (synth.gguf_bytes(Q4_K, n, k) + 2.0 * m * k + 4.0 * m * n) / (ms * 1e-3) / 1e9
    out = {"op": "matmul_bf16", "format": "Q4_K", "n": n, "k": k, "m": m, "us": round(ms * 1e3, 2),
           "TFLOPs": round(tflops, 1), "frac_tensor": round(tflops / tf, 3), "GBps": round(gbs, 1),
           "frac_hbm": round(gbs / hbm, 3), "peak": which, "copies": copies}
    # below the ridge (peak flops / peak bytes per second) a case is bound by HBM, above it by the tensor cores
    out["bound"] = "hbm" if 2.0 * m * n * k / (synth.gguf_bytes(Q4_K, n, k) + 2.0 * m * k + 4.0 * m * n) < tf * 1e3 / hbm else "tensor"
    return out


def moe_case(ctx, tokens, iters, hidden=4096, ffn=14336, experts=8, topk=2):
    dev = torch.device("cuda", torch.cuda.current_device())
    gu = [ctx.store_upload(Q4_K, 2 * ffn, hidden, synth.weights(Q4_K, 2 * ffn, hidden, 10 + e)) for e in range(experts)]
    dn = [ctx.store_upload(Q4_K, hidden, ffn, synth.weights(Q4_K, hidden, ffn, 30 + e)) for e in range(experts)]
    x = torch.randn(tokens, hidden, device=dev).to(torch.bfloat16)
    logits = torch.randn(tokens, experts, device=dev)
    ids = torch.empty(tokens, topk, dtype=torch.int32, device=dev)
    wts = torch.empty(tokens, topk, device=dev)
    out = torch.empty(tokens, hidden, device=dev)

    def enqueue():
        ctx.moe_route(logits.data_ptr(), tokens, experts, experts, topk, ids.data_ptr(), wts.data_ptr())
        ctx.moe_grouped(gu, dn, x.data_ptr(), tokens, hidden, ids.data_ptr(), wts.data_ptr(), topk, out.data_ptr(), hidden)

    ms = timed_eager(ctx, enqueue, iters)
    for w in gu + dn:
        w.free()
    _, tf, which = peaks()
    flops = 2.0 * tokens * topk * 3 * hidden * ffn
    tflops = flops / (ms * 1e-3) / 1e12
    return {"op": "moe_layer", "format": "Q4_K", "experts": experts, "topk": topk, "tokens": tokens,
            "hidden": hidden, "ffn": ffn, "ms": round(ms, 3), "tokens_per_s": round(tokens / (ms * 1e-3)),
            "TFLOPs": round(tflops, 1), "frac_tensor": round(tflops / tf, 3), "peak": which,
            "weight_bytes": sum(synth.gguf_bytes(Q4_K, 3 * ffn, hidden) for _ in range(experts))}


def moe_decode_case(ctx, tokens, iters, hidden=4096, ffn=14336, experts=8, topk=2):
    """Config 8: a decode step of an MoE layer. Bytes per step = the experts the pairs stream."""
    dev = torch.device("cuda", torch.cuda.current_device())
    gu = [ctx.store_upload(Q4_K, 2 * ffn, hidden, synth.weights(Q4_K, 2 * ffn, hidden, 10 + e)) for e in range(experts)]
    dn = [ctx.store_upload(Q4_K, hidden, ffn, synth.weights(Q4_K, hidden, ffn, 30 + e)) for e in range(experts)]
    md = ctx.moe_decode_create(gu, dn, topk, tokens)
    x = torch.randn(tokens, hidden, device=dev)
    out = torch.empty(tokens, hidden, device=dev)
    wts = torch.full((tokens, topk), 1.0 / topk, device=dev)
    # eight id sets that walk over all experts, so that consecutive steps do not find their experts in L2
    sets = [torch.tensor([[(2 * (t + r) + s * 3 + r) % experts for s in range(topk)] for t in range(tokens)],
                         dtype=torch.int32, device=dev) for r in range(8)]
    ids = torch.empty(tokens, topk, dtype=torch.int32, device=dev)

    def enqueue():
        for r in range(8):
            ids.copy_(sets[r])
            ctx.moe_decode_run(md, x.data_ptr(), tokens, hidden, ids.data_ptr(), wts.data_ptr(), out.data_ptr(), hidden)

    ms = timed_eager_torch(ctx, enqueue, iters) / 8
    rc, status = ctx.last_status()
    ctx.moe_decode_destroy(md)
    for w in gu + dn:
        w.free()
    hbm, _, which = peaks()
    nbytes = tokens * topk * synth.gguf_bytes(Q4_K, 3 * ffn, hidden)
    gbs = nbytes / (ms * 1e-3) / 1e9
    return {"op": "moe_decode", "format": "Q4_K", "experts": experts, "topk": topk, "tokens": tokens, "hidden": hidden,
            "ffn": ffn, "us": round(ms * 1e3, 1), "weight_GBps": round(gbs, 1), "frac_hbm": round(gbs / hbm, 3),
            "peak": which, "launches_per_step": 2, "status": [rc, status]}


def timed_eager_torch(ctx, enqueue, iters):
    """timed_eager for passes that also issue torch copies: everything on one torch stream."""
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        ctx.set_stream(s.cuda_stream)
        for _ in range(3):
            enqueue()
        s.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(s)
        for _ in range(iters):
            enqueue()
        e1.record(s)
        s.synchronize()
    ctx.set_stream(0)
    return e0.elapsed_time(e1) / iters


def selected_case(ctx, fmt, iters, rows=2048, cols=4096, experts=64, slots=6):
    """Config 8: *_selected_matvec_q8_1 at a DeepSeek-style routed-expert shape: `slots` of `experts` small matrices."""
    dev = torch.device("cuda", torch.cuda.current_device())
    one = synth.weights(fmt, rows, cols, 3)
    raw = np.concatenate([np.frombuffer(one, dtype=np.uint8)] * experts)
    w = ctx.store_upload(fmt, experts * rows, cols, raw)
    xf = synth.activations(1, cols, 9)
    xq_host = np.zeros((cols // 32) * 36, dtype=np.uint8)
    x = torch.from_numpy(xf).to(dev)
    xq = torch.from_numpy(xq_host).to(dev)
    ctx.rmsnorm_q8_1(x.data_ptr(), cols, 0, 1, cols, 1e-6, xq.data_ptr())
    y = torch.empty(slots, rows, device=dev)
    sets = [torch.tensor([(r * slots + s * 5) % experts for s in range(slots)], dtype=torch.int32, device=dev) for r in range(16)]

    def enqueue():
        for r in range(16):
            ctx.matvec_selected(w, experts, sets[r].data_ptr(), slots, xq.data_ptr(), 0, y.data_ptr(), _capi.FLAG_X_Q8_1)

    ms = timed_graph(ctx, enqueue, iters) / 16
    w.free()
    hbm, _, which = peaks()
    nbytes = slots * synth.gguf_bytes(fmt, rows, cols)
    gbs = nbytes / (ms * 1e-3) / 1e9
    return {"op": "selected_matvec_q8_1", "format": {10: "Q2_K", 16: "IQ2_XXS"}[fmt], "experts": experts, "slots": slots,
            "rows": rows, "cols": cols, "us": round(ms * 1e3, 2), "weight_GBps": round(gbs, 1),
            "frac_hbm": round(gbs / hbm, 3), "peak": which}


def q8_1_producer_case(ctx, rows, cols, iters):
    dev = torch.device("cuda", torch.cuda.current_device())
    x = torch.randn(rows, cols, device=dev)
    wt = torch.rand(cols, device=dev) + 0.5
    out = torch.empty(rows * cols // 32 * 36, dtype=torch.uint8, device=dev)

    def enqueue():
        for _ in range(16):
            ctx.rmsnorm_q8_1(x.data_ptr(), cols, wt.data_ptr(), rows, cols, 1e-6, out.data_ptr())

    ms = timed_graph(ctx, enqueue, iters) / 16
    return {"op": "rmsnorm_q8_1", "rows": rows, "cols": cols, "us": round(ms * 1e3, 2),
            "note": "latency-bound: %d bytes in, %d out" % (rows * cols * 4, rows * cols // 32 * 36)}


def moe_ep_case(tokens_total, iters, hidden=4096, ffn=14336, experts=8, topk=2, exchange="peer"):
    """Config 5 across the ranks of a torchrun launch: experts sharded by index, the batch of
    `tokens_total` tokens split evenly, rows exchanged through peer memory behind the C ABI
    (qm_ep_*, the default) or by NCCL all-to-all (lib_b200.moe, --exchange nccl)."""
    import torch.distributed as dist
    from lib_b200 import moe
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    ctx = lib_b200.Context(local)
    tokens = tokens_total // world
    if exchange == "peer":
        layer = moe.PeerExpertParallelLayer(ctx, experts, topk, hidden, ffn, 5, tokens, rank, world)
    else:
        layer = moe.MoELayer(ctx, experts, topk, hidden, ffn, 5, rank, world)
    x = torch.from_numpy(synth.activations(tokens, hidden, 40 + rank)).to(dev).to(torch.bfloat16)
    lg = torch.from_numpy(synth.activations(tokens, experts, 60 + rank)).to(dev)
    # a stream of its own: the library takes stream handle 0 to mean its private stream, which the events
    # of torch's default stream would not see
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        for _ in range(3):
            layer.forward(x, lg)
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(st)
        for _ in range(iters):
            layer.forward(x, lg)
        e1.record(st)
        torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    rc, status = ctx.last_status()
    line = {"op": "moe_layer_expert_parallel", "format": "Q4_K", "n_gpus": world, "experts": experts, "topk": topk,
            "tokens": tokens * world, "hidden": hidden, "ffn": ffn, "ms": round(ms, 3),
            "tokens_per_s": round(tokens * world / (ms * 1e-3)), "status": [rc, status],
            "TFLOPs": round(2.0 * tokens * world * topk * 3 * hidden * ffn / (ms * 1e-3) / 1e12, 1),
            "exchange": "peer stores behind the C ABI (qm_ep_moe: bf16 rows out, fp32 rows back, flags)" if exchange == "peer"
            else "NCCL all_to_all_single (bf16 rows out, fp32 rows back)", "scaling": "strong"}
    if rank == 0:
        print(json.dumps(line), flush=True)
    dist.barrier()
    torch.cuda.synchronize()
    sys.stdout.flush()
    os._exit(0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", type=int, required=True, choices=(1, 2, 3, 5, 7, 8))
    ap.add_argument("--m", type=int, default=0, help="only this batch size")
    ap.add_argument("--copies", type=int, default=0, help="weight copies cycled through (default: > L2)")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--tokens", type=int, default=512)
    ap.add_argument("--no-pdl", action="store_true")
    ap.add_argument("--exchange", choices=("peer", "nccl"), default="peer", help="config 5 on several GPUs")
    a = ap.parse_args()
    if a.config == 5 and int(os.environ.get("WORLD_SIZE", "1")) > 1:
        moe_ep_case(a.tokens, max(3, a.iters // 4), exchange=a.exchange)
        return
    ctx = lib_b200.Context(0)
    torch.cuda.init()
    flags = 0 if a.no_pdl else _capi.FLAG_PDL
    out = []
    if a.config == 1:
        out.append(gemv_case(ctx, Q8_0, 4096, 4096, a.m or 1, a.copies, a.iters, flags))
    elif a.config == 2:
        for rows, cols in ((14336, 4096), (4096, 14336)):
            for m in ((a.m,) if a.m else (1, 8)):
                out.append(gemv_case(ctx, Q4_0, rows, cols, m, a.copies, a.iters, flags))
    elif a.config == 7:
        for rows, cols in ((6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336)):
            for m in ((a.m,) if a.m else (1, 8)):
                out.append(gemv_case(ctx, Q4_K, rows, cols, m, a.copies, a.iters, flags))
    elif a.config == 3:
        for m in ((a.m,) if a.m else (64, 256, 2048)):
            out.append(gemm_case(ctx, m, a.copies, a.iters))
    elif a.config == 8:
        for t in ((a.m,) if a.m else (1, 2, 4)):
            out.append(moe_decode_case(ctx, t, max(3, a.iters // 4)))
        for fmt in (10, 16):
            out.append(selected_case(ctx, fmt, a.iters))
        for rows in (1, 8):
            out.append(q8_1_producer_case(ctx, rows, 4096, a.iters))
    else:
        out.append(moe_case(ctx, a.tokens, max(3, a.iters // 4)))
    for line in out:
        print(json.dumps(line), flush=True)
    ctx.close()


if __name__ == "__main__":
    main()
