#!/usr/bin/env python
"""Benchmark of the quantized decode hot path.

Workload (N=1): one decode step over a Llama-3-8B-shaped stack of Q4_K weights
— 32 layers of q|k|v (6144x4096), o (4096x4096), gate|up (28672x4096) and down
(4096x14336) matvecs with float32 activations — on seeded synthetic tensors
(no model file is read). `value` is decode tokens per second with the input
activation already on the device; `e2e` is the same step through the
host-buffer entry point (`qm_stack_step_host`), host->device copy of the input
and device->host copy of the outputs inside the timed region.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch M] [--impl reference]

N > 1 (launched under torchrun) shards every matrix by output rows over the
ranks (tensor parallel) and all-gathers the output slices with NCCL.
`--impl reference` times the CPU restatement of the reference's dequantize-and-
dot path (oracle/) on the host cores instead, on a bounded sample.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LAYERS, HIDDEN, KV, FFN, FMT = 32, 4096, 1024, 14336, 12
SHAPES = [(HIDDEN + 2 * KV, HIDDEN), (HIDDEN, HIDDEN), (2 * FFN, HIDDEN), (HIDDEN, FFN)]
NAMES = ["qkv", "o", "gate_up", "down"]
SEED = 20240229


# DRAM bytes per layer of the fused decode kernel at batch 1, from the ncu capture summarised in
# profiles/qm_fused_q4k_nt1_two_layer_stack.md (245.46 MB read + 4.11 MB written for 2 layers).
NCU_DRAM_BYTES_PER_LAYER_BATCH1 = (245.459712e6 + 4.109056e6) / 2


def layer_bytes():
    from lib_b200 import synth
    return sum(synth.gguf_bytes(FMT, r, c) for r, c in SHAPES)


def step_algorithmic_bytes(m, layers=LAYERS):
    """GGUF weight bytes plus float32 activation reads and writes of one step."""
    act = sum(4 * m * (c + r) for r, c in SHAPES)
    return layers * (layer_bytes() + act)


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return json.load(open(p)), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([f.strip() for f in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        self.proc.terminate()
        self.thread.join(timeout=2)
        sm = [float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def cpu_reference_step(m, threads, seconds):
    """Times the oracle's dequantize-and-dot on one layer's four matrices (of the 32)."""
    from lib_b200 import synth
    from oracle import oracle
    raws = [synth.weights(FMT, r, c, SEED + i) for i, (r, c) in enumerate(SHAPES)]
    xs = [synth.activations(m, c, SEED + 50 + i) for i, (r, c) in enumerate(SHAPES)]
    reps, t0 = 0, time.perf_counter()
    while True:
        for (r, c), raw, x in zip(SHAPES, raws, xs):
            oracle.MatVec(FMT, raw, r, c, x, threads=threads)
        reps += 1
        dt = time.perf_counter() - t0
        if dt >= seconds or reps >= 50:
            break
    return dt / reps  # seconds per layer


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    warm = cpu_reference_step(args.batch, cores, 0.0)
    del warm
    per_layer = []
    budget = max(1.0, min(20.0, 120.0 / max(args.steps, 1)))
    for _ in range(args.steps):
        per_layer.append(cpu_reference_step(args.batch, cores, budget / 4))
    t_layer = float(np.median(per_layer))
    step_s = t_layer * LAYERS
    value = args.batch / step_s
    sample = "1 of %d layers per step (4 matvecs, %.1f MB of Q4_K), time x%d" % (LAYERS, layer_bytes() / 1e6, LAYERS)
    line = {
        "impl": "reference", "metric": "decode_tokens_per_s", "value": value, "unit": "tok/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_s * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.batch, args.gpus, "cpu"),
        "cpu_baseline": {"value": value, "unit": "tok/s", "cores": cores, "kind": "port", "sample": sample,
                         "note": "C restatement of lm/quant dequantize + dot; the Go toolchain is absent"},
        "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def workload_config(batch, gpus, where):
    return {"workload": "Q4_K decode step, Llama-3-8B-shaped stack: 32 layers x {qkv 6144x4096, o 4096x4096, "
                        "gate_up 28672x4096, down 4096x14336}, fp32 activations",
            "batch": batch, "weights_gguf_bytes": LAYERS * layer_bytes(), "seed": SEED,
            "parallelism": "tp%d" % gpus if gpus > 1 else "single", "where": where,
            "l2": "weights (3.9 GB per step) exceed the 126 MB L2; no flush needed"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--layers", type=int, default=LAYERS, help=argparse.SUPPRESS)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-other-batch", action="store_true", help="skip the short run at the other batch size (8 or 1)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
        return

    import torch
    import lib_b200
    from lib_b200 import _capi, synth

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if world != args.gpus and rank == 0:
        print("warning: --gpus %d but WORLD_SIZE %d" % (args.gpus, world), file=sys.stderr)

    ctx = lib_b200.Context(local)
    stream = torch.cuda.Stream()
    ctx.set_stream(stream.cuda_stream)
    m, layers = args.batch, args.layers

    if world == 1:
        from lib_b200 import decode
        runner = decode.SingleGpuDecode(ctx, layers, HIDDEN, KV, FFN, FMT, SEED)
    else:
        from lib_b200 import decode
        runner = None
        if os.environ.get("QM_TP_MODE", "peer") != "nccl":
            # one persistent launch per GPU with peer-memory stores; if any rank cannot map its
            # peers' memory, all ranks agree to fall back to the NCCL all-gather arm
            try:
                runner = decode.PeerTensorParallelDecode(ctx, layers, HIDDEN, KV, FFN, FMT, SEED, rank, world,
                                                         barrier=False)
            except Exception as exc:   # noqa: BLE001
                print("rank %d: peer tensor parallelism unavailable (%s)" % (rank, exc), file=sys.stderr, flush=True)
            flag = torch.tensor([1 if runner is not None else 0], device="cuda")
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            if int(flag.item()) == 0:
                runner = None
        tp_mode = "peer stores + cross-GPU barrier in one launch per GPU"
        if runner is None:   # the plain NCCL all-gather arm
            tp_mode = "matvec launches + NCCL all-gather (CUDA graph)"
            runner = decode.TensorParallelDecode(ctx, layers, HIDDEN, KV, FFN, FMT, SEED, rank, world, stream)

    x_host = torch.from_numpy(synth.activations(m, HIDDEN, SEED + 999)).pin_memory()
    x_dev = x_host.to("cuda", non_blocking=False)
    h_dev = torch.empty(m, HIDDEN, device="cuda")
    h_host = torch.empty(m, HIDDEN).pin_memory()
    kv_host = torch.empty(layers, m, 2 * KV).pin_memory()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident steps ---------------------------------------------------------
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)   # nvidia-smi needs a moment before its first sample
    with torch.cuda.stream(stream):
        for _ in range(args.warmup):
            runner.step_device(x_dev, m, h_dev)
        stream.synchronize()
        barrier()
        launches0 = ctx.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps):
            runner.step_device(x_dev, m, h_dev)
        e1.record(stream)
        stream.synchronize()
        barrier()
        ms = e0.elapsed_time(e1) / args.steps
        launches = ctx.launch_count() - launches0

        # ---- end to end through host buffers ---------------------------------------------
        for _ in range(3):
            runner.step_host(x_host.numpy(), h_host.numpy(), kv_host.numpy())
        barrier()
        e0.record(stream)
        for _ in range(args.steps):
            runner.step_host(x_host.numpy(), h_host.numpy(), kv_host.numpy())
        e1.record(stream)
        stream.synchronize()
        barrier()
        ms_e2e = e0.elapsed_time(e1) / args.steps

        # ---- the other batch size the workload is quoted at (reported beside the metric) ----
        m2 = 8 if m == 1 else 1
        ms_other = None
        if not args.no_other_batch:
            x2_dev = torch.from_numpy(synth.activations(m2, HIDDEN, SEED + 998)).to("cuda")
            h2_dev = torch.empty(m2, HIDDEN, device="cuda")
            n2 = max(3, min(args.steps, 50))
            for _ in range(3):
                runner.step_device(x2_dev, m2, h2_dev)
            stream.synchronize()
            barrier()
            e0.record(stream)
            for _ in range(n2):
                runner.step_device(x2_dev, m2, h2_dev)
            e1.record(stream)
            stream.synchronize()
            barrier()
            ms_other = e0.elapsed_time(e1) / n2
    clocks = sampler.stop() if rank == 0 else None

    t = torch.tensor([ms, ms_e2e, ms_other or 0.0], device="cuda", dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_e2e, ms_other = float(t[0]), float(t[1]), float(t[2])
    if rank != 0:
        finish(dist)
        return

    pk, pk_kind = peaks()
    step_bytes = step_algorithmic_bytes(m, layers)
    achieved = step_bytes / (ms * 1e-3) / 1e9
    n_launch = 4 * layers
    line = {
        "metric": "decode_tokens_per_s", "value": m / (ms * 1e-3), "unit": "tok/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": dict(workload_config(m, world, "B200"), **({"exchange": tp_mode} if world > 1 else {})),
        "e2e": {"value": m / (ms_e2e * 1e-3), "unit": "tok/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": int(x_host.numel() * 4),
                "d2h_bytes_per_step": int(h_host.numel() * 4 + kv_host.numel() * 4)},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "roofline": {
            "bound": "hbm", "kernel": "qm_fused_q4k_nt1" if m <= 4 else "qm_fused_q4k_nt2",
            "achieved": achieved * world if world > 1 else achieved, "peak": pk["hbm_gbs"] * world, "unit": "GB/s",
            "frac": achieved / pk["hbm_gbs"], "frac_of_8TBs_datasheet": achieved / 8000.0, "peak_kind": pk_kind + " (copy bandwidth, MEASURED_PEAKS.json)",
            "per_launch": {"launches_per_step": max(1, round(launches / args.steps)), "matvecs_per_step": n_launch,
                           "bytes_per_step": step_bytes / world, "us_per_step": ms * 1e3},
            "traffic": None,
            "note": "achieved = GGUF weight bytes + fp32 activation bytes of the step / CUDA-event time; the "
                    "step is %d matvecs run by this one kernel (one persistent launch per step on 1 GPU)" % n_launch,
        },
    }
    if ms_other:
        line["other_batch"] = {"batch": m2, "value": m2 / (ms_other * 1e-3), "unit": "tok/s", "ms_per_step": ms_other,
                               "roofline_frac": step_algorithmic_bytes(m2, layers) / (ms_other * 1e-3) / 1e9 / pk["hbm_gbs"] / world}
    if world == 1 and not args.no_cpu_baseline:
        cores = os.cpu_count() or 1
        cpu_reference_step(m, cores, 0.0)
        t_layer = cpu_reference_step(m, cores, 12.0)
        line["cpu_baseline"] = {
            "value": m / (t_layer * LAYERS), "unit": "tok/s", "cores": cores, "kind": "port",
            "sample": "1 of %d layers (4 matvecs, %.1f MB of Q4_K) repeated ~12 s, time x%d" % (
                LAYERS, layer_bytes() / 1e6, LAYERS)}
    if world == 1 and m == 1:
        line["roofline"]["traffic"] = NCU_DRAM_BYTES_PER_LAYER_BATCH1 * layers
        line["roofline"]["traffic_note"] = ("dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of this "
                                            "kernel on a 2-layer stack, per layer x %d layers" % layers)
    print(json.dumps(line), flush=True)
    finish(dist)


def finish(dist):
    """Multi-rank runs leave through os._exit after a last barrier: tearing down CUDA graphs
    that hold NCCL kernels together with the process group can block at interpreter exit."""
    if dist is None:
        return
    import torch
    torch.cuda.synchronize()
    dist.barrier()
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
