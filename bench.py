#!/usr/bin/env python
"""Benchmark of the quantized decode hot path.

Workload: one decode step over a Llama-3-8B-shaped stack of Q4_K weights — 32 layers of q|k|v
(6144x4096), o (4096x4096), gate|up (28672x4096) and down (4096x14336) matvecs with float32
activations — on seeded synthetic tensors (no model file is read). `value` is decode tokens per
second with the input activation already on the device; `e2e` is the same step through the
host-buffer entry point (`qm_stack_step_host`), host->device copy of the input and
device->host copy of the outputs inside the timed region.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch M] [--impl reference]

N > 1 (launched under torchrun, one rank per GPU) slices every matrix by output rows over the
ranks (tensor parallel); each rank stores its slices of every matvec into all peers' activation
buffers over NVLink inside one persistent launch per step. NCCL carries set-up and the timing
barriers only.

Every line carries `parity`: outside the timed region the last layer's down-projection output is
compared with the CPU oracle fed the captured input of that matvec (normwise relative error), and
with N > 1 rank 0's outputs are compared bit for bit with every other rank's.

At N = 1 the line also carries `other_configs`: short runs of the other benchmark configurations
(Q8_0 and Q4_0 decode GEMV, single Q4_K GEMVs, the Q4_K prefill matmul, the MoE layer), each
with its roofline fraction.

`--impl reference` times the CPU restatement of the reference's dequantize-and-dot path
(oracle/) on the host cores instead, on a bounded sample; it loads nothing of the CUDA library.
"""
import argparse
import importlib.util
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
SEED = 20240229

# DRAM bytes of the fused decode kernel at batch 1 per layer, from one ncu capture of the kernel on
# a 2-layer stack (dram__bytes_read.sum + dram__bytes_write.sum; traffic grows with the layers).
NCU_DRAM_BYTES_PER_LAYER_BATCH1 = (245.563392e6 + 5.005568e6) / 2


def load_synth():
    """lib_b200/synth.py by path: it is plain numpy, and importing the package would load the CUDA library."""
    spec = importlib.util.spec_from_file_location("qm_synth", os.path.join(ROOT, "lib_b200", "synth.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def layer_bytes(synth):
    return sum(synth.gguf_bytes(FMT, r, c) for r, c in SHAPES)


def step_algorithmic_bytes(synth, m, layers=LAYERS):
    """GGUF weight bytes plus float32 activation reads and writes of one step."""
    act = sum(4 * m * (c + r) for r, c in SHAPES)
    return layers * (layer_bytes(synth) + act)


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


# ---- CPU legs (the oracle; the only use of oracle/ besides the parity check) ----------------------
def cpu_layer_inputs(synth, m):
    raws = [synth.weights(FMT, r, c, SEED + i) for i, (r, c) in enumerate(SHAPES)]
    xs = [synth.activations(m, c, SEED + 50 + i) for i, (r, c) in enumerate(SHAPES)]
    return raws, xs


def cpu_reference_layer(oracle, raws, xs, threads, seconds):
    """Seconds per layer (its four matvecs) of the oracle's dequantize-and-dot in float32, rows split
    over `threads` threads; repeated for about `seconds`."""
    reps, t0 = 0, time.perf_counter()
    while True:
        for (r, c), raw, x in zip(SHAPES, raws, xs):
            oracle.MatVec(FMT, raw, r, c, x, threads=threads)
        reps += 1
        dt = time.perf_counter() - t0
        if dt >= seconds or reps >= 50:
            break
    return dt / reps


def cpu_baseline_block(synth, oracle, m, seconds):
    """Both CPU legs: all host cores (row-parallel), and one thread in the reference's own shape —
    dequantize the whole matrix into a float32 buffer, then the dot products (a single goroutine
    calling quant.Dequantize* and looping, GOMAXPROCS-independent)."""
    cores = os.cpu_count() or 1
    raws, xs = cpu_layer_inputs(synth, m)
    cpu_reference_layer(oracle, raws, xs, cores, 0.0)
    t_layer = cpu_reference_layer(oracle, raws, xs, cores, seconds)
    t0 = time.perf_counter()
    for (r, c), raw, x in zip(SHAPES, raws, xs):
        oracle.MatVecFaithful(FMT, raw, r, c, x)
    t_single = time.perf_counter() - t0
    lb = layer_bytes(synth)
    return {
        "value": m / (t_layer * LAYERS), "unit": "tok/s", "cores": cores, "threads": cores, "kind": "port",
        "sample": "1 of %d layers (4 matvecs, %.1f MB of Q4_K) repeated ~%.0f s, time x%d" % (LAYERS, lb / 1e6, seconds, LAYERS),
        "single_thread_faithful": {"value": m / (t_single * LAYERS), "unit": "tok/s", "threads": 1,
                                   "sample": "1 of %d layers once (whole-matrix dequantize to float32, then dot), time x%d" % (LAYERS, LAYERS)},
        "compiler": "gcc -O2 -ffp-contract=off -fno-fast-math (oracle/Makefile)",
        "gomaxprocs": "n/a (Go toolchain absent; C restatement of lm/quant dequantize + dot)",
    }


def workload_config(synth, batch, gpus):
    return {"workload": "Q4_K decode step, Llama-3-8B-shaped stack: 32 layers x {qkv 6144x4096, o 4096x4096, "
                        "gate_up 28672x4096, down 4096x14336}, fp32 activations",
            "batch": batch, "weights_gguf_bytes": LAYERS * layer_bytes(synth), "seed": SEED,
            "parallelism": "tp%d" % gpus if gpus > 1 else "single",
            "l2": "weights (3.9 GB per step) exceed the 126 MB L2; no flush needed"}


def run_reference(args):
    """The reference arm: the CPU restatement of the reference's own path on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    synth = load_synth()
    from oracle import oracle
    cores = os.cpu_count() or 1
    raws, xs = cpu_layer_inputs(synth, args.batch)
    cpu_reference_layer(oracle, raws, xs, cores, 0.0)
    budget = max(1.0, min(20.0, 120.0 / max(args.steps, 1)))
    per_layer = [cpu_reference_layer(oracle, raws, xs, cores, budget / 4) for _ in range(args.steps)]
    step_s = float(np.median(per_layer)) * LAYERS
    value = args.batch / step_s
    sample = "1 of %d layers per step (4 matvecs, %.1f MB of Q4_K), time x%d" % (LAYERS, layer_bytes(synth) / 1e6, LAYERS)
    line = {
        "impl": "reference", "metric": "decode_tokens_per_s", "value": value, "unit": "tok/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_s * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(synth, args.batch, args.gpus),
        "cpu_baseline": {"value": value, "unit": "tok/s", "cores": cores, "threads": cores, "kind": "port", "sample": sample,
                         "compiler": "gcc -O2 -ffp-contract=off -fno-fast-math (oracle/Makefile)",
                         "gomaxprocs": "n/a (Go toolchain absent; C restatement of lm/quant dequantize + dot)"},
        "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "where": "host cores",
    }
    print(json.dumps(line))


def parity_check(ctx, runner, synth, m, layers, x_host, dist, rank, world):
    """Outside the timed region: one more step through the host entry point, then
    (a) the last layer's down-projection output against the oracle fed that matvec's captured input,
    (b) with several ranks, rank 0's h and k|v against every other rank's, bit for bit."""
    import torch
    from lib_b200 import decode
    from oracle import oracle
    h = np.empty((m, HIDDEN), np.float32)
    kv = np.empty((layers, m, 2 * KV), np.float32)
    runner.step_host(x_host, h, kv)
    rc, status = ctx.last_status()
    out = {"status": int(status), "rc": int(rc)}
    ptrs = runner.stack.buffers()
    gu = np.empty((m, 2 * FFN), np.float32)
    ctx.d2h(gu, ptrs[3])
    if world > 1 and getattr(runner, "paired", False):
        # every rank holds only its own gate and up slices (its down part needs no others): put them together
        f = FFN // world
        own = np.zeros_like(gu)
        own[:, rank * f:(rank + 1) * f] = gu[:, rank * f:(rank + 1) * f]
        own[:, FFN + rank * f:FFN + (rank + 1) * f] = gu[:, FFN + rank * f:FFN + (rank + 1) * f]
        t = torch.from_numpy(own).cuda()
        dist.all_reduce(t)
        gu = t.cpu().numpy()
    down_raw = decode.layer_tensors(FMT, HIDDEN, KV, FFN, SEED, layers - 1)[6][3]
    want = oracle.MatVec(FMT, down_raw, HIDDEN, FFN, oracle.RMSNorm(gu[:, :FFN] + gu[:, FFN:]))
    out["nre"] = float(np.linalg.norm(h.astype(np.float64) - want) / max(np.linalg.norm(want), 1e-30))
    out["checked"] = "last layer's down matvec (4096x14336) vs oracle on the captured gate|up output"
    out["finite"] = bool(np.isfinite(h).all() and np.isfinite(kv).all())
    if world > 1:
        mine = torch.from_numpy(np.concatenate([h.reshape(-1), kv.reshape(-1)]).view(np.int32)).cuda()
        ref = mine.clone()
        dist.broadcast(ref, src=0)
        same = torch.tensor([1 if torch.equal(mine, ref) else 0], device="cuda")
        dist.all_reduce(same, op=dist.ReduceOp.MIN)
        out["ranks_agree"] = bool(int(same.item()))
        st = torch.tensor([int(status)], device="cuda")
        dist.all_reduce(st, op=dist.ReduceOp.MAX)
        out["status"] = int(st.item())
    out["green"] = bool(out["nre"] <= 1e-3 and out["finite"] and out["status"] == 0 and out.get("ranks_agree", True))
    return out


def other_configs(ctx):
    """Short runs of the benchmark's other configurations (cold L2: each case cycles through more
    weight copies than the L2 holds), one dict per case with its roofline fraction."""
    import bench_configs as bc
    out = []
    flags = bc.PDL
    for label, fn in [
        ("config 1: Q8_0 GEMV 4096x4096, batch 1", lambda: bc.gemv_case(ctx, bc.Q8_0, 4096, 4096, 1, 0, 10, flags)),
        ("config 2: Q4_0 GEMV 14336x4096, batch 1", lambda: bc.gemv_case(ctx, bc.Q4_0, 14336, 4096, 1, 0, 10, flags)),
        ("config 2: Q4_0 GEMV 14336x4096, batch 8", lambda: bc.gemv_case(ctx, bc.Q4_0, 14336, 4096, 8, 0, 10, flags)),
        ("config 2: Q4_0 GEMV 4096x14336, batch 1", lambda: bc.gemv_case(ctx, bc.Q4_0, 4096, 14336, 1, 0, 10, flags)),
        ("config 2: Q4_0 GEMV 4096x14336, batch 8", lambda: bc.gemv_case(ctx, bc.Q4_0, 4096, 14336, 8, 0, 10, flags)),
        ("Q4_K GEMV 28672x4096, batch 1", lambda: bc.gemv_case(ctx, bc.Q4_K, 28672, 4096, 1, 0, 10, flags)),
        ("Q4_K GEMV 4096x14336, batch 1", lambda: bc.gemv_case(ctx, bc.Q4_K, 4096, 14336, 1, 0, 10, flags)),
        ("config 3: Q4_K matmul 4096x4096, M=64", lambda: bc.gemm_case(ctx, 64, 0, 10)),
        ("config 3: Q4_K matmul 4096x4096, M=256", lambda: bc.gemm_case(ctx, 256, 0, 10)),
        ("config 3: Q4_K matmul 4096x4096, M=2048", lambda: bc.gemm_case(ctx, 2048, 0, 10)),
        ("config 5: MoE layer 8 experts top-2, 512 tokens", lambda: bc.moe_case(ctx, 512, 5)),
        ("decode-time MoE (qm_moe_decode): 8 Q4_K experts top-2, 1 token", lambda: bc.moe_decode_case(ctx, 1, 5)),
        ("decode-time MoE (qm_moe_decode): 8 Q4_K experts top-2, 4 tokens", lambda: bc.moe_decode_case(ctx, 4, 5)),
        ("selected-expert matvec, Q2_K, Q8_1 activations, 6 of 64 experts of 2048x4096", lambda: bc.selected_case(ctx, 10, 10)),
        ("selected-expert matvec, IQ2_XXS, Q8_1 activations, 6 of 64 experts of 2048x4096", lambda: bc.selected_case(ctx, 16, 10)),
        ("RMSNorm -> Q8_1, 8 rows of 4096", lambda: bc.q8_1_producer_case(ctx, 8, 4096, 10)),
    ]:
        try:
            r = fn()
            r["case"] = label
            out.append(r)
        except Exception as exc:   # noqa: BLE001 — a failing side case must not lose the headline line
            out.append({"case": label, "error": repr(exc)})
    return out


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
    ap.add_argument("--no-other-configs", action="store_true", help="skip the short runs of the other configurations")
    ap.add_argument("--tp", choices=("auto", "paired", "rows"), default="auto",
                    help="sharding on several GPUs: paired (q|k|v, gate|up by rows; o, down by K; up to batch 4), every matrix "
                         "by rows, or auto = paired where the batch allows (measured 0.96 / 0.85 / 0.87 ms against 0.98 / 0.92 / "
                         "0.89 by rows on 2 / 4 / 8 GPUs)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
        return

    import torch
    import lib_b200
    from lib_b200 import decode, synth

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
        runner = decode.SingleGpuDecode(ctx, layers, HIDDEN, KV, FFN, FMT, SEED)
        tp_mode = None
    else:
        paired = args.tp in ("paired", "auto") and m <= 4
        runner = decode.PeerTensorParallelDecode(ctx, layers, HIDDEN, KV, FFN, FMT, SEED, rank, world, m_max=4 if paired else 8,
                                                 barrier=False, paired=paired)
        tp_mode = ("paired: q|k|v and gate|up sliced by rows, o and down by the K columns of the rank's own slices; partial "
                   "outputs stored into all peers' arenas over NVLink, polled there and added in rank order by the consumer "
                   "(two exchanges per layer); one persistent launch per GPU and step" if paired else
                   "every matrix sliced by rows; slices stored into all peers' arenas over NVLink and polled "
                   "there (four exchanges per layer); one persistent launch per GPU and step")

    x_host = torch.from_numpy(synth.activations(m, HIDDEN, SEED + 999)).pin_memory()
    x_dev = x_host.to("cuda", non_blocking=False)
    h_dev = torch.empty(m, HIDDEN, device="cuda")
    h_host = torch.empty(m, HIDDEN).pin_memory()
    kv_host = torch.empty(layers, m, 2 * KV).pin_memory()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    barrier()   # every rank has mapped every arena before any rank stores into one
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
        if not args.no_other_batch and not (getattr(runner, "paired", False) and m2 > 4):   # the paired form holds up to four rows
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

    parity = parity_check(ctx, runner, synth, m, layers, x_host.numpy(), dist, rank, world)
    if rank != 0:
        finish(dist)
        return

    pk, pk_kind = peaks()
    step_bytes = step_algorithmic_bytes(synth, m, layers)
    gpu_bytes = step_bytes / world            # every matrix is sliced (by rows or by K): each GPU streams 1/N of the weights
    achieved = gpu_bytes / (ms * 1e-3) / 1e9  # per GPU
    kernel = ("qm_fused_q4k_dd_c4d4" if m == 1 else "qm_fused_q4k_dd_c4d3" if m == 2 else "qm_fused_q4k_dd_c2d3" if m == 3
              else "qm_fused_q4k_nt1_img" if m == 4 else "qm_fused_q4k_dd_n2d3")
    if world > 1:
        kernel = kernel + "_tp" if m <= 3 else ("qm_fused_q4k_dd_c2d3_tp" if (m == 4 and getattr(runner, "paired", False))
                                                else "qm_fused_q4k_nt1_tp" if m == 4 else "qm_fused_q4k_nt2_tp")
    line = {
        "metric": "decode_tokens_per_s", "value": m / (ms * 1e-3), "unit": "tok/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(synth, m, world),
        "e2e": {"value": m / (ms_e2e * 1e-3), "unit": "tok/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": int(x_host.numel() * 4),
                "d2h_bytes_per_step": int(h_host.numel() * 4 + kv_host.numel() * 4)},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "parity": parity,
        "roofline": {
            "bound": "hbm", "kernel": kernel,
            "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
            "frac": achieved / pk["hbm_gbs"], "frac_of_8TBs_datasheet": achieved / 8000.0,
            "peak_kind": pk_kind + " (copy bandwidth, MEASURED_PEAKS.json)",
            "per_gpu": True,
            "per_launch": {"launches_per_step": max(1, round(launches / args.steps)), "matvecs_per_step": 4 * layers,
                           "bytes_per_step_per_gpu": gpu_bytes, "us_per_step": ms * 1e3},
            "traffic": None,
            "note": "achieved = (GGUF weight bytes + fp32 activation bytes of the step) / GPUs / CUDA-event time: "
                    "what one GPU streams; the step is %d matvecs run by this one kernel (one persistent launch "
                    "per GPU and step)" % (4 * layers),
        },
    }
    if tp_mode:
        line["config"]["exchange"] = tp_mode
    if ms_other:
        line["other_batch"] = {"batch": m2, "value": m2 / (ms_other * 1e-3), "unit": "tok/s", "ms_per_step": ms_other,
                               "roofline_frac": step_algorithmic_bytes(synth, m2, layers) / world / (ms_other * 1e-3) / 1e9 / pk["hbm_gbs"]}
    if world == 1 and m == 1:
        line["roofline"]["traffic"] = NCU_DRAM_BYTES_PER_LAYER_BATCH1 * layers
        line["roofline"]["traffic_note"] = ("dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of this "
                                            "kernel on a 2-layer stack, per layer x %d layers" % layers)
    if world == 1 and not args.no_other_configs:
        runner.close()
        line["other_configs"] = other_configs(ctx)
    if world == 1 and not args.no_cpu_baseline:
        from oracle import oracle
        line["cpu_baseline"] = cpu_baseline_block(synth, oracle, m, 10.0)
    print(json.dumps(line), flush=True)
    finish(dist)


def finish(dist):
    """Multi-rank runs leave through os._exit after a last barrier: tearing down CUDA contexts that
    still map peers' memory together with the process group can block at interpreter exit."""
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
