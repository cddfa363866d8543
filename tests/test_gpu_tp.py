"""Tensor-parallel decode stack on two GPUs (one persistent launch per GPU, results stored into the
peer's buffers over NVLink and polled there), in both shardings — every matrix by rows, and the paired
form (q|k|v and gate|up by rows, o and down by K) — against the same stack on one GPU. Needs two visible GPUs; skipped otherwise. The ranks run as child processes and
exchange the 64-byte IPC handles over a gloo group."""
import os
import socket
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r'''
import os, sys
import numpy as np
import torch
import torch.distributed as dist
sys.path.insert(0, os.environ["QM_ROOT"])
import lib_b200
from lib_b200 import decode, synth
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("gloo", rank=rank, world_size=world)
ctx = lib_b200.Context(rank)
layers, hidden, kv, ffn, fmt, seed = 3, 512, 128, 768, 12, 77
paired = os.environ.get("QM_TEST_PAIRED") == "1"
if paired:
    hidden, ffn = 512, 1024                    # K slices of o and down must be whole 256-column units
tp = decode.PeerTensorParallelDecode(ctx, layers, hidden, kv, ffn, fmt, seed, rank, world, m_max=4 if paired else 8, paired=paired)
one = decode.SingleGpuDecode(ctx, layers, hidden, kv, ffn, fmt, seed)
ok = True
for m in ((1, 3, 4) if paired else (1, 3, 8)):
    x = synth.activations(m, hidden, 300 + m)
    for rep in range(3):                       # several steps: the arena halves alternate, the epochs grow
        h = np.full((m, hidden), np.nan, np.float32)
        kvb = np.full((layers, m, 2 * kv), np.nan, np.float32)
        tp.step_host(x, h, kvb)
    want, want_kv = one.stack.step_host(x, want_kv=True)
    rc, status = ctx.last_status()
    err = float(np.linalg.norm(h.astype(np.float64) - want) / np.linalg.norm(want))
    # every rank holds all k|v rows: each GPU's slice was stored into every arena
    kv_ok = bool(np.isfinite(kvb).all()) and float(np.linalg.norm(kvb - want_kv) / np.linalg.norm(want_kv)) <= 1e-4
    good = rc == 0 and status == 0 and bool(np.isfinite(h).all()) and err <= 1e-4 and kv_ok
    print("rank", rank, "m", m, "err", err, "status", rc, status, "kv", kv_ok, "ok", good, flush=True)
    ok = ok and good
dist.barrier()
sys.stdout.flush()
os._exit(0 if ok else 1)
'''


@pytest.mark.parametrize("paired", [False, True], ids=["rows", "paired"])
def test_two_gpu_tensor_parallel_matches_single_gpu(paired):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), QM_ROOT=ROOT,
                   QM_TEST_PAIRED="1" if paired else "0")
        procs.append(subprocess.Popen([sys.executable, "-c", CHILD], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            o, _ = p.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            p.kill()
            o, _ = p.communicate()
            o += "\n[timed out]"
        outs.append(o)
    assert all(p.returncode == 0 for p in procs), "\n".join(outs)
