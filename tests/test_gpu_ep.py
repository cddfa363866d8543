"""Expert-parallel MoE on two GPUs (NCCL all-to-all token dispatch) against the same layer on
one GPU. Needs two visible GPUs; skipped otherwise. The ranks run as child processes."""
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
from lib_b200 import moe, synth
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
ctx = lib_b200.Context(rank)
experts, topk, hidden, ffn, seed = 4, 2, 512, 768, 21
dev = torch.device("cuda", rank)

def inputs(r):
    tokens = 40 + 24 * r
    x = torch.from_numpy(synth.activations(tokens, hidden, 700 + r)).to(dev).to(torch.bfloat16)
    lg = torch.from_numpy(synth.activations(tokens, experts, 800 + r)).to(dev)
    return x, lg

ep = moe.MoELayer(ctx, experts, topk, hidden, ffn, seed, rank, world)
x, lg = inputs(rank)
for _ in range(2):                      # twice: buffers and scratch are reused
    out = ep.forward(x, lg)
torch.cuda.synchronize()
full = moe.MoELayer(ctx, experts, topk, hidden, ffn, seed)     # all experts on this GPU
want = full.forward(x, lg)
torch.cuda.synchronize()
rc, status = ctx.last_status()
err = float((out.double() - want.double()).norm() / want.double().norm())
ok = rc == 0 and status == 0 and bool(torch.isfinite(out).all()) and err <= 1e-4
print("rank", rank, "err", err, "ok", ok, flush=True)
dist.barrier()
torch.cuda.synchronize()
sys.stdout.flush()
os._exit(0 if ok else 1)
'''


def test_two_gpu_expert_parallel_matches_single_gpu():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                   QM_ROOT=ROOT, NCCL_NVLS_ENABLE="0")
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
