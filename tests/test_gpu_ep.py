"""Expert-parallel MoE against the same layer on one GPU: the exchange through peer memory behind the C ABI
(qm_ep_*) with 1, 2 and 4 ranks emulated on one GPU (one process, one stream, each phase for all ranks before
the next, so that no kernel ever waits for a later launch) and as two processes on two GPUs; and the NCCL
all-to-all form of lib_b200.moe on two GPUs. The two-GPU tests are skipped on a one-GPU box."""
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


PEER_CHILD = r"""
import os, sys
import numpy as np
import torch
import torch.distributed as dist
sys.path.insert(0, os.environ["QM_ROOT"])
import lib_b200
from lib_b200 import moe, synth
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("gloo", rank=rank, world_size=world)
ctx = lib_b200.Context(rank)
experts, topk, hidden, ffn, seed = 4, 2, 512, 768, 21
dev = torch.device("cuda", rank)
tokens = 40 + 24 * rank
x = torch.from_numpy(synth.activations(tokens, hidden, 700 + rank)).to(dev).to(torch.bfloat16)
lg = torch.from_numpy(synth.activations(tokens, experts, 800 + rank)).to(dev)
ep = moe.PeerExpertParallelLayer(ctx, experts, topk, hidden, ffn, seed, 64, rank, world)
for _ in range(3):                      # several steps: arenas and flags are reused, the epochs grow
    out = ep.forward(x, lg)
torch.cuda.synchronize()
full = moe.MoELayer(ctx, experts, topk, hidden, ffn, seed)     # all experts on this GPU
want = full.forward(x, lg)
torch.cuda.synchronize()
rc, status = ctx.last_status()
err = float((out.double() - want.double()).norm() / want.double().norm())
ok = rc == 0 and status == 0 and bool(torch.isfinite(out).all()) and err <= 1e-6
print("rank", rank, "err", err, "status", rc, status, "ok", ok, flush=True)
dist.barrier()
sys.stdout.flush()
os._exit(0 if ok else 1)
"""


def test_two_gpu_peer_expert_parallel_matches_single_gpu():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), QM_ROOT=ROOT)
        procs.append(subprocess.Popen([sys.executable, "-c", PEER_CHILD], env=env, stdout=subprocess.PIPE,
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


@pytest.mark.parametrize("world", [1, 2, 4])
def test_peer_exchange_with_emulated_ranks(ctx, devbuf, world):
    import numpy as np
    from lib_b200 import _capi, synth
    experts, topk, hidden, ffn, seed = 8, 2, 512, 768, 33
    per = experts // world
    raws = [(synth.weights(12, 2 * ffn, hidden, seed + 2 * e), synth.weights(12, hidden, ffn, seed + 2 * e + 1))
            for e in range(experts)]
    gu = [ctx.store_upload(12, 2 * ffn, hidden, r[0]) for r in raws]
    dn = [ctx.store_upload(12, hidden, ffn, r[1]) for r in raws]
    eps = [_capi.ExpertParallel(ctx, gu[r * per:(r + 1) * per], dn[r * per:(r + 1) * per], experts, topk, 96, r, world)
           for r in range(world)]
    if world > 1:
        bases = [e.arena()[0] for e in eps]
        for e in eps:
            e.set_peer_pointers(bases)

    def bf16(x):
        u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
        return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)

    for step in range(2):                                      # the second step reuses arenas, flags, lists
        toks = [0 if (r == 1 and step == 1) else 30 + 17 * r + step for r in range(world)]   # uneven, once empty
        bufs = []
        for r in range(world):
            t = max(toks[r], 1)
            x = devbuf(bf16(synth.activations(t, hidden, 100 * step + r)))
            lg = devbuf(synth.activations(t, experts, 200 * step + r))
            ids, wts = devbuf(nbytes=t * topk * 4), devbuf(nbytes=t * topk * 4)
            out, want = devbuf(np.full((t, hidden), np.nan, np.float32)), devbuf(np.full((t, hidden), np.nan, np.float32))
            ctx.moe_route(lg.ptr, t, experts, experts, topk, ids.ptr, wts.ptr)
            if step == 1 and r == 0:                           # one pair that names no expert
                bad = ids.get((t, topk), np.int32)
                bad[3, 1] = experts + 5
                ctx.h2d(ids.ptr, bad)
            bufs.append((x, ids, wts, out, want, t))
        for r, e in enumerate(eps):
            x, ids, wts, out, want, t = bufs[r]
            e.begin(x.ptr, toks[r], hidden, ids.ptr, wts.ptr, out.ptr, hidden)
        for e in eps:
            e.run()
        for e in eps:
            e.end()
        assert ctx.last_status() == (0, 0)
        for r in range(world):
            x, ids, wts, out, want, t = bufs[r]
            if toks[r] == 0:
                continue
            idv = ids.get((t, topk), np.int32)
            if (idv >= experts).any():                         # the reference layer on one GPU: that pair weighs nothing
                w0 = wts.get((t, topk))
                w0[idv >= experts] = 0
                idv[idv >= experts] = 0
                ctx.h2d(ids.ptr, idv)
                ctx.h2d(wts.ptr, w0)
            ctx.moe_grouped(gu, dn, x.ptr, t, hidden, ids.ptr, wts.ptr, topk, want.ptr, hidden)
            got, ref = out.get((t, hidden)), want.get((t, hidden))
            assert np.isfinite(got).all()
            assert np.linalg.norm(got - ref) <= 1e-6 * np.linalg.norm(ref), (world, step, r)
    for e in eps:
        e.close()
    for w in gu + dn:
        w.free()
