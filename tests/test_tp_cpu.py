"""CPU test (gloo, world_size 2) of the tensor-parallel host logic: every rank cuts its row
shard out of the row-stacked GGUF tensors with the same helpers the GPU runner uses
(lib_b200.decode.shard_range / shard_slices), multiplies it (here with the oracle — no GPU in
this test), and an all-gather of the output slices must reproduce the unsharded product."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, fmt, hidden, kv, ffn, m, q):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    from lib_b200 import decode, synth
    from oracle import oracle
    dist.init_process_group("gloo", rank=rank, world_size=world, init_method="tcp://127.0.0.1:%d" % port)
    try:
        tensors = decode.layer_tensors(fmt, hidden, kv, ffn, seed=77, layer=0)
        x = synth.activations(m, hidden, 5)
        ok = True
        for rows, cols, parts in decode.stacked(tensors):
            xin = x if cols == hidden else synth.activations(m, cols, 6)
            full_bytes = np.concatenate([d for _, _, d in parts])
            want = oracle.MatVec(fmt, full_bytes, rows, cols, xin)
            lo, hi = decode.shard_range(rows, rank, world)
            shard = np.concatenate([d for _, _, d in decode.shard_slices(fmt, cols, parts, lo, hi)])
            mine = torch.from_numpy(oracle.MatVec(fmt, shard, hi - lo, cols, xin))
            gathered = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(gathered, mine)
            got = torch.cat(gathered, dim=1).numpy()
            ok = ok and np.array_equal(got, want)
        q.put((rank, ok))
    finally:
        dist.destroy_process_group()


def test_row_shards_gather_to_the_full_product():
    import torch.multiprocessing as mp
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, 12, 512, 128, 768, 2, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(res) == [(0, True), (1, True)]


def _paired_worker(rank, world, port, fmt, hidden, kv, ffn, m, q):
    """The paired sharding (q|k|v, gate|up by rows; o, down by K over the rank's own slices) on the CPU: a rank
    multiplies its column shard by its own slice of the input, the partial vectors of all ranks are added in
    rank order (all_gather + ordered sum, as the consumers do), and that must be the unsharded product."""
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    from lib_b200 import decode, synth
    from oracle import oracle
    dist.init_process_group("gloo", rank=rank, world_size=world, init_method="tcp://127.0.0.1:%d" % port)
    try:
        t = {n: (r, c, b) for n, r, c, b in decode.layer_tensors(fmt, hidden, kv, ffn, seed=78, layer=0)}
        ok = True
        # o and down: column shards times the rank's slice of x
        for name, cols in (("o", hidden), ("down", ffn)):
            rows, _, data = t[name]
            x = synth.activations(m, cols, 9)
            want = oracle.MatVec(fmt, data, rows, cols, x).astype(np.float64)
            lo, hi = decode.shard_range(cols, rank, world)
            shard = decode.column_shard(fmt, rows, cols, data, lo, hi)
            part = torch.from_numpy(oracle.MatVec(fmt, shard, rows, hi - lo, np.ascontiguousarray(x[:, lo:hi])))
            parts = [torch.empty_like(part) for _ in range(world)]
            dist.all_gather(parts, part)
            got = np.zeros_like(want)
            for p in parts:                       # rank order
                got += p.numpy().astype(np.float64)
            ok = ok and np.linalg.norm(got - want) <= 1e-6 * np.linalg.norm(want)
        # q|k|v: the rank's q slice and k|v slice, stacked; gathered per range they give the full rows
        x = synth.activations(m, hidden, 10)
        for ranges in ([("q", hidden), ("kv", 2 * kv)], [("gate", ffn), ("up", ffn)]):
            tensors = []
            for name, rows in ranges:
                data = np.concatenate([np.asarray(t["k"][2]), np.asarray(t["v"][2])]) if name == "kv" else np.asarray(t[name][2])
                tensors.append((rows, data))
            be, bb = synth.BLOCK[fmt]
            row_bytes = hidden // be * bb
            mine, off = [], 0
            for rows, data in tensors:
                lo, hi = decode.shard_range(rows, rank, world)
                mine.append(data[lo * row_bytes:hi * row_bytes])
            local = oracle.MatVec(fmt, np.concatenate(mine), sum(r for r, _ in tensors) // world, hidden, x)
            loc = torch.from_numpy(local)
            allp = [torch.empty_like(loc) for _ in range(world)]
            dist.all_gather(allp, loc)
            col = 0
            for rows, data in tensors:
                n = rows // world
                got = np.concatenate([p.numpy()[:, col:col + n] for p in allp], axis=1)
                ok = ok and np.array_equal(got, oracle.MatVec(fmt, data, rows, hidden, x))
                col += n
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def test_paired_shards_add_up_to_the_full_product():
    import torch.multiprocessing as mp
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_paired_worker, args=(r, 2, port, 12, 512, 128, 1024, 2, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(res) == [(0, True), (1, True)]
