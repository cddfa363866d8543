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
