"""CPU test (gloo, world_size 2) of the expert-parallel host logic in lib_b200.moe: the split
sizes, the two all-to-all exchanges and the regrouping on the receiver, with the three device
stages replaced by numpy stand-ins and experts that are simple known functions. The result must
equal the direct evaluation of sum_s w[t][s] * f_e(x_t)."""
import os
import socket
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_ep_plan_split_sizes():
    sys.path.insert(0, ROOT)
    from lib_b200.moe import ep_plan
    counts = np.array([[3, 0, 2, 1], [1, 4, 0, 2]])       # [src][expert], 2 experts per rank
    send, recv, ids = ep_plan(counts, 0, 2)
    assert send == [3, 3] and recv == [3, 5]
    assert list(ids) == [0, 0, 0, 0, 1, 1, 1, 1]           # src 0: 3x e0; src 1: 1x e0, 4x e1
    send, recv, ids = ep_plan(counts, 1, 2)
    assert send == [5, 2] and recv == [3, 2]
    assert list(ids) == [0, 0, 1, 1, 1]                    # src 0: 2x e2, 1x e3; src 1: 2x e3


class NumpyStages:
    """Stand-ins for the three device stages, same contracts, on CPU tensors."""

    def __init__(self, first_expert):
        self.first = first_expert

    def dispatch(self, ids, x, experts):
        import torch
        flat = ids.numpy().reshape(-1)
        topk = ids.shape[1]
        order = np.argsort(flat, kind="stable")
        pos = np.empty_like(order)
        pos[order] = np.arange(len(order))
        rows = x[torch.from_numpy(order // topk)]
        return rows, torch.from_numpy(pos.astype(np.int32)), [int((flat == e).sum()) for e in range(experts)]

    def run_experts(self, rows, counts):
        import torch
        out = torch.empty(rows.shape, dtype=torch.float32)
        off = 0
        for e, n in enumerate(counts):
            g = self.first + e
            out[off:off + n] = rows[off:off + n].float() * (g + 1) + g
            off += n
        return out

    def combine(self, y, pos, weights):
        import torch
        tokens, topk = weights.shape
        out = torch.zeros((tokens, y.shape[1]), dtype=torch.float32)
        p = pos.long().reshape(tokens, topk)
        for s in range(topk):
            out += weights[:, s:s + 1] * y[p[:, s]]
        return out


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    from lib_b200.moe import expert_parallel_forward
    dist.init_process_group("gloo", rank=rank, world_size=world, init_method="tcp://127.0.0.1:%d" % port)
    try:
        experts, topk, hidden = 8, 2, 16
        g = np.random.Generator(np.random.Philox(key=100 + rank))
        tokens = 37 + 5 * rank                                       # ragged: the ranks hold different counts
        x = torch.from_numpy(g.standard_normal((tokens, hidden), dtype=np.float32))
        ids = np.stack([g.permutation(experts)[:topk] for _ in range(tokens)]).astype(np.int32)
        if rank == 1:
            ids[:, 0] = 7                                            # skew: expert 7 gets every token of rank 1
            ids[:, 1] = np.where(ids[:, 1] == 7, 0, ids[:, 1])
        w = torch.from_numpy(g.random((tokens, topk), dtype=np.float32))
        per = experts // world
        out = expert_parallel_forward(NumpyStages(rank * per), x, torch.from_numpy(ids), w, experts, rank, world)
        want = torch.zeros_like(x)
        for s in range(topk):
            e = torch.from_numpy(ids[:, s].astype(np.float32)).reshape(-1, 1)
            want += w[:, s:s + 1] * (x * (e + 1) + e)
        q.put((rank, bool(torch.allclose(out, want, rtol=1e-6, atol=1e-6))))
    finally:
        dist.destroy_process_group()


def test_expert_parallel_exchange_two_ranks():
    import torch.multiprocessing as mp
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(res) == [(0, True), (1, True)]
