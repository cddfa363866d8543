"""Runners of the decode step used by the benchmark and the tests: a single-GPU
runner over `qm_stack`, the tensor-parallel runner over peer memory (row-sharded or
paired), and an older runner that all-gathers row slices with NCCL (kept as a comparison).

Weights are seeded synthetic tensors (lib_b200.synth); q, k, v and gate, up are
generated as separate tensors and written into one store entry by rows, the way
a loader would place a GGUF file's tensors.
"""
import os
import sys
import time

import numpy as np

from . import _capi, synth


def _trace(msg):
    if os.environ.get("QM_TRACE"):
        print("[rank %s %.1fs] %s" % (os.environ.get("RANK", "0"), time.perf_counter(), msg), file=sys.stderr, flush=True)


def layer_tensors(fmt, hidden, kv, ffn, seed, layer):
    """[(name, rows, cols, gguf bytes)] of one layer, in store order."""
    spec = [("q", hidden, hidden), ("k", kv, hidden), ("v", kv, hidden), ("o", hidden, hidden),
            ("gate", ffn, hidden), ("up", ffn, hidden), ("down", hidden, ffn)]
    return [(n, r, c, synth.weights(fmt, r, c, seed + 16 * layer + i)) for i, (n, r, c) in enumerate(spec)]


def stacked(tensors):
    """Groups q|k|v and gate|up: [(rows, cols, [(row_offset, nrows, bytes)])] for the four matrices."""
    t = {n: (r, c, b) for n, r, c, b in tensors}
    out = []
    for names in (("q", "k", "v"), ("o",), ("gate", "up"), ("down",)):
        parts, off = [], 0
        for n in names:
            r, c, b = t[n]
            parts.append((off, r, b))
            off += r
        out.append((off, t[names[0]][1], parts))
    return out


def shard_slices(fmt, cols, parts, row_lo, row_hi):
    """The pieces of the row-stacked tensors `parts` that fall in rows [row_lo, row_hi):
    yields (row offset inside the shard, row count, GGUF bytes of those rows)."""
    be, bb = synth.BLOCK[fmt]
    row_bytes = cols // be * bb
    for off, nrows, data in parts:
        lo, hi = max(off, row_lo), min(off + nrows, row_hi)
        if lo < hi:
            yield lo - row_lo, hi - lo, data[(lo - off) * row_bytes:(hi - off) * row_bytes]


def shard_range(rows, rank, world):
    """Rows [lo, hi) of a matrix that tensor-parallel rank `rank` of `world` holds."""
    return rank * rows // world, (rank + 1) * rows // world


def upload_rows(ctx, fmt, rows, cols, parts, row_lo=0, row_hi=None):
    """Store entry holding rows [row_lo, row_hi) of the row-stacked tensors `parts`."""
    row_hi = rows if row_hi is None else row_hi
    w = ctx.store_create(fmt, row_hi - row_lo, cols)
    for off, nrows, data in shard_slices(fmt, cols, parts, row_lo, row_hi):
        w.write_rows(off, nrows, data)
    return w


class SingleGpuDecode:
    def __init__(self, ctx, layers, hidden, kv, ffn, fmt, seed, m_max=8):
        self.ctx, self.hidden = ctx, hidden
        self.stack = _capi.Stack(ctx, layers, hidden, kv, ffn, m_max)
        for L in range(layers):
            ws = [upload_rows(ctx, fmt, rows, cols, parts)
                  for rows, cols, parts in stacked(layer_tensors(fmt, hidden, kv, ffn, seed, L))]
            self.stack.set_layer(L, *ws)
        import os
        if os.environ.get("QM_STACK_MODE"):
            self.stack.use_graph(int(os.environ["QM_STACK_MODE"]))

    def step_device(self, x_dev, m, h_dev):
        self.stack.step(x_dev.data_ptr(), m, self.hidden, h_dev.data_ptr(), self.hidden)

    def step_host(self, x, h, kv):
        self.stack.step_host(x, h_out=h, kv_out=kv)

    def close(self):
        """Frees the stack and its weights."""
        weights = [w for layer in self.stack.weights for w in layer]
        self.stack.close()
        for w in weights:
            w.free()


def column_shard(fmt, rows, cols, data, col_lo, col_hi):
    """GGUF bytes of the columns [col_lo, col_hi) of a rows x cols tensor: for every row the blocks of that range."""
    be, bb = synth.BLOCK[fmt]
    a = np.asarray(data, dtype=np.uint8).reshape(rows, cols // be * bb)
    return np.ascontiguousarray(a[:, col_lo // be * bb:col_hi // be * bb]).reshape(-1)


def upload_row_slices(ctx, fmt, cols, tensors, rank, world):
    """One store entry: slice `rank` of the rows of every tensor in `tensors` [(rows, bytes)], stacked in order."""
    be, bb = synth.BLOCK[fmt]
    row_bytes = cols // be * bb
    w = ctx.store_create(fmt, sum(r for r, _ in tensors) // world, cols)
    off = 0
    for rows, data in tensors:
        lo, hi = shard_range(rows, rank, world)
        w.write_rows(off, hi - lo, data[lo * row_bytes:hi * row_bytes])
        off += hi - lo
    return w


class PeerTensorParallelDecode:
    """Tensor-parallel decode step as ONE persistent launch per GPU. Every rank stores its results straight
    into the peers' activation buffers over NVLink; consumers poll their own arena for the words they read,
    so no barrier crosses the GPUs inside a step (one ends it). torch.distributed only carries the 64-byte
    IPC handles at set-up.
    paired=False (qm_stack_create_tp): rank r holds rows [r*N/g, (r+1)*N/g) of every matrix; four exchanges
    per layer. paired=True (qm_stack_create_tp_paired, up to four activation rows): q|k|v and gate|up by rows,
    o and down by the K columns of the rank's own slices; two exchanges per layer."""

    def __init__(self, ctx, layers, hidden, kv, ffn, fmt, seed, rank, world, m_max=8, barrier=True, paired=False):
        """barrier=False: the caller runs a collective of its own on all ranks before the first
        step (every rank must have mapped every arena before any rank stores into one)."""
        import torch.distributed as dist
        self.ctx, self.hidden, self.rank, self.world, self.paired = ctx, hidden, rank, world, paired
        self.stack = _capi.Stack(ctx, layers, hidden, kv, ffn, m_max, rank, world, paired=paired)
        for L in range(layers):
            if paired:
                t = {n: (r, c, b) for n, r, c, b in layer_tensors(fmt, hidden, kv, ffn, seed, L)}
                kvt = (2 * kv, np.concatenate([np.asarray(t["k"][2]), np.asarray(t["v"][2])]))   # k|v as one tensor of 2*kv rows
                klo, khi = shard_range(hidden, rank, world)
                flo, fhi = shard_range(ffn, rank, world)
                ws = [upload_row_slices(ctx, fmt, hidden, [(hidden, t["q"][2]), kvt], rank, world),
                      ctx.store_upload(fmt, hidden, khi - klo, column_shard(fmt, hidden, hidden, t["o"][2], klo, khi)),
                      upload_row_slices(ctx, fmt, hidden, [(ffn, t["gate"][2]), (ffn, t["up"][2])], rank, world),
                      ctx.store_upload(fmt, hidden, fhi - flo, column_shard(fmt, hidden, ffn, t["down"][2], flo, fhi))]
                self.stack.set_layer(L, *ws)
                continue
            ws = []
            for i, (rows, cols, parts) in enumerate(stacked(layer_tensors(fmt, hidden, kv, ffn, seed, L))):
                lo, hi = shard_range(rows, rank, world)   # every matrix sliced by rows
                ws.append(upload_rows(ctx, fmt, rows, cols, parts, lo, hi))
            self.stack.set_layer(L, *ws)
        handles = [None] * world
        dist.all_gather_object(handles, self.stack.ipc_handle())
        self.stack.set_peers(handles)
        if barrier:
            dist.barrier()   # every rank has mapped every arena before the first step

    def step_device(self, x_dev, m, h_dev):
        self.stack.step(x_dev.data_ptr(), m, self.hidden, h_dev.data_ptr(), self.hidden)

    def step_host(self, x, h, kv):
        self.stack.step_host(x, h_out=h, kv_out=kv)


class TensorParallelDecode:
    """Row-sharded decode step: rank r holds rows [r*N/g, (r+1)*N/g) of every stacked matrix,
    computes its slice of each matvec and all-gathers the slices (NCCL) so that every rank
    holds the full activation vector for the next matvec. The step is captured into one CUDA
    graph per batch size."""

    def __init__(self, ctx, layers, hidden, kv, ffn, fmt, seed, rank, world, stream):
        import torch
        self.torch, self.ctx, self.rank, self.world, self.stream = torch, ctx, rank, world, stream
        self.layers, self.hidden, self.kv, self.ffn = layers, hidden, kv, ffn
        self.rows = [hidden + 2 * kv, hidden, 2 * ffn, hidden]
        for n in self.rows:
            if n % (world * 4) != 0:
                raise ValueError("rows %d do not split over %d ranks" % (n, world))
        self.w = []
        for L in range(layers):
            ws = []
            for rows, cols, parts in stacked(layer_tensors(fmt, hidden, kv, ffn, seed, L)):
                lo, hi = shard_range(rows, rank, world)
                ws.append(upload_rows(ctx, fmt, rows, cols, parts, lo, hi))
            self.w.append(ws)
        _trace("weights uploaded")
        self.graphs = {}

    def _buffers(self, m):
        t, dev = self.torch, "cuda"
        g = self.world
        return {
            "x": t.empty(m, self.hidden, device=dev),
            "shard": [t.empty(m, n // g, device=dev) for n in self.rows],
            "gath": [t.empty(g, m, n // g, device=dev) for n in self.rows],
            "full": [t.empty(m, n, device=dev) for n in self.rows],
            "qkv_all": t.empty(self.layers, m, self.rows[0], device=dev),
        }

    def _enqueue(self, b, m):
        import torch.distributed as dist
        t, g = self.torch, self.world
        ops = [_capi.XOP_RMSNORM, _capi.XOP_RMSNORM, _capi.XOP_RMSNORM, _capi.XOP_ADD_RMSNORM]
        x, ldx, x2 = b["x"], self.hidden, 0
        for L in range(self.layers):
            for i in range(4):
                n = self.rows[i]
                if i == 3:
                    x2 = x.data_ptr() + self.ffn * 4
                # no programmatic dependent launch here: the neighbours in the stream are NCCL kernels
                self.ctx.matvec(self.w[L][i], x.data_ptr(), m, ldx, b["shard"][i].data_ptr(), n // g,
                                ops[i], x2 if i == 3 else 0)
                full = b["qkv_all"][L] if i == 0 else b["full"][i]
                if m == 1:
                    dist.all_gather_into_tensor(full.view(-1), b["shard"][i].view(-1))
                else:
                    dist.all_gather_into_tensor(b["gath"][i].view(-1), b["shard"][i].view(-1))
                    full.view(m, g, n // g).copy_(b["gath"][i].permute(1, 0, 2))
                x, ldx = full, n
        return x  # the last down-projection output, gathered

    def _graph(self, m):
        if m not in self.graphs:
            t = self.torch
            b = self._buffers(m)
            with t.cuda.stream(self.stream):
                self.ctx.set_stream(self.stream.cuda_stream)
                _trace("eager warm-up pass")
                self._enqueue(b, m)  # warm-up outside capture (NCCL connection set-up)
                self.stream.synchronize()
                _trace("capturing")
                graph = t.cuda.CUDAGraph()
                with t.cuda.graph(graph, stream=self.stream):
                    self.ctx.set_stream(t.cuda.current_stream().cuda_stream)
                    out = self._enqueue(b, m)
                self.ctx.set_stream(self.stream.cuda_stream)
            _trace("captured")
            self.graphs[m] = (graph, b, out)
        return self.graphs[m]

    def step_device(self, x_dev, m, h_dev):
        graph, b, out = self._graph(m)
        b["x"].copy_(x_dev, non_blocking=True)
        _trace("replay")
        graph.replay()
        h_dev.copy_(out, non_blocking=True)

    def step_host(self, x, h, kv):
        t = self.torch
        m = x.shape[0]
        graph, b, out = self._graph(m)
        b["x"].copy_(t.from_numpy(x), non_blocking=True)
        graph.replay()
        t.from_numpy(h).copy_(out, non_blocking=True)
        t.from_numpy(kv).copy_(b["qkv_all"][:, :, self.hidden:], non_blocking=True)
        t.cuda.current_stream().synchronize()
