"""Mixture-of-experts layer over the quantized expert store: single GPU, and expert-parallel
across the GPUs of one box with an all-to-all token dispatch.

The routing follows lm/moe GroupedTopKRouter.Route (lm/moe/moe.go:73-141); the device gather
of routed rows corresponds to nvidia/x/cudamoe/moe.go:72-96. The reference has no multi-GPU
dispatch of its own: the exchange here is torch.distributed's all_to_all_single (NCCL on the
GPUs, gloo in the CPU tests), everything on either side of it is this package's kernels.

Expert-parallel data flow, per rank (T local tokens, E experts, E/world experts per rank):

  route -> dispatch (rows grouped by global expert, so also by destination rank)
        -> all-gather of the E list lengths           (tiny, decides the split sizes)
        -> all-to-all of the bf16 rows
        -> dispatch again on the receiver (rows from all sources regrouped by local expert)
        -> grouped expert matmuls -> back to arrival order
        -> all-to-all of the fp32 results back to their senders
        -> combine with the routing weights, slots in order (deterministic).
"""
import numpy as np
import torch
import torch.distributed as dist

from . import synth

Q4_K = 12


def ep_plan(counts, rank, world):
    """Split sizes of the exchange. counts[src][e] = rows that rank `src` holds for global expert
    e. Returns (send_splits, recv_splits, recv_ids): rows this rank sends to every rank, rows
    it receives from every rank, and the LOCAL expert index of every received row in arrival
    order (source-major, expert-major inside a source)."""
    counts = np.asarray(counts, dtype=np.int64)
    experts = counts.shape[1]
    if experts % world:
        raise ValueError("experts must divide evenly over the ranks")
    per = experts // world
    send = [int(counts[rank, d * per:(d + 1) * per].sum()) for d in range(world)]
    recv = [int(counts[s, rank * per:(rank + 1) * per].sum()) for s in range(world)]
    ids = np.concatenate([np.repeat(np.arange(per, dtype=np.int32), counts[s, rank * per:(rank + 1) * per])
                          for s in range(world)]) if sum(recv) else np.zeros(0, np.int32)
    return send, recv, ids.astype(np.int32)


def expert_parallel_forward(ops, x, ids, weights, experts, rank, world, group=None):
    """The exchange logic around the kernels. `ops` supplies the three stages on tensors of
    its device: dispatch(ids[T,k], x[T,H], experts) -> (rows[P,H], pos[P], counts list),
    run_experts(rows[R,H], counts list over the local experts) -> y[R,H] float32,
    combine(y[P,H], pos[P], weights[T,k]) -> out[T,H] float32."""
    tokens, topk = ids.shape
    rows, pos, counts = ops.dispatch(ids, x, experts)
    if world == 1:
        y = ops.run_experts(rows, counts)
        return ops.combine(y, pos, weights)
    mine = torch.tensor(counts, dtype=torch.int32, device=x.device)
    allc = torch.empty(world * experts, dtype=torch.int32, device=x.device)
    dist.all_gather_into_tensor(allc, mine, group=group)
    send, recv, recv_ids = ep_plan(allc.cpu().numpy().reshape(world, experts), rank, world)
    got = torch.empty((sum(recv), x.shape[1]), dtype=x.dtype, device=x.device)
    dist.all_to_all_single(got, rows[:sum(send)].contiguous(), recv, send, group=group)
    # regroup what arrived by local expert, run the experts, and undo the regrouping
    rid = torch.from_numpy(recv_ids).to(x.device).reshape(-1, 1)
    rows2, pos2, counts2 = ops.dispatch(rid, got, experts // world)
    y2 = ops.run_experts(rows2, counts2)
    ones = torch.ones((got.shape[0], 1), dtype=torch.float32, device=x.device)
    y_arrival = ops.combine(y2, pos2, ones)
    back = torch.empty((sum(send), x.shape[1]), dtype=torch.float32, device=x.device)
    dist.all_to_all_single(back, y_arrival, send, recv, group=group)
    return ops.combine(back, pos, weights)


class GpuStages:
    """The three stages on this GPU through the C ABI (qm_moe_dispatch / _experts / _combine)."""

    def __init__(self, ctx, gate_up, down, hidden):
        self.ctx, self.gate_up, self.down, self.hidden = ctx, gate_up, down, hidden

    def dispatch(self, ids, x, experts):
        tokens, topk = ids.shape
        pairs = tokens * topk
        rows = torch.empty((max(pairs, 1), self.hidden), dtype=torch.bfloat16, device=x.device)
        pos = torch.empty(max(pairs, 1), dtype=torch.int32, device=x.device)
        if tokens == 0:
            return rows[:0], pos[:0], [0] * experts
        ids = ids.contiguous()
        counts = self.ctx.moe_dispatch(ids.data_ptr(), tokens, topk, experts, x.data_ptr(), x.stride(0), self.hidden,
                                       rows.data_ptr(), pos.data_ptr())
        return rows[:pairs], pos[:pairs], counts

    def run_experts(self, rows, counts):
        y = torch.empty((max(rows.shape[0], 1), self.hidden), dtype=torch.float32, device=rows.device)
        if rows.shape[0]:
            self.ctx.moe_experts(self.gate_up, self.down, rows.data_ptr(), counts, y.data_ptr())
        return y[:rows.shape[0]]

    def combine(self, y, pos, weights):
        tokens, topk = weights.shape
        out = torch.empty((max(tokens, 1), self.hidden), dtype=torch.float32, device=weights.device)
        if tokens:
            if y.shape[0] == 0:   # nothing routed anywhere: cannot happen with topk >= 1
                return out[:tokens].zero_()
            self.ctx.moe_combine(y.data_ptr(), pos.data_ptr(), weights.contiguous().data_ptr(), tokens, topk,
                                 self.hidden, out.data_ptr(), self.hidden)
        return out[:tokens]


def expert_weights(hidden, ffn, expert, seed):
    """GGUF bytes of expert `expert`: (gate|up [2*ffn][hidden], down [hidden][ffn]), Q4_K."""
    return (synth.weights(Q4_K, 2 * ffn, hidden, seed * 1000 + 2 * expert),
            synth.weights(Q4_K, hidden, ffn, seed * 1000 + 2 * expert + 1))


class MoELayer:
    """One SwiGLU mixture-of-experts layer with seeded random Q4_K experts. With world > 1 rank r
    holds experts [r*E/world, (r+1)*E/world) and `forward` exchanges rows with the other ranks;
    the seeds depend on the global expert index only, so every world size computes the same
    layer."""

    def __init__(self, ctx, experts, topk, hidden, ffn, seed, rank=0, world=1, group=None):
        if experts % world:
            raise ValueError("experts must divide evenly over the ranks")
        self.ctx, self.experts, self.topk, self.hidden, self.ffn = ctx, experts, topk, hidden, ffn
        self.rank, self.world, self.group = rank, world, group
        per = experts // world
        self.gate_up, self.down = [], []
        for e in range(rank * per, (rank + 1) * per):
            gu, dn = expert_weights(hidden, ffn, e, seed)
            self.gate_up.append(ctx.store_upload(Q4_K, 2 * ffn, hidden, gu))
            self.down.append(ctx.store_upload(Q4_K, hidden, ffn, dn))
        self.stages = GpuStages(ctx, self.gate_up, self.down, hidden)
        self.weight_bytes = per * (synth.gguf_bytes(Q4_K, 2 * ffn, hidden) + synth.gguf_bytes(Q4_K, hidden, ffn))

    def route(self, logits):
        tokens = logits.shape[0]
        ids = torch.empty((tokens, self.topk), dtype=torch.int32, device=logits.device)
        w = torch.empty((tokens, self.topk), dtype=torch.float32, device=logits.device)
        if tokens:
            self.ctx.moe_route(logits.data_ptr(), tokens, logits.stride(0), self.experts, self.topk,
                               ids.data_ptr(), w.data_ptr())
        return ids, w

    def forward(self, x, logits):
        """x bf16 [T][hidden], logits float32 [T][experts] (this rank's tokens) -> float32 [T][hidden].
        Runs on torch's current CUDA stream."""
        self.ctx.set_stream(torch.cuda.current_stream().cuda_stream)
        ids, w = self.route(logits)
        return expert_parallel_forward(self.stages, x, ids, w, self.experts, self.rank, self.world, self.group)

    def close(self):
        for w in self.gate_up + self.down:
            w.free()
        self.gate_up, self.down = [], []


class PeerExpertParallelLayer(MoELayer):
    """The same layer with the exchange behind the C ABI (qm_ep_*): routed rows and results travel through
    peer memory, no collective library on the data path. `group` (any torch.distributed backend) is used
    once, at set-up, to hand the 64-byte IPC handles of the arenas around."""

    def __init__(self, ctx, experts, topk, hidden, ffn, seed, max_tokens, rank=0, world=1, group=None):
        super().__init__(ctx, experts, topk, hidden, ffn, seed, rank, world, group)
        from ._capi import ExpertParallel
        self.ep = ExpertParallel(ctx, self.gate_up, self.down, experts, topk, max_tokens, rank, world)
        if world > 1:
            handles = [None] * world
            dist.all_gather_object(handles, self.ep.ipc_handle(), group=group)
            self.ep.set_peers(handles)
            dist.barrier(group=group)       # every rank has mapped its peers before any rank runs a step

    def forward(self, x, logits):
        self.ctx.set_stream(torch.cuda.current_stream().cuda_stream)
        ids, w = self.route(logits)
        tokens = x.shape[0]
        out = torch.empty((max(tokens, 1), self.hidden), dtype=torch.float32, device=x.device)
        self.ep.moe(x.data_ptr(), tokens, x.stride(0) if tokens else self.hidden, ids.data_ptr(), w.data_ptr(),
                    out.data_ptr(), self.hidden)
        self._keep = (ids, w)               # the step reads them asynchronously
        return out[:tokens]

    def close(self):
        self.ep.close()
        super().close()


class ExpertCacheManager:
    """moe.ExpertCacheManager (lm/moe/moe.go:143-287) over the library's host-side cache: at most
    max_hot expert blobs in memory, least recently used spilled to <dir>/expert_<id>.bin, cold
    experts paged back in by get_expert. Method names follow the Go API."""

    def __init__(self, directory, max_hot):
        import ctypes
        from ._capi import lib, _check
        self._lib, self._check, self._ct = lib, _check, ctypes
        h = ctypes.c_void_p()
        _check(lib.qm_expert_cache_create((directory or "").encode(), int(max_hot), ctypes.byref(h)),
               "NewExpertCacheManager")
        self._h = h

    def register_expert(self, expert_id, weights):
        data = bytes(weights)
        self._check(self._lib.qm_expert_cache_register(self._h, int(expert_id), data, len(data)), "RegisterExpert")

    def get_expert(self, expert_id):
        ct = self._ct
        size = ct.c_int64()
        self._check(self._lib.qm_expert_cache_get(self._h, int(expert_id), None, 0, ct.byref(size)), "GetExpert")
        buf = (ct.c_ubyte * max(1, size.value))()
        self._check(self._lib.qm_expert_cache_get(self._h, int(expert_id), buf, size.value, ct.byref(size)), "GetExpert")
        return bytes(buf[:size.value])

    def hot_experts(self):
        return int(self._lib.qm_expert_cache_hot(self._h))

    def evict_cold_expert(self, expert_id):
        self._check(self._lib.qm_expert_cache_evict(self._h, int(expert_id)), "EvictColdExpert")

    def close(self):
        if self._h:
            self._lib.qm_expert_cache_close(self._h)
            self._h = None


class ExpertPool:
    """qm_expert_pool: device-side residency over an ExpertCacheManager — at most max_resident experts of
    one shape hold a device store entry; `get` pages an expert in over the least recently used entry."""

    def __init__(self, ctx, cache, fmt, rows, cols, max_resident):
        import ctypes
        from ._capi import lib, _check, Weight
        self._lib, self._check, self._ct, self._Weight, self.ctx, self.cache = lib, _check, ctypes, Weight, ctx, cache
        h = ctypes.c_void_p()
        _check(lib.qm_expert_pool_create(ctx._h, cache._h, fmt, rows, cols, int(max_resident), ctypes.byref(h)),
               "expert_pool_create")
        self._h = h

    def get(self, expert_id):
        """The store entry (Weight) that holds the expert now; do not free it."""
        w = self._ct.c_uint64(0)
        self._check(self._lib.qm_expert_pool_get(self.ctx._h, self._h, int(expert_id), self._ct.byref(w)), "expert_pool_get")
        return self._Weight(self.ctx, w.value)

    def info(self):
        """(experts resident, entries, hits, misses)"""
        v = (self._ct.c_int64 * 4)()
        self._check(self._lib.qm_expert_pool_info(self._h, v), "expert_pool_info")
        return tuple(int(x) for x in v)

    def evict(self, expert_id):
        self._check(self._lib.qm_expert_pool_evict(self._h, int(expert_id)), "expert_pool_evict")

    def close(self):
        if self._h:
            self._lib.qm_expert_pool_close(self.ctx._h, self._h)
            self._h = None
