// qm_moe.cu — mixture-of-experts plumbing around the quantized matmuls (sm_100a):
// top-k routing with the reference's exact semantics, per-expert token lists, gather,
// SwiGLU and the weighted combine.
//
// Routing restates GroupedTopKRouter.Route (lm/moe/moe.go:73-141): experts are ranked by
// logit + bias (descending, ties to the lower index), the weights are the softmax of the
// UNBIASED logits of the selected experts with exp evaluated in double precision and rounded
// to float32, summed in float32 in selection order. The gather supersedes the reference's
// moe_gather (nvidia/x/cudamoe/moe.go:72-96).
#include <cuda_bf16.h>
#include <stdint.h>

#include "qm_kernel_args.h"

// One thread per token.
extern "C" __global__ void __launch_bounds__(128) qm_moe_route(const __grid_constant__ QmRouteArgs a) {
    const int tok = blockIdx.x * blockDim.x + threadIdx.x;
    if (tok >= a.tokens) return;
    const float *lg = a.logits + (int64_t)tok * a.ld;
    const int n = a.experts, k = min(a.topk, n);
    int32_t *ids = a.ids + (int64_t)tok * a.topk;
    float *wts = a.weights + (int64_t)tok * a.topk;
    unsigned long long taken[QM_MAX_EXPERTS / 64] = {};   // one bit per expert
    float max_logit = 0.f;
    for (int s = 0; s < k; s++) {
        int best = -1;
        float best_score = 0.f;
        for (int e = 0; e < n; e++) {
            if (taken[e >> 6] >> (e & 63) & 1ull) continue;
            const float sc = __fadd_rn(lg[e], a.bias ? a.bias[e] : 0.f);
            if (best < 0 || sc > best_score) { best = e; best_score = sc; }   // strict: ties keep the lower index
        }
        taken[best >> 6] |= 1ull << (best & 63);
        ids[s] = best;
        const float l = lg[best];
        if (s == 0 || l > max_logit) max_logit = l;
    }
    float sum = 0.f;
    for (int s = 0; s < k; s++) {
        const float e = (float)exp((double)__fsub_rn(lg[ids[s]], max_logit));
        wts[s] = e;
        sum = __fadd_rn(sum, e);
    }
    if (sum > 0.f)
        for (int s = 0; s < k; s++) wts[s] = __fdiv_rn(wts[s], sum);
    for (int s = k; s < a.topk; s++) { ids[s] = -1; wts[s] = 0.f; }
}

// Token lists per expert, in ascending (token, slot) order: one warp per expert compacts the
// pairs with ballots. counts[e], offsets[e] (exclusive prefix, written by warp 0 at the end),
// list[] = pair index (token*topk + slot) grouped by expert, pos[pair] = row in that grouping.
extern "C" __global__ void __launch_bounds__(1024) qm_moe_lists(const __grid_constant__ QmListArgs a) {
    __shared__ int s_count[QM_MAX_EXPERTS], s_off[QM_MAX_EXPERTS + 1];
    // up to kSmall pairs the expert numbers and ranks stay in shared memory (one pass over ids)
    constexpr int kSmall = 8192;
    __shared__ short s_id[kSmall], s_rank[kSmall];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int npairs = a.tokens * a.topk;
    const bool small = npairs <= kSmall;
    if (small) {
        for (int pr = threadIdx.x; pr < npairs; pr += blockDim.x) {
            const int e = a.ids[pr];
            s_id[pr] = (short)((e < 0 || e >= a.experts) ? -1 : e);
        }
        __syncthreads();
    }
    for (int e = warp; e < a.experts; e += blockDim.x >> 5) {
        int cnt = 0;
        for (int base = 0; base < npairs; base += 32) {
            const int pr = base + lane;
            const bool mine = pr < npairs && (small ? (int)s_id[pr] : a.ids[pr]) == e;
            const unsigned int bal = __ballot_sync(0xffffffffu, mine);
            if (mine) {
                const int r = cnt + __popc(bal & ((1u << lane) - 1u));
                if (small) s_rank[pr] = (short)r;
                else a.rank[pr] = r;
            }
            cnt += __popc(bal);
        }
        if (lane == 0) s_count[e] = cnt;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int off = 0;
        for (int e = 0; e < a.experts; e++) {
            a.counts[e] = s_count[e];
            a.offsets[e] = off;
            s_off[e] = off;
            off += s_count[e];
        }
        a.offsets[a.experts] = off;
    }
    __syncthreads();
    for (int pr = threadIdx.x; pr < npairs; pr += blockDim.x) {
        const int e = small ? (int)s_id[pr] : a.ids[pr];
        if (e < 0 || e >= a.experts) { a.pos[pr] = -1; continue; }   // names no expert: in no list
        const int p = s_off[e] + (small ? (int)(unsigned short)s_rank[pr] : a.rank[pr]);
        a.pos[pr] = p;
        a.list[p] = pr;
    }
}

// gathered[p][:] = x[token(list[p])][:], bf16 rows of `hidden` elements (16-byte pieces).
extern "C" __global__ void __launch_bounds__(256) qm_moe_gather(const __grid_constant__ QmGatherArgs a) {
    const int pieces = a.hidden / 8;
    const int64_t total = (int64_t)a.rows * pieces;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int p = (int)(i / pieces), c = (int)(i - (int64_t)p * pieces);
        const int pr = a.list[p];
        const int tok = pr / a.topk;
        reinterpret_cast<uint4 *>(a.out + (int64_t)p * a.hidden)[c] =
            reinterpret_cast<const uint4 *>(a.x + (int64_t)tok * a.ldx)[c];
    }
}

// out[tok][:] = sum_s weights[tok][s] * y[pos[tok*topk+s]][:] in slot order (deterministic).
extern "C" __global__ void __launch_bounds__(256) qm_moe_combine(const __grid_constant__ QmCombineArgs a) {
    if (((a.hidden | a.ldo) & 3) == 0 && (((uintptr_t)a.y | (uintptr_t)a.out) & 15) == 0) {   // four columns per thread
        const int h4 = a.hidden >> 2;
        const int64_t total4 = (int64_t)a.tokens * h4;
        for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total4; i += (int64_t)gridDim.x * blockDim.x) {
            const int tok = (int)(i / h4), c = (int)(i - (int64_t)tok * h4);
            float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int k = 0; k < a.topk; k++) {
                const int p = a.pos[tok * a.topk + k];
                if (p >= 0) {
                    const float w = a.weights[tok * a.topk + k];
                    const float4 v = reinterpret_cast<const float4 *>(a.y + (int64_t)p * a.hidden)[c];
                    s.x = fmaf(w, v.x, s.x); s.y = fmaf(w, v.y, s.y); s.z = fmaf(w, v.z, s.z); s.w = fmaf(w, v.w, s.w);
                }
            }
            reinterpret_cast<float4 *>(a.out + (int64_t)tok * a.ldo)[c] = s;
        }
        return;
    }
    const int64_t total = (int64_t)a.tokens * a.hidden;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int tok = (int)(i / a.hidden), c = (int)(i - (int64_t)tok * a.hidden);
        float s = 0.f;
        for (int k = 0; k < a.topk; k++) {
            const int p = a.pos[tok * a.topk + k];
            if (p >= 0) s = fmaf(a.weights[tok * a.topk + k], a.y[(int64_t)p * a.hidden + c], s);
        }
        a.out[(int64_t)tok * a.ldo + c] = s;
    }
}

// Decode-time MoE: the weighted sum of a token's slot outputs, in slot order.
extern "C" __global__ void __launch_bounds__(256) qm_moe_decode_combine(const __grid_constant__ QmDecodeCombineArgs a) {
    const int64_t total = (int64_t)a.tokens * a.hidden;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int tok = (int)(i / a.hidden), c = (int)(i - (int64_t)tok * a.hidden);
        float s = 0.f;
        bool bad = false;
        for (int k = 0; k < a.topk; k++) {
            const int id = a.ids[tok * a.topk + k];
            bad |= id < 0 || id >= a.experts;
            s = fmaf(a.weights[tok * a.topk + k], a.y[(int64_t)(tok * a.topk + k) * a.hidden + c], s);
        }
        a.out[(int64_t)tok * a.ldo + c] = bad ? __int_as_float(0x7fffffff) : s;
    }
}

// ---- expert parallelism over peer memory ----------------------------------------------------------
// Four kernels per step and rank. push: this rank's routed rows go straight into the arenas of the ranks
// that own their experts (plain 16-byte peer stores), then one flag per peer says "rank r has pushed".
// collect: waits (bounded) for every rank's flag, regroups what arrived by local expert. [grouped expert
// matmuls] return: every result row goes back into its sender's arena, flag "owner o has returned".
// combine: waits for every owner's flag, adds a token's slots with the routing weights, slots in order.
// No kernel waits for a kernel of its own GPU: flags come from other GPUs, or from launches that precede
// the waiting one in the stream.
namespace {
template <typename T>
__device__ __forceinline__ T *at_peer(T *p, int64_t delta) {
    return reinterpret_cast<T *>(reinterpret_cast<char *>(p) + delta);
}
__device__ __forceinline__ void ep_st_release_sys(unsigned int *p, unsigned int v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ep_ld_acquire_sys(const unsigned int *p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// The last CTA of the grid to get here publishes `epoch` in flag [phase][rank] of every rank's arena.
__device__ __forceinline__ void ep_signal(const QmEpArgs &a, int phase) {
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        if (atomicAdd(a.done + phase, 1u) + 1u == gridDim.x) {
            __threadfence_system();
            for (int p = 0; p < a.world; p++)
                ep_st_release_sys(at_peer(a.flags + phase * QM_MAX_PEERS + a.rank, a.peer_delta[p]), a.epoch);
        }
    }
}
// Every CTA waits until all ranks' flags of `phase` have reached the epoch; gives up after wait_cycles.
__device__ __forceinline__ void ep_wait(const QmEpArgs &a, int phase) {
    if ((int)threadIdx.x < a.world) {
        const long long t0 = clock64();
        while ((int)(ep_ld_acquire_sys(a.flags + phase * QM_MAX_PEERS + threadIdx.x) - a.epoch) < 0) {
            if (clock64() - t0 > a.wait_cycles) {
                atomicOr(a.status, QM_STATUS_TIMEOUT);
                break;
            }
        }
    }
    __syncthreads();
}
}  // namespace

extern "C" __global__ void __launch_bounds__(256) qm_ep_push(const __grid_constant__ QmEpArgs a) {
    const int lane = threadIdx.x & 31;
    const int nwarps = (gridDim.x * blockDim.x) >> 5, gwarp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (blockIdx.x == 0)
        for (int i = threadIdx.x; i < a.world * a.eloc; i += blockDim.x) {
            const int o = i / a.eloc, e = i - o * a.eloc, ge = o * a.eloc + e;
            *at_peer(a.counts_in + a.rank * a.eloc + e, a.peer_delta[o]) = a.offsets[ge + 1] - a.offsets[ge];
        }
    const int routed = a.offsets[a.experts], pieces = a.hidden / 8;
    for (int p = gwarp; p < routed; p += nwarps) {
        const int pr = a.list[p], o = a.ids[pr] / a.eloc;
        const int idx = p - a.offsets[o * a.eloc];   // place in the segment that goes to owner o
        const uint4 *src = reinterpret_cast<const uint4 *>(a.x + (int64_t)(pr / a.topk) * a.ldx);
        uint4 *dst = reinterpret_cast<uint4 *>(at_peer(a.rows_in + ((int64_t)a.rank * a.cap + idx) * a.hidden, a.peer_delta[o]));
        for (int c = lane; c < pieces; c += 32) dst[c] = src[c];
    }
    ep_signal(a, 0);
}

extern "C" __global__ void __launch_bounds__(256) qm_ep_collect(const __grid_constant__ QmEpArgs a) {
    __shared__ int cnt[QM_MAX_PEERS * 64], from[QM_MAX_PEERS * 64], seg[QM_MAX_PEERS * 64 + 1];
    ep_wait(a, 0);
    const int lane = threadIdx.x & 31, W = a.world, E = a.eloc;
    for (int i = threadIdx.x; i < W * E; i += blockDim.x) cnt[i] = min(max(__ldcg(a.counts_in + i), 0), a.cap);
    __syncthreads();
    if (threadIdx.x == 0) {
        // compact order: local expert, then source rank; a source's rows arrive grouped by local expert
        int run = 0;
        for (int e = 0; e < E; e++)
            for (int s = 0; s < W; s++) {
                seg[e * W + s] = run;
                run += cnt[s * E + e];
            }
        seg[E * W] = run;
        for (int s = 0; s < W; s++) {
            int f = 0;
            for (int e = 0; e < E; e++) {
                from[s * E + e] = f;
                f += cnt[s * E + e];
            }
        }
    }
    __syncthreads();
    const int R = min(seg[E * W], W * a.cap);
    if (blockIdx.x == 0 && (int)threadIdx.x <= E) a.loff[threadIdx.x] = threadIdx.x == E ? R : min(seg[threadIdx.x * W], R);
    const int nwarps = (gridDim.x * blockDim.x) >> 5, gwarp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int pieces = a.hidden / 8;
    for (int c = gwarp; c < R; c += nwarps) {
        int lo = 0, hi = E * W;   // the segment k with seg[k] <= c < seg[k + 1]
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (seg[mid] <= c) lo = mid; else hi = mid;
        }
        const int e = lo / W, s = lo - e * W;
        const int idx = min(from[s * E + e] + (c - seg[lo]), a.cap - 1);
        const uint4 *src = reinterpret_cast<const uint4 *>(a.rows_in + ((int64_t)s * a.cap + idx) * a.hidden);
        uint4 *dst = reinterpret_cast<uint4 *>(a.compact + (int64_t)c * a.hidden);
        for (int q = lane; q < pieces; q += 32) dst[q] = __ldcg(src + q);
        if (lane == 0) a.back[c] = (s << 24) | idx;
    }
}

extern "C" __global__ void __launch_bounds__(256) qm_ep_return(const __grid_constant__ QmEpArgs a) {
    const int lane = threadIdx.x & 31;
    const int nwarps = (gridDim.x * blockDim.x) >> 5, gwarp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int R = min(a.loff[a.eloc], a.world * a.cap), pieces = a.hidden / 4;
    for (int c = gwarp; c < R; c += nwarps) {
        const int b = a.back[c], s = b >> 24, idx = b & 0xFFFFFF;
        const uint4 *src = reinterpret_cast<const uint4 *>(a.y + (int64_t)c * a.hidden);
        uint4 *dst = reinterpret_cast<uint4 *>(at_peer(a.ret_in + ((int64_t)a.rank * a.cap + idx) * a.hidden, a.peer_delta[s]));
        for (int q = lane; q < pieces; q += 32) dst[q] = src[q];
    }
    ep_signal(a, 1);
}

extern "C" __global__ void __launch_bounds__(256) qm_ep_combine(const __grid_constant__ QmEpArgs a) {
    ep_wait(a, 1);
    const int64_t total = (int64_t)a.tokens * a.hidden;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int tok = (int)(i / a.hidden), c = (int)(i - (int64_t)tok * a.hidden);
        float s = 0.f;
        for (int k = 0; k < a.topk; k++) {
            const int pr = tok * a.topk + k, p = a.pos[pr];
            if (p < 0) continue;
            const int o = a.ids[pr] / a.eloc, idx = p - a.offsets[o * a.eloc];
            s = fmaf(a.weights[pr], __ldcg(a.ret_in + ((int64_t)o * a.cap + idx) * a.hidden + c), s);
        }
        a.out[(int64_t)tok * a.ldo + c] = s;
    }
}
