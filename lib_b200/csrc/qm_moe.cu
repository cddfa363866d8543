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
    unsigned long long taken = 0ull;   // experts <= 64
    float max_logit = 0.f;
    for (int s = 0; s < k; s++) {
        int best = -1;
        float best_score = 0.f;
        for (int e = 0; e < n; e++) {
            if (taken >> e & 1ull) continue;
            const float sc = __fadd_rn(lg[e], a.bias ? a.bias[e] : 0.f);
            if (best < 0 || sc > best_score) { best = e; best_score = sc; }   // strict: ties keep the lower index
        }
        taken |= 1ull << best;
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
    __shared__ int s_count[64];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int npairs = a.tokens * a.topk;
    for (int e = warp; e < a.experts; e += blockDim.x >> 5) {
        int cnt = 0;
        for (int base = 0; base < npairs; base += 32) {
            const int pr = base + lane;
            const bool mine = pr < npairs && a.ids[pr] == e;
            const unsigned int bal = __ballot_sync(0xffffffffu, mine);
            if (mine) a.rank[pr] = cnt + __popc(bal & ((1u << lane) - 1u));
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
            off += s_count[e];
        }
        a.offsets[a.experts] = off;
    }
    __syncthreads();
    for (int pr = threadIdx.x; pr < npairs; pr += blockDim.x) {
        const int e = a.ids[pr];
        if (e < 0) { a.pos[pr] = -1; continue; }
        int off = 0;
        for (int x = 0; x < e; x++) off += s_count[x];
        const int p = off + a.rank[pr];
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
