// qm_stack.cpp — a decode step over a stack of transformer-shaped layers whose
// matrices are all block-quantized: per layer q|k|v, o, gate|up and down
// matvecs, RMS normalisation fused into each consumer's activation staging.
// The 4*layers launches are captured once per batch size into a CUDA graph with
// programmatic dependent launch, the capture/replay path the reference exposes
// as Stream.BeginCapture / Graph.Instantiate / GraphExec.Launch
// (nvidia/driver/stream.gen.go:115, graph.gen.go:651, graph_exec.gen.go:354).
#include <string.h>

#include <algorithm>
#include <new>
#include <vector>

#include "qm_internal.h"

#define QM_STACK_MAGIC 0x514D534Bu  // "QMSK"

struct QmLayer {
    QmWeight *qkv, *o, *gu, *dn;
    // part-major copies of the o / down weights for steps that run them in K parts ([part][tile][units/parts]
    // items; same bytes in another order), made on first use and dropped when the layer is set again
    CUdeviceptr o_parts, dn_parts;
    int o_nparts, dn_nparts;
};

struct qm_stack {
    uint32_t magic;
    int layers, hidden, kv, ffn, m_max;
    std::vector<QmLayer> layer;
    // Activations: the step's input h0 [m][hidden], then one block per layer holding that layer's
    // q|k|v, o, gate|up and down outputs (rows packed for the batch m of the step). Every
    // matvec has an output buffer of its own, which lets dependent matvecs hand over through
    // the data itself (see build_fused).
    // Tensor-parallel stacks hold two such halves and alternate between them from step to step:
    // while a step runs in one half, the other is refilled with the "not yet written" pattern
    // for the next step (a peer may start that step, and store into this GPU's arena, before this
    // GPU has left the current one). `act` is the half of the most recent step.
    CUdeviceptr h0, act, act_half[2];
    CUdeviceptr h_sum;          // [m][hidden]: the last down projection summed over its K parts
    int cur_half;
    int half_m[2];              // batch of the last step run in each half (0: the half is all "not yet written")
    size_t act_bytes;
    CUgraphExec graph[9];
    CUdeviceptr ops_dev[9];     // fused op lists, one per batch size
    QmFusedPlan fused_plan[9];
    int fused_nops[9];          // ops in the list (a matrix whose K does not fit is several ops)
    int fused_ncross[9];        // barriers over all GPUs in one tensor-parallel launch
    CUdeviceptr img_dev[9];     // two activation images per batch size, used alternately
    CUdeviceptr sync_dev[9];    // grid barrier word (first 256 bytes), then the unit counters
    size_t sync_bytes[9];
    int img_units[9];
    bool fused_img[9];          // the op list uses activation images
    bool fused_dd[9];           // the op list hands over through the data (no grid barriers)
    int fused_dd_kernel[9];
    int fused_half0[9];         // tensor-parallel: arena half that the first copy of the op list addresses
    int fused_parts_o[9], fused_parts_dn[9];   // K parts of the o / down projections in the op list (1 = whole)
    int fused_ngroups[9];       // CTA groups with a copy of the op list each (data-driven form with K parts)
    // tensor-parallel: one arena holds all activation buffers and the peers' arrival flags; the
    // peers map it through CUDA IPC and this GPU stores its row slices into all of them
    int tp_world, tp_rank;
    // Tensor-parallel sharding. Rows (false): every matrix sliced by output rows, four exchanges per layer.
    // Paired (true): q|k|v and gate|up by rows, o and down by K over the rank's own slice of their inputs —
    // their partial outputs (one vector per GPU) are added by the consumer, two exchanges per layer.
    bool tp_paired;
    int parts_cap;              // partial vectors the o / down buffers of a layer have room for
    CUdeviceptr arena;
    size_t arena_bytes, flags_off;
    CUdeviceptr peer_base[QM_MAX_PEERS];
    bool peers_open;
    bool peers_ipc;             // the peers' arenas were opened from IPC handles (closed again at destroy)
    bool tp_counter;            // peers reachable with native NVLink atomics: counter barrier
    unsigned int tp_epoch;
    bool use_graph, use_fused;
    int last_m;                 // batch of the most recent step
    bool last_dd;               // the most recent step ran in the data-driven form
};

// Device addresses of layer L's output buffers in a step of batch m. The o and down projections
// have room for QM_MAX_PARTS partial output vectors each (see QmOp::parts; steps that do not cut
// them into K parts use the first), followed by the words their K parts publish.
#define QM_MAX_PARTS 4           // K parts of one GPU's op (CTA groups); a paired tensor-parallel stack has one part per GPU
struct LayerBufs {
    CUdeviceptr qkv, o, gu, dn;
    CUdeviceptr ssq_o, ssq_dn;   // [parts_cap][8] floats each
    int64_t part_stride;         // floats between the partial vectors of o (and of dn)
};
static size_t layer_floats(const qm_stack *s, int m) {
    const size_t qkv_ld = (size_t)s->hidden + 2 * s->kv;
    return (size_t)m * (qkv_ld + 2 * (size_t)s->ffn + 2 * s->parts_cap * (size_t)s->hidden) + 2 * s->parts_cap * 8;
}
static LayerBufs layer_bufs(const qm_stack *s, int L, int m) {
    const size_t qkv_ld = (size_t)s->hidden + 2 * s->kv;
    LayerBufs b;
    b.part_stride = (int64_t)m * s->hidden;
    b.qkv = s->act + (size_t)L * layer_floats(s, m) * 4;
    b.o = b.qkv + (size_t)m * qkv_ld * 4;
    b.gu = b.o + (size_t)s->parts_cap * m * s->hidden * 4;
    b.dn = b.gu + (size_t)m * 2 * s->ffn * 4;
    b.ssq_o = b.dn + (size_t)s->parts_cap * m * s->hidden * 4;
    b.ssq_dn = b.ssq_o + s->parts_cap * 8 * 4;
    return b;
}

static qm_stack *stack_check(qm_stack *s) { return (s && s->magic == QM_STACK_MAGIC) ? s : nullptr; }
static CUdeviceptr h_source(const qm_stack *s, int m);

static int32_t stack_create(qm_ctx *c, int32_t layers, int32_t hidden, int32_t kv_dim, int32_t ffn, int32_t m_max,
                            int32_t rank, int32_t world, bool paired, qm_stack **out) {
    CHECK_CTX(c);
    if (!out) return QM_ERR_ARG;
    *out = nullptr;
    if (layers < 1 || layers > 1024 || hidden < 32 || kv_dim < 0 || ffn < 32 || m_max < 1 || m_max > 8)
        return QM_ERR_SHAPE;
    if ((hidden & 3) || (kv_dim & 3) || (ffn & 3)) return QM_ERR_SHAPE;
    if (world < 1 || world > QM_MAX_PEERS || rank < 0 || rank >= world) return QM_ERR_ARG;
    if (world > 1 && ((hidden % (16 * world)) || ((2 * ffn) % (16 * world)) || ((hidden + 2 * kv_dim) % (16 * world))))
        return QM_ERR_SHAPE;   // every GPU's row slice must be whole 16-row tiles
    // paired: the row slices of q, of k|v, of gate and of up are whole tiles, the K slices of o and down whole units
    if (paired && (world < 2 || (hidden % (256 * world)) || (ffn % (256 * world)) || ((2 * kv_dim) % (16 * world)) || m_max > 4))
        return QM_ERR_SHAPE;
    qm_stack *s = new (std::nothrow) qm_stack();
    if (!s) return QM_ERR_NOMEM;
    s->magic = QM_STACK_MAGIC;
    s->layers = layers;
    s->hidden = hidden;
    s->kv = kv_dim;
    s->ffn = ffn;
    s->m_max = m_max;
    s->tp_world = world;
    s->tp_rank = rank;
    s->tp_paired = paired;
    s->parts_cap = paired ? 8 : QM_MAX_PARTS;   // paired: one part per GPU, or several per GPU while the total stays at eight
    s->arena = 0;
    s->peers_open = false;
    s->peers_ipc = false;
    s->tp_epoch = 0;
    memset(s->peer_base, 0, sizeof s->peer_base);
    s->layer.resize(layers);
    memset(s->layer.data(), 0, sizeof(QmLayer) * layers);
    memset(s->graph, 0, sizeof s->graph);
    memset(s->ops_dev, 0, sizeof s->ops_dev);
    memset(s->img_dev, 0, sizeof s->img_dev);
    memset(s->sync_dev, 0, sizeof s->sync_dev);
    s->use_graph = true;
    s->use_fused = true;
    s->last_m = 0;
    s->last_dd = false;
    s->h0 = s->act = 0;
    s->act_half[0] = s->act_half[1] = 0;
    s->cur_half = 0;
    s->half_m[0] = s->half_m[1] = 0;
    CtxGuard g(c);
    CUresult r = g.rc;
    auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
    const size_t b_h0 = up((size_t)m_max * hidden * 4);
    s->act_bytes = up((size_t)layers * layer_floats(s, m_max) * 4);
    if (world == 1) {
        if (r == CUDA_SUCCESS) r = c->drv->cuMemAlloc_v2(&s->h0, 2 * b_h0);
        s->h_sum = s->h0 + b_h0;
        if (r == CUDA_SUCCESS) r = c->drv->cuMemAlloc_v2(&s->act, s->act_bytes);
        s->act_half[0] = s->act_half[1] = s->act;
    } else {
        s->flags_off = 2 * b_h0 + 2 * s->act_bytes;
        s->arena_bytes = s->flags_off + 256;
        if (r == CUDA_SUCCESS) r = c->drv->cuMemAlloc_v2(&s->arena, s->arena_bytes);
        if (r == CUDA_SUCCESS) r = c->drv->cuMemsetD8Async(s->arena, 0, s->arena_bytes, c->stream);
        s->h0 = s->arena;
        s->h_sum = s->h0 + b_h0;
        s->act_half[0] = s->h_sum + b_h0;
        s->act_half[1] = s->act_half[0] + s->act_bytes;
        s->act = s->act_half[0];
        // both halves start as "not yet written" (all ones)
        if (r == CUDA_SUCCESS) r = c->drv->cuMemsetD8Async(s->act_half[0], 0xFF, 2 * s->act_bytes, c->stream);
        if (r == CUDA_SUCCESS) r = c->drv->cuStreamSynchronize(c->stream);
    }
    if (r != CUDA_SUCCESS) {
        qm_stack_destroy(c, s);
        return (int32_t)r;
    }
    *out = s;
    return QM_OK;
}

extern "C" int32_t qm_stack_create(qm_ctx *c, int32_t layers, int32_t hidden, int32_t kv_dim, int32_t ffn,
                                   int32_t m_max, qm_stack **out) {
    return stack_create(c, layers, hidden, kv_dim, ffn, m_max, 0, 1, false, out);
}

// Tensor-parallel stack: rank `rank` of `world` GPUs of one box. The gate|up and down matrices
// handed to qm_stack_set_layer hold this rank's slice of the rows, rows
// [rank*R/world, (rank+1)*R/world); q|k|v and o are whole on every rank.
extern "C" int32_t qm_stack_create_tp(qm_ctx *c, int32_t layers, int32_t hidden, int32_t kv_dim, int32_t ffn,
                                      int32_t m_max, int32_t rank, int32_t world, qm_stack **out) {
    return stack_create(c, layers, hidden, kv_dim, ffn, m_max, rank, world, false, out);
}

// The paired form: rank r holds of q|k|v the rows of q slice r followed by the rows of k|v slice r, of gate|up the
// rows of gate slice r followed by those of up slice r (slice r of N rows = [r*N/world, (r+1)*N/world)), and of
// o and down ALL rows of the K columns [r*K/world, (r+1)*K/world) — the columns that multiply the rank's own
// slice of q, respectively of gate and up. Up to four activation rows.
extern "C" int32_t qm_stack_create_tp_paired(qm_ctx *c, int32_t layers, int32_t hidden, int32_t kv_dim, int32_t ffn,
                                             int32_t m_max, int32_t rank, int32_t world, qm_stack **out) {
    return stack_create(c, layers, hidden, kv_dim, ffn, m_max, rank, world, true, out);
}

// The CUDA IPC handle (64 bytes) of this stack's activation arena, for the peers.
extern "C" int32_t qm_stack_ipc_handle(qm_ctx *c, qm_stack *s, void *handle64) {
    CHECK_CTX(c);
    if (!stack_check(s) || !handle64 || s->tp_world < 2) return QM_ERR_ARG;
    CtxGuard g(c);
    DRV(g.rc);
    CUipcMemHandle h;
    DRV(c->drv->cuIpcGetMemHandle(&h, s->arena));
    static_assert(sizeof(CUipcMemHandle) == 64, "IPC handle size");
    memcpy(handle64, &h, 64);
    return QM_OK;
}

// handles: world x 64 bytes, entry p = the handle of rank p's arena (entry tp_rank is ignored).
// Maps every peer's arena into this process; a step can run afterwards.
extern "C" int32_t qm_stack_set_peers(qm_ctx *c, qm_stack *s, const void *handles) {
    CHECK_CTX(c);
    if (!stack_check(s) || !handles || s->tp_world < 2 || s->peers_open) return QM_ERR_ARG;
    CtxGuard g(c);
    DRV(g.rc);
    for (int p = 0; p < s->tp_world; p++) {
        if (p == s->tp_rank) {
            s->peer_base[p] = s->arena;
            continue;
        }
        CUipcMemHandle h;
        memcpy(&h, (const char *)handles + (size_t)p * 64, 64);
        CUresult r = c->drv->cuIpcOpenMemHandle_v2(&s->peer_base[p], h, CU_IPC_MEM_LAZY_ENABLE_PEER_ACCESS);
        if (r != CUDA_SUCCESS) {
            for (int q = 0; q < p; q++)
                if (q != s->tp_rank && s->peer_base[q]) c->drv->cuIpcCloseMemHandle(s->peer_base[q]);
            memset(s->peer_base, 0, sizeof s->peer_base);
            return (int32_t)r;
        }
    }
    // Counter barrier if every peer takes native atomics from this GPU (NVLink), else flags.
    s->tp_counter = qm_env_int("QM_TP_BARRIER_FLAGS", 0) == 0;
    CUdevice me = 0;
    if (c->drv->cuDeviceGet(&me, c->device) != CUDA_SUCCESS) s->tp_counter = false;
    for (int p = 0; p < s->tp_world && s->tp_counter; p++) {
        if (p == s->tp_rank) continue;
        int ordinal = -1, native = 0;
        CUdevice peer = 0;
        if (c->drv->cuPointerGetAttribute(&ordinal, CU_POINTER_ATTRIBUTE_DEVICE_ORDINAL, s->peer_base[p]) != CUDA_SUCCESS ||
            c->drv->cuDeviceGet(&peer, ordinal) != CUDA_SUCCESS ||
            c->drv->cuDeviceGetP2PAttribute(&native, CU_DEVICE_P2P_ATTRIBUTE_NATIVE_ATOMIC_SUPPORTED, me, peer) != CUDA_SUCCESS ||
            !native)
            s->tp_counter = false;
    }
    s->peers_open = true;
    s->peers_ipc = true;
    return QM_OK;
}

// Base address and size of the tensor-parallel activation arena, for callers that drive all GPUs from
// one process and hand the peers' arenas over as plain device pointers (qm_stack_set_peer_pointers).
extern "C" int32_t qm_stack_arena(qm_ctx *c, qm_stack *s, uint64_t *base, int64_t *bytes) {
    CHECK_CTX(c);
    if (!stack_check(s) || !base || !bytes || s->tp_world < 2) return QM_ERR_ARG;
    *base = (uint64_t)s->arena;
    *bytes = (int64_t)s->arena_bytes;
    return QM_OK;
}

// Single-process form of qm_stack_set_peers: bases[p] = the arena of rank p as this process addresses
// it (peer access between the devices enabled by the caller, the reference's
// Context.EnablePeerAccess, nvidia/driver/context.gen.go:98). Entry tp_rank is ignored.
extern "C" int32_t qm_stack_set_peer_pointers(qm_ctx *c, qm_stack *s, const uint64_t *bases) {
    CHECK_CTX(c);
    if (!stack_check(s) || !bases || s->tp_world < 2 || s->peers_open) return QM_ERR_ARG;
    for (int p = 0; p < s->tp_world; p++) {
        s->peer_base[p] = p == s->tp_rank ? s->arena : (CUdeviceptr)bases[p];
        if (!s->peer_base[p]) return QM_ERR_ARG;
    }
    s->tp_counter = false;
    s->peers_open = true;
    s->peers_ipc = false;
    return QM_OK;
}

extern "C" int32_t qm_stack_destroy(qm_ctx *c, qm_stack *s) {
    CHECK_CTX(c);
    if (!stack_check(s)) return QM_ERR_ARG;
    CtxGuard g(c);
    DRV(g.rc);
    c->drv->cuStreamSynchronize(c->stream);
    for (QmLayer &ly : s->layer) {
        if (ly.o_parts) c->drv->cuMemFree_v2(ly.o_parts);
        if (ly.dn_parts) c->drv->cuMemFree_v2(ly.dn_parts);
    }
    for (int i = 0; i < 9; i++) {
        if (s->graph[i]) c->drv->cuGraphExecDestroy(s->graph[i]);
        if (s->ops_dev[i]) c->drv->cuMemFree_v2(s->ops_dev[i]);
        if (s->img_dev[i]) c->drv->cuMemFree_v2(s->img_dev[i]);
        if (s->sync_dev[i]) c->drv->cuMemFree_v2(s->sync_dev[i]);
    }
    if (s->tp_world > 1) {
        if (s->peers_open && s->peers_ipc)
            for (int p = 0; p < s->tp_world; p++)
                if (p != s->tp_rank && s->peer_base[p]) c->drv->cuIpcCloseMemHandle(s->peer_base[p]);
        if (s->arena) c->drv->cuMemFree_v2(s->arena);
    } else {
        if (s->h0) c->drv->cuMemFree_v2(s->h0);
        if (s->act) c->drv->cuMemFree_v2(s->act);
    }
    s->magic = 0;
    delete s;
    return QM_OK;
}

extern "C" int32_t qm_stack_set_layer(qm_ctx *c, qm_stack *s, int32_t layer, qm_weight qkv, qm_weight o,
                                      qm_weight gate_up, qm_weight down) {
    CHECK_CTX(c);
    if (!stack_check(s) || layer < 0 || layer >= s->layers) return QM_ERR_ARG;
    QmWeight *w[4] = {qm_weight_from_handle(qkv), qm_weight_from_handle(o), qm_weight_from_handle(gate_up),
                      qm_weight_from_handle(down)};
    for (QmWeight *p : w)
        if (!p) return QM_ERR_ARG;
    // tensor-parallel: every matrix is this rank's slice of the rows
    const int64_t W = s->tp_world;
    int64_t want[4][2] = {{(s->hidden + 2 * s->kv) / W, s->hidden}, {s->hidden / W, s->hidden},
                          {2 * s->ffn / W, s->hidden}, {s->hidden / W, s->ffn}};
    if (s->tp_paired) {   // o and down: all rows of the rank's K columns
        want[1][0] = s->hidden; want[1][1] = s->hidden / W;
        want[3][0] = s->hidden; want[3][1] = s->ffn / W;
    }
    for (int i = 0; i < 4; i++)
        if (w[i]->rows != want[i][0] || w[i]->cols != want[i][1]) return QM_ERR_SHAPE;
    {
        CtxGuard g(c);
        QmLayer &old = s->layer[layer];
        if (old.o_parts || old.dn_parts) c->drv->cuStreamSynchronize(c->stream);
        if (old.o_parts) c->drv->cuMemFree_v2(old.o_parts);
        if (old.dn_parts) c->drv->cuMemFree_v2(old.dn_parts);
    }
    s->layer[layer] = QmLayer{w[0], w[1], w[2], w[3], 0, 0, 0, 0};
    for (int i = 0; i < 9; i++) {
        CtxGuard g(c);
        if (s->graph[i]) c->drv->cuGraphExecDestroy(s->graph[i]);
        s->graph[i] = nullptr;
        if (s->ops_dev[i]) {
            c->drv->cuStreamSynchronize(c->stream);
            c->drv->cuMemFree_v2(s->ops_dev[i]);
            if (s->img_dev[i]) c->drv->cuMemFree_v2(s->img_dev[i]);
            if (s->sync_dev[i]) c->drv->cuMemFree_v2(s->sync_dev[i]);
        }
        s->ops_dev[i] = 0;
        s->img_dev[i] = 0;
        s->sync_dev[i] = 0;
    }
    return QM_OK;
}

// Device pointers of the activation buffers as the last step (of batch m) left them, for
// per-matvec checks: [0]=h0 [m][hidden], [1]=q|k|v outputs of layer 0 [m][hidden+2kv], and of the
// LAST layer [2]=o output, [3]=gate|up output [m][2*ffn], [4]=h [m][hidden]. When the step cut
// the o projection into K parts (qm_stack_parts), [2] is the first of `parts` partial vectors
// [m][hidden], `stride` floats apart, whose sum times the RMS scale of the o projection's input
// is the o output.
extern "C" int32_t qm_stack_buffers(qm_ctx *c, qm_stack *s, uint64_t *ptrs5) {
    CHECK_CTX(c);
    if (!stack_check(s) || !ptrs5) return QM_ERR_ARG;
    const int m = s->last_m > 0 ? s->last_m : 1;
    const LayerBufs last = layer_bufs(s, s->layers - 1, m);
    ptrs5[0] = s->h0;
    ptrs5[1] = layer_bufs(s, 0, m).qkv;
    ptrs5[2] = last.o;
    ptrs5[3] = last.gu;
    ptrs5[4] = h_source(s, m);
    return QM_OK;
}

// info2[0] = K parts of the o projection in the most recent step (1 = whole), info2[1] = floats
// between its partial vectors.
extern "C" int32_t qm_stack_parts(qm_ctx *c, qm_stack *s, int64_t *info2) {
    CHECK_CTX(c);
    if (!stack_check(s) || !info2) return QM_ERR_ARG;
    const int m = s->last_m > 0 ? s->last_m : 1;
    info2[0] = s->last_dd ? s->fused_parts_o[m] : 1;
    info2[1] = layer_bufs(s, s->layers - 1, m).part_stride;
    return QM_OK;
}

// on: 0 = one launch per matvec, issued one by one; 1 = the same launches replayed as a
// captured graph; 2 (default) = the whole step as ONE persistent launch where the format
// and the shapes allow it (Q4_K, activations of the longest K fit in shared memory),
// falling back to 1 otherwise.
extern "C" int32_t qm_stack_use_graph(qm_ctx *c, qm_stack *s, int32_t on) {
    CHECK_CTX(c);
    if (!stack_check(s)) return QM_ERR_ARG;
    s->use_graph = on != 0;
    s->use_fused = on == 2;
    return QM_OK;
}

// Uploads an op list; tensor-parallel stacks get a second copy that addresses the other arena half.
static int32_t upload_ops(qm_ctx *c, qm_stack *s, int m, std::vector<QmOp> &ops) {
    const size_t nops = ops.size();
    if (s->tp_world > 1) {
        const CUdeviceptr lo = s->act, other = s->act_half[s->act == s->act_half[0] ? 1 : 0];
        auto moved = [&](const void *ptr) -> uintptr_t {
            const CUdeviceptr a0 = (CUdeviceptr)(uintptr_t)ptr;
            return (uintptr_t)((a0 >= lo && a0 < lo + s->act_bytes) ? a0 - lo + other : a0);
        };
        for (size_t k = 0; k < nops; k++) {
            QmOp op = ops[k];
            op.x = (const float *)moved(op.x);
            op.x2 = (const float *)moved(op.x2);
            op.y = (float *)moved(op.y);
            op.y2 = (float *)moved(op.y2);
            op.ssq_out = (float *)moved(op.ssq_out);
            op.ssq_in = (const float *)moved(op.ssq_in);
            ops.push_back(op);
        }
        s->fused_half0[m] = s->act == s->act_half[0] ? 0 : 1;   // which half the first copy addresses
    }
    CUdeviceptr dev = 0;
    DRV(c->drv->cuMemAlloc_v2(&dev, ops.size() * sizeof(QmOp)));
    CUresult r = c->drv->cuMemcpyHtoD_v2(dev, ops.data(), ops.size() * sizeof(QmOp));
    if (r != CUDA_SUCCESS) {
        c->drv->cuMemFree_v2(dev);
        return (int32_t)r;
    }
    s->ops_dev[m] = dev;
    s->fused_nops[m] = (int)nops;
    return QM_OK;
}

// The op list of a step for the data-driven kernels (qm_fused_q4k_dd_*): every output buffer is
// filled with the "not yet written" pattern before the launch and consumers poll the words they
// read, so no grid barrier separates dependent matvecs. Needs whole tiles per CTA, no K slices
// and one row tile of mma columns; used below the batch from which activation images win.
// The o and down projections are cut into K parts (QmOp::parts): their CTAs stage a quarter of x
// each and spread over four times as many (tile, part) pieces; the consumer adds the parts up
// while it stages them. QM_ERR_SHAPE when the step does not qualify (the caller then builds the
// barrier form).
static int32_t part_major_copy(qm_ctx *c, const QmWeight *w, int parts, CUdeviceptr *out, int *out_parts) {
    if (*out && *out_parts == parts) return QM_OK;
    if (*out) {
        DRV(c->drv->cuStreamSynchronize(c->stream));
        c->drv->cuMemFree_v2(*out);
        *out = 0;
    }
    DRV(c->drv->cuMemAlloc_v2(out, (size_t)w->qbytes + 64));
    QmPartsArgs a;
    memset(&a, 0, sizeof a);
    a.src = (const uint8_t *)(uintptr_t)w->wq;
    a.dst = (uint8_t *)(uintptr_t)*out;
    a.tiles = (int32_t)((w->rows + 15) / 16);
    a.units = w->units;
    a.ups = w->units / parts;
    *out_parts = parts;
    return qm_launch(c, QM_K_REPACK_PARTS, (unsigned)c->sm_count * 8, 1, 256, 0, &a, false);
}

static int32_t build_fused_dd(qm_ctx *c, qm_stack *s, int m) {
    // up to three rows, and five to eight (two column tiles; single GPU); four rows run with activation images
    const bool two_tiles = m > 4 && s->tp_world == 1 && qm_env_int("QM_DD8", 1) != 0;
    if ((m >= qm_env_int("QM_IMAGE_MIN_M", 4) && !two_tiles) || qm_env_int("QM_DD", 1) == 0) return QM_ERR_SHAPE;
    const int grid = qm_fused_grid(c);
    // The down projection (long K: its CTAs would each quantize all 2 x 14336 activations) runs in
    // four K parts. The o projection stays whole by default: its x is short, and every part adds a
    // vector that each CTA of the consumer polls and loads.
    auto parts_for = [&](const QmWeight *w, int want) {
        for (int k = QM_MAX_PARTS; k > 1; k >>= 1)
            if (k <= want && w->units % k == 0 && grid % k == 0) return k;
        return 1;
    };
    const int want_o = qm_env_int("QM_PARTS_O", 1), want_dn = qm_env_int("QM_PARTS_DN", QM_MAX_PARTS);
    int max_units = 0, So = QM_MAX_PARTS, Sd = QM_MAX_PARTS;
    for (int L = 0; L < s->layers; L++) {
        const QmLayer &ly = s->layer[L];
        if (!ly.qkv) return QM_ERR_STATE;
        const QmWeight *ws[4] = {ly.qkv, ly.o, ly.gu, ly.dn};
        for (const QmWeight *w : ws)
            if (w->fmt != QM_FMT_Q4_K) return QM_ERR_FORMAT;
        So = std::min(So, parts_for(ly.o, want_o));
        Sd = std::min(Sd, parts_for(ly.dn, want_dn));
    }
    for (int L = 0; L < s->layers; L++) {
        const QmLayer &ly = s->layer[L];
        max_units = std::max({max_units, (int)ly.qkv->units, (int)ly.gu->units, (int)ly.o->units / So, (int)ly.dn->units / Sd});
    }
    QmFusedPlan p;
    if (qm_plan_fused(c, m, max_units, false, &p) != QM_OK) return QM_ERR_SHAPE;
    int kernel = -1;
    if (p.nt == 1 && p.consumers == 16 && p.depth >= 2 && p.depth <= 4)
        kernel = (p.cpm == 4 ? QM_K_FUSED_Q4K_DD_C4D2 : QM_K_FUSED_Q4K_DD_C2D2) + (p.depth - 2);
    if (p.nt == 2 && p.consumers == 16 && p.depth >= 2) {
        if (p.depth > 3) {   // the two-tile kernels exist with two and three stages
            p.smem -= (p.depth - 3) * 16 * QM_Q4K_ITEM_BYTES;
            p.depth = 3;
        }
        kernel = QM_K_FUSED_Q4K_DD_N2D2 + (p.depth - 2);
    }
    if (kernel < 0) return QM_ERR_SHAPE;
    for (int L = 0; L < s->layers; L++) {
        QmLayer &ly = s->layer[L];
        int32_t rc = QM_OK;
        if (So > 1) rc = part_major_copy(c, ly.o, So, &ly.o_parts, &ly.o_nparts);
        if (!rc && Sd > 1) rc = part_major_copy(c, ly.dn, Sd, &ly.dn_parts, &ly.dn_nparts);
        if (rc) return rc;
    }

    // One copy of the op list per CTA group; the copies differ in the ops that run in parts.
    const int ngroups = std::max(So, Sd);
    std::vector<QmOp> ops;
    const int64_t qkv_ld = s->hidden + 2 * s->kv;
    const bool tp = s->tp_world > 1;
    const size_t R = (size_t)s->tp_rank * 4;
    for (int g = 0; g < ngroups; g++) {
        // Tensor-parallel: every matrix is sliced by rows (GPU r of g holds rows [r*N/g, (r+1)*N/g)); y
        // points at this rank's rows of the full-width output and the results go to every GPU's arena.
        auto add = [&](const QmWeight *w, CUdeviceptr parts_copy, CUdeviceptr x, CUdeviceptr x2, int64_t ldx, CUdeviceptr y,
                       int64_t ldy, uint32_t xop, bool first, int parts, int64_t y_part_stride, CUdeviceptr ssq_out) -> QmOp & {
            QmOp op;
            const int ups = w->units / parts;
            qm_fill_op(c, p, w, x, x2, ldx, y + R * w->rows, ldy, xop, !first, 0, ups, 0, &op);
            if (parts > 1) {
                const int per = ngroups / parts;          // CTA groups that share one part
                const int part = g / per, G = grid / ngroups * per;
                op.wq = (const uint8_t *)(uintptr_t)(parts_copy + (size_t)part * op.tiles * ups * QM_Q4K_ITEM_BYTES);
                op.units_total = ups;                     // the part's items are contiguous in the copy
                op.unit0 = part * ups;                    // ... and cover these K units of x
                op.y = (float *)((uintptr_t)op.y + (size_t)part * y_part_stride * 4);
                op.parts = parts;
                op.part = part;
                op.cta0 = part * G;
                op.nctas = G;
                op.q = op.tiles / G;
                op.rem = op.tiles % G;
                op.ssq_out = (float *)(uintptr_t)ssq_out;
            }
            op.tp_shared = tp ? 1 : 0;
            ops.push_back(op);
            return ops.back();
        };
        auto consumes = [&](QmOp &op, int parts, int64_t stride, CUdeviceptr ssq, const QmWeight *producer) {
            op.x_parts = parts;
            op.x_part_stride = stride;
            if (parts > 1) {
                op.ssq_in = (const float *)(uintptr_t)ssq;
                op.ssq_in_inv_cols = 1.f / (float)producer->cols;
                op.ssq_in_eps = 1e-6f;
            }
        };
        for (int L = 0; L < s->layers; L++) {
            const QmLayer &ly = s->layer[L];
            const LayerBufs b = layer_bufs(s, L, m);
            QmOp &qkv = add(ly.qkv, 0, L == 0 ? s->h0 : layer_bufs(s, L - 1, m).dn, 0, s->hidden, b.qkv, qkv_ld,
                            QM_XOP_RMSNORM, L == 0, 1, 0, 0);
            if (L > 0) consumes(qkv, Sd, b.part_stride, layer_bufs(s, L - 1, m).ssq_dn, s->layer[L - 1].dn);
            add(ly.o, ly.o_parts, b.qkv, 0, qkv_ld, b.o, s->hidden, QM_XOP_RMSNORM, false, So, b.part_stride, b.ssq_o);
            QmOp &gu = add(ly.gu, 0, b.o, 0, s->hidden, b.gu, 2 * s->ffn, QM_XOP_RMSNORM, false, 1, 0, 0);
            consumes(gu, So, b.part_stride, b.ssq_o, ly.o);
            add(ly.dn, ly.dn_parts, b.gu, b.gu + (size_t)s->ffn * 4, 2 * s->ffn, b.dn, s->hidden, QM_XOP_ADD_RMSNORM, false,
                Sd, b.part_stride, b.ssq_dn);
        }
    }
    for (const QmOp &op : ops)
        if ((int64_t)op.tiles * op.units >= (1ll << 31)) return QM_ERR_SHAPE;
    CUdeviceptr sync = 0;
    DRV(c->drv->cuMemAlloc_v2(&sync, 256));
    int32_t rc = upload_ops(c, s, m, ops);
    if (rc) {
        c->drv->cuMemFree_v2(sync);
        return rc;
    }
    s->fused_nops[m] = (int)(ops.size() / (size_t)ngroups / (tp ? 2 : 1));
    s->fused_ngroups[m] = ngroups;
    s->img_dev[m] = 0;
    s->sync_dev[m] = sync;
    s->sync_bytes[m] = 256;
    s->img_units[m] = max_units;
    s->fused_ncross[m] = 1;
    s->fused_img[m] = false;
    s->fused_dd[m] = true;
    s->fused_dd_kernel[m] = kernel;
    s->fused_parts_o[m] = So;
    s->fused_parts_dn[m] = Sd;
    s->fused_plan[m] = p;
    return QM_OK;
}

// The op list of a paired tensor-parallel step (see qm_stack_create_tp_paired), data-driven form. Per layer:
//   q|k|v  rows of this rank   x = the W partial vectors of the previous down projection   -> q slice (own arena),
//                                                                                              k|v slice (all arenas)
//   o      K part of this rank x = the rank's own q slice (no exchange)                     -> partial vector r (all)
//   gate|up rows of this rank  x = the W partial vectors of o                               -> own arena only
//   down   K part of this rank x = the rank's own gate and up slices (no exchange)          -> partial vector r (all)
// A K part leaves its products without the RMS scale of its input and publishes its sum of squares; the consumer
// adds the W vectors in rank order and corrects its epsilon (QmOp::parts).
static int32_t build_fused_paired(qm_ctx *c, qm_stack *s, int m) {
    if (m > 4) return QM_ERR_SHAPE;
    const int W = s->tp_world, r = s->tp_rank, grid = qm_fused_grid(c);
    for (int L = 0; L < s->layers; L++) {
        const QmLayer &ly = s->layer[L];
        if (!ly.qkv) return QM_ERR_STATE;
        const QmWeight *ws[4] = {ly.qkv, ly.o, ly.gu, ly.dn};
        for (const QmWeight *w : ws)
            if (w->fmt != QM_FMT_Q4_K) return QM_ERR_FORMAT;
    }
    // A rank's down part can be cut further into S parts run by S groups of its CTAs (a CTA then stages a 1/(W*S)
    // of gate and up, not 1/W), as long as the consumer has at most parts_cap vectors to add. Off by default:
    // on 2 GPUs one part per GPU measured 0.97 ms per step, two 0.98, four 1.07 — every further vector costs the
    // consumers more than the shorter staging saves (QM_PAIRED_PARTS_DN).
    const int dn_units = (s->ffn / W) / 256;
    int S = 1;
    for (int k = QM_MAX_PARTS; k > 1; k >>= 1)
        if (k <= qm_env_int("QM_PAIRED_PARTS_DN", 1) && W * k <= s->parts_cap && dn_units % k == 0 && grid % k == 0) {
            S = k;
            break;
        }
    const int max_units = std::max(s->hidden / 256, dn_units / S);
    QmFusedPlan p;
    if (qm_plan_fused(c, m, max_units, false, &p) != QM_OK || p.nt != 1 || p.consumers != 16 || p.depth < 2 || p.depth > 4)
        return QM_ERR_SHAPE;
    const int kernel = (p.cpm == 4 ? QM_K_FUSED_Q4K_DD_C4D2 : QM_K_FUSED_Q4K_DD_C2D2) + (p.depth - 2);
    if (S > 1)
        for (int L = 0; L < s->layers; L++) {
            QmLayer &ly = s->layer[L];
            const int32_t rc = part_major_copy(c, ly.dn, S, &ly.dn_parts, &ly.dn_nparts);
            if (rc) return rc;
        }
    std::vector<QmOp> ops;
    const int64_t qkv_ld = s->hidden + 2 * s->kv;
    const int64_t q_rows = s->hidden / W, kv_rows = 2 * s->kv / W, f_rows = s->ffn / W;
    auto add = [&](const QmWeight *w, CUdeviceptr x, CUdeviceptr x2, int64_t ldx, CUdeviceptr y, int64_t ldy, uint32_t xop,
                   bool first, int unit0, int units) -> QmOp & {
        QmOp op;
        qm_fill_op(c, p, w, x, x2, ldx, y, ldy, xop, !first, unit0, units, 0, &op);
        ops.push_back(op);
        return ops.back();
    };
    auto consumes = [&](QmOp &op, int parts, int64_t stride, CUdeviceptr ssq, int64_t producer_cols) {
        op.x_parts = parts;
        op.x_part_stride = stride;
        op.ssq_in = (const float *)(uintptr_t)ssq;
        op.ssq_in_inv_cols = 1.f / (float)producer_cols;
        op.ssq_in_eps = 1e-6f;
    };
    for (int g = 0; g < S; g++)   // one copy of the list per CTA group; the copies differ in the down op only
        for (int L = 0; L < s->layers; L++) {
            const QmLayer &ly = s->layer[L];
            const LayerBufs b = layer_bufs(s, L, m);
            // q|k|v: q rows into this arena only (the rank's own o part reads them), k|v rows into every arena
            QmOp &qkv = add(ly.qkv, L == 0 ? s->h0 : layer_bufs(s, L - 1, m).dn, 0, s->hidden, b.qkv + (size_t)r * q_rows * 4,
                            qkv_ld, QM_XOP_RMSNORM, L == 0, 0, ly.qkv->units);
            qkv.split_row = (int32_t)q_rows;
            qkv.y2 = (float *)(uintptr_t)(b.qkv + (size_t)(s->hidden + r * kv_rows) * 4);
            qkv.tp_shared = 2;
            if (L > 0) consumes(qkv, W * S, b.part_stride, layer_bufs(s, L - 1, m).ssq_dn, s->ffn);
            // o: the K columns that multiply this rank's q slice; one part per GPU
            QmOp &o = add(ly.o, b.qkv, 0, qkv_ld, b.o + (size_t)r * b.part_stride * 4, s->hidden, QM_XOP_RMSNORM, false,
                          (int)(r * q_rows / 256), ly.o->units);
            o.parts = W;
            o.part = r;
            o.ssq_out = (float *)(uintptr_t)b.ssq_o;
            o.tp_shared = 1;
            // gate|up: gate rows then up rows of this rank, for its own down parts only
            QmOp &gu = add(ly.gu, b.o, 0, s->hidden, b.gu + (size_t)r * f_rows * 4, 2 * s->ffn, QM_XOP_RMSNORM, false, 0,
                           ly.gu->units);
            gu.split_row = (int32_t)f_rows;
            gu.y2 = (float *)(uintptr_t)(b.gu + (size_t)(s->ffn + r * f_rows) * 4);
            gu.tp_shared = 0;
            consumes(gu, W, b.part_stride, b.ssq_o, s->hidden);
            // down: the K columns that multiply this rank's gate and up slices, part r*S + g of W*S by CTA group g
            const int ups = dn_units / S, part = r * S + g, G = grid / S;
            QmOp &dn = add(ly.dn, b.gu, b.gu + (size_t)s->ffn * 4, 2 * s->ffn, b.dn + (size_t)part * b.part_stride * 4,
                           s->hidden, QM_XOP_ADD_RMSNORM, false, (int)(r * f_rows / 256) + g * ups, ups);
            if (S > 1) dn.wq = (const uint8_t *)(uintptr_t)(ly.dn_parts + (size_t)g * dn.tiles * ups * QM_Q4K_ITEM_BYTES);
            dn.units_total = ups;
            dn.parts = W * S;
            dn.part = part;
            dn.cta0 = g * G;
            dn.nctas = G;
            dn.q = dn.tiles / G;
            dn.rem = dn.tiles % G;
            dn.ssq_out = (float *)(uintptr_t)b.ssq_dn;
            dn.tp_shared = 1;
        }
    for (const QmOp &op : ops)
        if ((int64_t)op.tiles * op.units >= (1ll << 31)) return QM_ERR_SHAPE;
    CUdeviceptr sync = 0;
    DRV(c->drv->cuMemAlloc_v2(&sync, 256));
    int32_t rc = upload_ops(c, s, m, ops);
    if (rc) {
        c->drv->cuMemFree_v2(sync);
        return rc;
    }
    s->fused_nops[m] = (int)(ops.size() / (size_t)S / 2);   // per list; upload_ops appended the copies for the other arena half
    s->fused_ngroups[m] = S;
    s->img_dev[m] = 0;
    s->sync_dev[m] = sync;
    s->sync_bytes[m] = 256;
    s->img_units[m] = max_units;
    s->fused_ncross[m] = 1;
    s->fused_img[m] = false;
    s->fused_dd[m] = true;
    s->fused_dd_kernel[m] = kernel;
    s->fused_parts_o[m] = W;
    s->fused_parts_dn[m] = W * S;
    s->fused_plan[m] = p;
    return QM_OK;
}

// Builds the op list of a whole step for batch m; QM_ERR_SHAPE/FORMAT when the step cannot
// run as one launch.
static int32_t build_fused(qm_ctx *c, qm_stack *s, int m) {
    int max_units = 0;
    for (int L = 0; L < s->layers; L++) {
        const QmLayer &ly = s->layer[L];
        if (!ly.qkv) return QM_ERR_STATE;
        const QmWeight *ws[4] = {ly.qkv, ly.o, ly.gu, ly.dn};
        for (const QmWeight *w : ws) {
            if (w->fmt != QM_FMT_Q4_K) return QM_ERR_FORMAT;
            max_units = std::max(max_units, (int)w->units);
        }
    }
    QmFusedPlan p;
    int32_t rc = qm_plan_fused(c, m, max_units, true, &p);
    if (rc) return rc;
    // One group of ops per matrix: a matrix whose K units exceed what a CTA can hold of the
    // activations is cut into K slices, the later ones adding to y.
    std::vector<QmOp> ops;
    std::vector<int> group_first, group_last;
    auto add_matvec = [&](const QmWeight *w, CUdeviceptr x, CUdeviceptr x2, int64_t ldx, CUdeviceptr y, int64_t ldy,
                          uint32_t xop, bool first, bool shared) {
        const int nslices = (w->units + p.max_units - 1) / p.max_units;
        const int ups = (w->units + nslices - 1) / nslices;
        group_first.push_back((int)ops.size());
        for (int sl = 0; sl < nslices; sl++) {
            QmOp op;
            const int u0 = sl * ups, n = std::min(ups, (int)w->units - u0);
            qm_fill_op(c, p, w, x, x2, ldx, y, ldy, xop, !(first && sl == 0), u0, n, sl > 0, &op);
            op.tp_shared = shared ? 1 : 0;
            ops.push_back(op);
        }
        group_last.push_back((int)ops.size() - 1);
    };
    const int64_t qkv_ld = s->hidden + 2 * s->kv;
    for (int L = 0; L < s->layers; L++) {
        const QmLayer &ly = s->layer[L];
        const LayerBufs b = layer_bufs(s, L, m);
        const CUdeviceptr x0 = L == 0 ? s->h0 : layer_bufs(s, L - 1, m).dn;
        // Tensor-parallel: every matrix is sliced by rows (GPU r of g holds rows [r*N/g, (r+1)*N/g));
        // y points at this rank's rows of the full-width output and the results go to every GPU's arena.
        const bool tp = s->tp_world > 1;
        const size_t R = (size_t)s->tp_rank * 4;
        add_matvec(ly.qkv, x0, 0, s->hidden, b.qkv + R * ly.qkv->rows, qkv_ld, QM_XOP_RMSNORM, L == 0, tp);
        add_matvec(ly.o, b.qkv, 0, qkv_ld, b.o + R * ly.o->rows, s->hidden, QM_XOP_RMSNORM, false, tp);
        add_matvec(ly.gu, b.o, 0, s->hidden, b.gu + R * ly.gu->rows, 2 * s->ffn, QM_XOP_RMSNORM, false, tp);
        add_matvec(ly.dn, b.gu, b.gu + (size_t)s->ffn * 4, 2 * s->ffn, b.dn + R * ly.dn->rows,
                   s->hidden, QM_XOP_ADD_RMSNORM, false, tp);
    }
    for (const QmOp &op : ops)
        if ((int64_t)op.tiles * op.units >= (1ll << 31)) return QM_ERR_SHAPE;
    // every unsliced op but the first writes a buffer that the op before it does not touch
    // (ops shared between GPUs keep whole tiles per CTA: their outputs are plain stores to every GPU)
    for (QmOp &op : ops) op.parts = op.x_parts = 1;
    for (size_t k = 1; k < ops.size(); k++)
        if (ops[k].units == ops[k].units_total && !ops[k].tp_shared) qm_balance_op(c, &ops[k]);
    // barriers over all GPUs in one launch: after every shared op, and the one that ends the launch
    int ncross = 1;
    for (size_t k = 1; k < ops.size(); k++) ncross += ops[k - 1].tp_shared && ops[k].barrier ? 1 : 0;

    // Activation images: the last op of a matrix quantizes the next matrix's x as its outputs
    // complete, so that the CTAs of the next op copy the quantized form instead of each
    // quantizing all of x. Two images alternate (the readers of one are a grid barrier away from
    // its next writers); one completion counter per (matrix, unit), zeroed before each launch.
    const int NT = p.nt, NL = p.cpm == 4 ? 3 : 2, P = m * NL;
    const int img_units = max_units;
    const size_t img_bytes = (size_t)P * (img_units * 256 + 64) + (size_t)img_units * 8 * NT * 20 + (size_t)img_units * 32;
    const size_t img_stride = (img_bytes + 255) & ~(size_t)255;
    const size_t ngroups = group_first.size();
    const size_t sync_bytes = 256 + ngroups * (size_t)img_units * 4;
    CUdeviceptr img = 0, sync = 0;
    CUresult r = c->drv->cuMemAlloc_v2(&img, 2 * img_stride);
    if (r == CUDA_SUCCESS) r = c->drv->cuMemAlloc_v2(&sync, sync_bytes);
    if (r == CUDA_SUCCESS) r = c->drv->cuMemsetD8Async(img, 0, 2 * img_stride, c->stream);
    // With up to three activation rows the per-CTA quantization is as cheap as or cheaper than the
    // producers' fences and counters (measured per step, batch 1: 1.83 ms against 2.30 ms; batch 2:
    // 2.09 against 2.33; batch 3: 2.34 against 2.37); from four rows on the image wins (batch 4:
    // 2.46 ms against 2.63 ms; batch 8: 3.52 ms against 5.93 ms).
    bool uses_img = false;
    const int min_m = qm_env_int("QM_IMAGE_MIN_M", 4), min_units = qm_env_int("QM_IMAGE_MIN_UNITS", 1 << 30);
    if (r == CUDA_SUCCESS && !qm_env_int("QM_NO_IMAGE", 0) && s->tp_world == 1) {
        for (size_t k = 0; k + 1 < ngroups; k++) {
            QmOp &prod = ops[group_last[k]];
            const QmOp &cons = ops[group_first[k + 1]];
            const bool two = cons.xop == QM_XOP_ADD_RMSNORM;
            if (m < min_m && cons.units_total < min_units) continue;
            if (cons.xop > QM_XOP_ADD_RMSNORM || (cons.cols & 255) || cons.x != prod.y || cons.ldx != prod.ldy) continue;
            if (two && cons.x2 != prod.y + cons.cols) continue;
            if ((int64_t)cons.cols * (two ? 2 : 1) > prod.rows) continue;
            prod.q_img = (uint8_t *)(uintptr_t)(img + ((k + 1) & 1) * img_stride);
            prod.q_cnt = (unsigned int *)(uintptr_t)(sync + 256 + (k + 1) * (size_t)img_units * 4);
            prod.q_half_tiles = cons.cols / 16;
            prod.q_halves = two ? 2 : 1;
            for (int o = group_first[k + 1]; o <= group_last[k + 1]; o++) ops[o].img = prod.q_img;
            uses_img = true;
        }
    }
    if (r != CUDA_SUCCESS) {
        if (img) c->drv->cuMemFree_v2(img);
        if (sync) c->drv->cuMemFree_v2(sync);
        return (int32_t)r;
    }
    rc = upload_ops(c, s, m, ops);
    if (rc) {
        c->drv->cuMemFree_v2(img);
        c->drv->cuMemFree_v2(sync);
        return rc;
    }
    s->img_dev[m] = img;
    s->sync_dev[m] = sync;
    s->sync_bytes[m] = sync_bytes;
    s->img_units[m] = img_units;
    s->fused_ncross[m] = ncross;
    s->fused_img[m] = uses_img;
    s->fused_dd[m] = false;
    s->fused_dd_kernel[m] = -1;
    s->fused_parts_o[m] = s->fused_parts_dn[m] = 1;
    s->fused_ngroups[m] = 1;
    s->fused_plan[m] = p;
    return QM_OK;
}

// The last layer's down projection, when it ran in K parts: h = c * (sum of the partial vectors), c the RMS
// scale of its input, into s->h_sum.
static int32_t sum_last_parts(qm_ctx *c, qm_stack *s, int m) {
    if (s->fused_parts_dn[m] <= 1) return QM_OK;
    const LayerBufs b = layer_bufs(s, s->layers - 1, m);
    QmSumPartsArgs a;
    memset(&a, 0, sizeof a);
    a.parts = (const float *)(uintptr_t)b.dn;
    a.ssq = (const float *)(uintptr_t)b.ssq_dn;
    a.out = (float *)(uintptr_t)s->h_sum;
    a.part_stride = b.part_stride;
    a.ld_in = s->hidden;
    a.ld_out = s->hidden;
    a.nparts = s->fused_parts_dn[m];
    a.m = m;
    a.n = s->hidden;
    a.inv_cols = 1.f / (float)s->ffn;
    a.eps = 1e-6f;
    return qm_launch(c, QM_K_SUM_PARTS, (unsigned)std::min(148, (m * s->hidden + 255) / 256), 1, 256, 0, &a, false);
}

// Where the most recent step left h [m][hidden].
static CUdeviceptr h_source(const qm_stack *s, int m) {
    if (s->last_dd && s->fused_parts_dn[m] > 1) return s->h_sum;
    return layer_bufs(s, s->layers - 1, m).dn;
}

static int32_t launch_fused(qm_ctx *c, qm_stack *s, int m) {
    const QmFusedPlan &p = s->fused_plan[m];
    QmFusedArgs a;
    memset(&a, 0, sizeof a);
    a.ops = (const QmOp *)(uintptr_t)s->ops_dev[m];
    a.status = (unsigned int *)(uintptr_t)c->status_dev;
    a.grid_bar = (unsigned int *)(uintptr_t)s->sync_dev[m];
    a.nops = s->fused_nops[m];
    a.ngroups = s->fused_ngroups[m];
    a.img_units = s->img_units[m];
    a.m = m;
    a.consumers = p.consumers;
    a.depth = p.depth;
    a.max_units = p.max_units;
    a.cpm = p.cpm;
#ifdef QM_DEBUG
    a.debug = qm_env_int("QM_DEBUG_SKIP", 0);
    a.debug_slot = qm_env_int("QM_DEBUG_OP", 0);
#endif
    a.wait_cycles = qm_wait_cycles();
    DRV(c->drv->cuMemsetD32Async(s->sync_dev[m], 0, s->sync_bytes[m] / 4, c->stream));
    // cooperative: every CTA must be resident (grid barriers, or CTAs polling each other's outputs)
    if (s->tp_world > 1) {
        if (!s->peers_open) return QM_ERR_STATE;
        const bool second = (s->act == s->act_half[0] ? 0 : 1) != s->fused_half0[m];
        a.ops = (const QmOp *)(uintptr_t)(s->ops_dev[m] + (second ? (size_t)a.nops * a.ngroups * sizeof(QmOp) : 0));
        a.tp_world = s->tp_world;
        a.tp_rank = s->tp_rank;
        a.tp_epoch0 = s->tp_epoch;
        a.tp_flags = (unsigned int *)(uintptr_t)(s->arena + s->flags_off);
        for (int q = 0; q < s->tp_world; q++) a.peer_delta[q] = (int64_t)s->peer_base[q] - (int64_t)s->arena;
        // the half this step does not use is refilled for the next step; its last readers and writers
        // finished with the step before this one (every launch ends with a barrier over the GPUs)
        // (only the part the last step in that half wrote: a step of batch m touches the first
        // layers*m rows' worth of the half)
        const int cur = s->act == s->act_half[0] ? 0 : 1, other = cur ^ 1;
        if (s->half_m[other] > 0) {
            DRV(c->drv->cuMemsetD32Async(s->act_half[other], 0xFFFFFFFFu,
                                         (size_t)s->layers * layer_floats(s, s->half_m[other]), c->stream));
            s->half_m[other] = 0;
        }
        s->half_m[cur] = m;
        if (s->fused_dd[m]) {
            a.tp_counter = 0;
            s->tp_epoch += 1;   // one barrier over the GPUs per launch
            int32_t rc = qm_launch_ex(c, s->fused_dd_kernel[m] + (QM_K_FUSED_Q4K_DD_C4D2_TP - QM_K_FUSED_Q4K_DD_C4D2),
                                      (unsigned)qm_fused_grid(c), (unsigned)p.consumers * 32, (unsigned)p.smem, &a, false, true);
            return rc ? rc : sum_last_parts(c, s, m);
        }
        a.tp_counter = s->tp_counter ? 1u : 0u;
        // the epoch counts the launch's barriers over all GPUs; the counter form counts CTA arrivals
        s->tp_epoch += (unsigned int)s->fused_ncross[m] * (s->tp_counter ? (unsigned int)(qm_fused_grid(c) * s->tp_world) : 1u);
        return qm_launch_ex(c, p.nt == 1 ? QM_K_FUSED_Q4K_NT1_TP : QM_K_FUSED_Q4K_NT2_TP, (unsigned)qm_fused_grid(c),
                            (unsigned)p.consumers * 32, (unsigned)p.smem, &a, false, true);
    }
    if (s->fused_dd[m]) {
        // every output word of the step starts as "not yet written" (all ones)
        const size_t bytes = (size_t)(layer_bufs(s, s->layers, m).qkv - s->act);
        DRV(c->drv->cuMemsetD32Async(s->act, 0xFFFFFFFFu, bytes / 4, c->stream));
        int32_t rc = qm_launch_ex(c, s->fused_dd_kernel[m], (unsigned)qm_fused_grid(c), (unsigned)p.consumers * 32,
                                  (unsigned)p.smem, &a, false, true);
        return rc ? rc : sum_last_parts(c, s, m);
    }
    const int kern = s->fused_img[m] ? (p.nt == 1 ? QM_K_FUSED_Q4K_NT1_IMG : QM_K_FUSED_Q4K_NT2_IMG)
                                     : (p.nt == 1 ? QM_K_FUSED_Q4K_NT1 : QM_K_FUSED_Q4K_NT2);
    return qm_launch_ex(c, kern, (unsigned)qm_fused_grid(c),
                        (unsigned)p.consumers * 32, (unsigned)p.smem, &a, false, true);
}

// The launches of one step for batch m, in stream order.
static int32_t enqueue_layers(qm_ctx *c, qm_stack *s, int m, int upto_layers) {
    const int64_t qkv_ld = s->hidden + 2 * s->kv;
    const uint32_t F = QM_FLAG_PDL;
    for (int L = 0; L < upto_layers; L++) {
        const QmLayer &ly = s->layer[L];
        if (!ly.qkv) return QM_ERR_STATE;
        const LayerBufs b = layer_bufs(s, L, m);
        const CUdeviceptr x0 = L == 0 ? s->h0 : layer_bufs(s, L - 1, m).dn;
        int32_t rc = qm_matvec_launch(c, ly.qkv, x0, 0, m, s->hidden, b.qkv, qkv_ld,
                                      QM_XOP_RMSNORM | F, c->partials_dev, c->tickets_dev);
        if (!rc) rc = qm_matvec_launch(c, ly.o, b.qkv, 0, m, qkv_ld, b.o, s->hidden, QM_XOP_RMSNORM | F,
                                       c->partials_dev, c->tickets_dev);
        if (!rc) rc = qm_matvec_launch(c, ly.gu, b.o, 0, m, s->hidden, b.gu, 2 * s->ffn,
                                       QM_XOP_RMSNORM | F, c->partials_dev, c->tickets_dev);
        if (!rc) rc = qm_matvec_launch(c, ly.dn, b.gu, b.gu + (size_t)s->ffn * 4, m, 2 * s->ffn,
                                       b.dn, s->hidden, QM_XOP_ADD_RMSNORM | F, c->partials_dev,
                                       c->tickets_dev);
        if (rc) return rc;
    }
    return QM_OK;
}

// The data-driven form where the step qualifies, else the form with grid barriers.
static int32_t build_any(qm_ctx *c, qm_stack *s, int m) {
    if (s->tp_paired) return build_fused_paired(c, s, m);
    int32_t rc = build_fused_dd(c, s, m);
    if (rc == QM_ERR_SHAPE) rc = build_fused(c, s, m);
    return rc;
}

static int32_t step_device(qm_ctx *c, qm_stack *s, int m) {
    s->last_m = m;
    s->last_dd = false;
    if (s->tp_world > 1) {   // tensor-parallel steps exist as the one fused launch only
        int32_t rc = s->ops_dev[m] ? QM_OK : build_any(c, s, m);
        if (rc) return rc;
        s->last_dd = s->fused_dd[m];
        s->cur_half ^= 1;    // this step's half: the one refilled during the step before
        s->act = s->act_half[s->cur_half];
        return launch_fused(c, s, m);
    }
    if (s->use_graph && s->use_fused) {
        int32_t rc = s->ops_dev[m] ? QM_OK : build_any(c, s, m);
        if (rc == QM_OK) {
            s->last_dd = s->fused_dd[m];
            return launch_fused(c, s, m);
        }
        if (rc != QM_ERR_SHAPE && rc != QM_ERR_FORMAT) return rc;
    }
    if (!s->use_graph) return enqueue_layers(c, s, m, s->layers);
    if (!s->graph[m]) {
        QmDriver *d = c->drv;
        DRV(d->cuStreamBeginCapture_v2(c->stream, CU_STREAM_CAPTURE_MODE_THREAD_LOCAL));
        const int64_t before = c->launches;
        int32_t rc = enqueue_layers(c, s, m, s->layers);
        c->launches = before;  // captured, not launched
        CUgraph graph = nullptr;
        CUresult r = d->cuStreamEndCapture(c->stream, &graph);
        if (rc) {
            if (graph) d->cuGraphDestroy(graph);
            return rc;
        }
        DRV(r);
        r = d->cuGraphInstantiateWithFlags(&s->graph[m], graph, 0);
        d->cuGraphDestroy(graph);
        DRV(r);
    }
    DRV(c->drv->cuGraphLaunch(s->graph[m], c->stream));
    c->launches += 4 * (int64_t)s->layers;
    return QM_OK;
}

// x_dev [m][ldx] float32 -> h_out_dev [m][ldh] float32 (the last layer's down-projection
// output). Asynchronous on the context's stream.
extern "C" int32_t qm_stack_step(qm_ctx *c, qm_stack *s, uint64_t x_dev, int32_t m, int64_t ldx,
                                 uint64_t h_out_dev, int64_t ldh) {
    CHECK_CTX(c);
    if (!stack_check(s) || !x_dev) return QM_ERR_ARG;
    if (m < 1 || m > s->m_max || ldx < s->hidden || (h_out_dev && ldh < s->hidden)) return QM_ERR_SHAPE;
    CtxGuard g(c);
    DRV(g.rc);
    for (int j = 0; j < m; j++)
        DRV(c->drv->cuMemcpyDtoDAsync_v2(s->h0 + (size_t)j * s->hidden * 4, x_dev + (size_t)j * ldx * 4,
                                         (size_t)s->hidden * 4, c->stream));
    int32_t rc = step_device(c, s, m);
    if (rc) return rc;
    if (h_out_dev)
        for (int j = 0; j < m; j++)
            DRV(c->drv->cuMemcpyDtoDAsync_v2(h_out_dev + (size_t)j * ldh * 4, h_source(s, m) + (size_t)j * s->hidden * 4,
                                             (size_t)s->hidden * 4, c->stream));
    return QM_OK;
}

// Host-buffer form: copies x in, runs the step, copies h [m][hidden] and (when kv_host is not
// null) every layer's k|v rows [layers][m][2*kv] back, and synchronizes.
extern "C" int32_t qm_stack_step_host(qm_ctx *c, qm_stack *s, const float *x_host, int32_t m, float *h_host,
                                      float *kv_host) {
    CHECK_CTX(c);
    if (!stack_check(s) || !x_host || !h_host) return QM_ERR_ARG;
    if (m < 1 || m > s->m_max) return QM_ERR_SHAPE;
    CtxGuard g(c);
    DRV(g.rc);
    QmDriver *d = c->drv;
    DRV(d->cuMemcpyHtoDAsync_v2(s->h0, x_host, (size_t)m * s->hidden * 4, c->stream));
    int32_t rc = step_device(c, s, m);
    if (rc) return rc;
    DRV(d->cuMemcpyDtoHAsync_v2(h_host, h_source(s, m), (size_t)m * s->hidden * 4, c->stream));
    if (kv_host && s->kv) {
        const int64_t qkv_ld = s->hidden + 2 * s->kv;
        // (tensor-parallel: every GPU's slice of q|k|v has been stored into this arena)
        // One strided copy per activation row: the layers' buffers lie a fixed distance apart.
        for (int j = 0; j < m; j++) {
            CUDA_MEMCPY2D cp;
            memset(&cp, 0, sizeof cp);
            cp.srcMemoryType = CU_MEMORYTYPE_DEVICE;
            cp.srcDevice = layer_bufs(s, 0, m).qkv + ((size_t)j * qkv_ld + s->hidden) * 4;
            cp.srcPitch = layer_floats(s, m) * 4;
            cp.dstMemoryType = CU_MEMORYTYPE_HOST;
            cp.dstHost = kv_host + (size_t)j * 2 * s->kv;
            cp.dstPitch = (size_t)m * 2 * s->kv * 4;
            cp.WidthInBytes = (size_t)2 * s->kv * 4;
            cp.Height = (size_t)s->layers;
            DRV(d->cuMemcpy2DAsync_v2(&cp, c->stream));
        }
    }
    DRV(d->cuStreamSynchronize(c->stream));
    return QM_OK;
}
