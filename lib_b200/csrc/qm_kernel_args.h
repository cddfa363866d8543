// Kernel parameter blocks shared by the device code and the host launcher.
// Every kernel takes ONE pointer-free-of-padding POD struct by value, made of
// 8-byte pointers, 8-byte and 4-byte integers and floats only — the parameter
// kinds the reference's ABI schema can describe
// (nvidia/x/cudakernel/abi.go:43-100).
#pragma once
#include <cuda.h>
#include <stdint.h>

#define QM_K_UNIT 256          // columns covered by one K unit (one Q4_K super-block)
#define QM_GEMV_MAX_THREADS 512  // up to 16 warps per CTA
#define QM_GEMV_TILE_ROWS 16   // rows of one mma tile
#define QM_STATUS_TIMEOUT 1u
#define QM_STATUS_BOUNDS 2u
#define QM_STATUS_DOMAIN 4u   // a Q8_1 producer met a zero denominator or a nonfinite value

// Device layouts held by the weight store.
//   Q4_K : the GGUF super-blocks regrouped so that one (16-row tile, K unit) item is 2304
//          contiguous bytes: [tiles][units][ 16 x 16-byte headers (d|dmin|scales) |
//          4 groups p x 16 rows x 32 quant bytes ]. A pure permutation of the 144-byte
//          blocks; rows past the last one are zero.
//   Q2_K : the GGUF bytes unchanged, [rows][units][84].
//   Q4_0 : quants [rows][units*8] x 16 bytes, scales [rows][units*8] fp16.
//   Q8_0 : quants [rows][units*8] x 32 bytes, scales [rows][units*8] fp16.
// Rows of Q4_0/Q8_0 are padded with zero-scale blocks up to a whole K unit.

struct QmGemvArgs {
    const uint8_t *wq;       // quant bytes (see layouts above)
    const uint16_t *wd;      // fp16 scale plane (Q4_0/Q8_0), unused for Q4_K
    const float *x;          // activations [m][ldx]
    const float *x2;         // second activation operand or null
    float *y;                // outputs [m][ldy]
    float *partials;         // scratch [ksplit][tiles][maxseg][8][16] partial sums
    unsigned int *tickets;   // scratch [tiles] arrival counters, zero between launches
    unsigned int *status;    // device status word
    int64_t ldx, ldy;
    int32_t rows, cols;      // logical matrix shape (cols = K)
    int32_t units;           // K units per row (cols rounded up / 256)
    int32_t m;               // activation rows, 1..8
    int32_t tiles;           // 16-row tiles: ceil(rows / 16)
    int32_t ksplit;          // K slices; CTAs [s*ctas_per_slice, (s+1)*ctas_per_slice) own slice s
    int32_t units_per_slice; // K units per slice (the last slice may be shorter)
    int32_t ctas_per_slice;
    int32_t consumers;       // warps per CTA
    int32_t depth;           // bulk-copy stages per warp
    int32_t kc;              // K units per stage
    int32_t maxseg;          // partial-sum slots per (slice, tile)
    int32_t xop;             // QM_XOP_*
    float eps;
};

// One Q4_0 / Q8_0 matvec of up to four activation rows on the integer tensor-core path (lean_body).
struct QmLeanArgs {
    const uint8_t *wq;       // quant plane [rows][units*8][16 or 32 B] (layouts above)
    const uint16_t *wd;      // fp16 scale plane [rows][units*8]
    const float *x, *x2;     // activations [m][ldx]; x2: second operand of QM_XOP_ADD_RMSNORM / QM_XOP_SWIGLU
    float *y;                // outputs [m][ldy]
    int64_t ldx, ldy;
    int32_t rows, cols, m;
    int32_t units;           // K units of one part (all of a row's when parts == 1)
    int32_t units_total;     // K units of a whole row of the store
    int32_t xop;
    float eps;
    int32_t q, rem;          // 16-row tiles per CTA of a part: q, the first rem CTAs one more
    int32_t parts;           // K parts (CTA groups); > 1: y holds `parts` partial vectors, part_stride floats apart
    int32_t pad_;
    int64_t part_stride;
    float *ssq;              // parts > 1 with a normalising xop: [parts][8] sums of squares of x per part and row
};

// One matvec of a fused sequence (Q4_K weights, integer tensor-core path).
#define QM_Q4K_ITEM_BYTES 2304
#define QM_MAX_INLINE_OPS 8
#define QM_MAX_PEERS 8

struct alignas(16) QmOp {   // a multiple of 16 bytes: the kernels copy descriptors in 16-byte pieces
    const uint8_t *wq;   // tiled Q4_K store layout
    const float *x;      // activations [m][ldx]
    const float *x2;     // second operand of QM_XOP_ADD_RMSNORM / QM_XOP_SWIGLU, or null
    float *y;            // outputs [m][ldy]
    int64_t ldx, ldy;
    int32_t rows, cols, units, tiles;   // units = K units of this op's K slice
    int32_t units_total; // K units of a whole row of the matrix
    int32_t unit0;       // first K unit of the slice
    int32_t accumulate;  // 1: add to y instead of overwriting it (later K slices)
    int32_t xop;         // QM_XOP_*
    int32_t barrier;     // 1: every CTA must have finished the previous op before x is read
    float eps;
    // balanced == 0: the tiles of the op are dealt to the CTAs in contiguous runs, CTA c owns q
    // tiles, the first `rem` CTAs one more. balanced == 1: the (tile, unit) ITEMS are dealt that
    // way, so two CTAs may share a tile; both add their part to y with red.global.add (two
    // addends on a zero: order-independent), and y's shared tiles are zeroed during the op before
    int32_t q, rem;
    int32_t balanced;
    int32_t tp_shared;   // tensor-parallel launch: bit 0 = the op's results (and the words of its K part) go into every
                         // GPU's arena, else into this GPU's only; bit 1 = the same for the second output (y2)
    // Activation image: the quantized form of an op's x (limb planes, sub-block sums, column
    // weights, sums of squares per unit) in global memory. An op whose x is the previous op's y
    // can read it ready-made instead of every CTA quantizing all of x: the previous op builds
    // it unit by unit, each unit by the warp whose store completes the unit's 256 outputs.
    const uint8_t *img;       // consumer side: image of this op's x, or null (quantize in the CTA)
    uint8_t *q_img;           // producer side: image of the NEXT op's x, or null
    unsigned int *q_cnt;      // producer side: one completion counter per unit of the next op's x, zero at launch
    int32_t q_half_tiles;     // 16-row tiles of y per operand of the next op (its cols / 16)
    int32_t q_halves;         // 1, or 2 when the next op's x is the sum of two halves of y
    // K parts (data-driven kernels only). An op can be cut into S column ranges ("parts") of
    // `units` K units each. The CTAs of a launch then form groups (QmFusedArgs::ngroups), every
    // group runs its own copy of the op list, and in the copy of group g the op IS part
    // `part`: wq points at that part's items (the stack keeps a part-major copy of the matrix, so
    // they are contiguous), unit0 is its first K unit of x, y its partial output vector, and only
    // the CTAs [cta0, cta0 + nctas) work on it. A part leaves its products WITHOUT the RMS scale
    // of its input. The consumer (x_parts = S) adds the S partial vectors while it stages them;
    // it normalises that sum itself, and to make the result equal to normalising the scaled sum
    // it needs the producer's input mean square: part s leaves the sum of squares of its range
    // per activation row in ssq_out[s*8 + row], the consumer reads all S from ssq_in.
    int32_t parts;            // producer side: K parts this op is one of (1 = the op is whole)
    int32_t part;             // which part
    int32_t cta0, nctas;      // the CTAs that work on this op: [cta0, cta0 + nctas)
    int32_t x_parts;          // consumer side: partial vectors that add up to x (1 = x is one vector)
    int64_t x_part_stride;    // floats between the partial input vectors
    float *ssq_out;           // producer side: [parts][8] sums of squares of x per K part and activation row
    const float *ssq_in;      // consumer side: the same words of the op that produced x
    float ssq_in_inv_cols;    // 1 / K of the op that produced x
    float ssq_in_eps;         // its epsilon
    // Selected expert (kernels *_sel only): when sel_table is set the op's matrix is not wq but
    // sel_table[sel_ids[sel_index]] (an id outside [0, sel_count) is clamped into it), read on the
    // device when the op's first copy is issued — all candidates have this op's shape.
    const uint8_t *const *sel_table;
    const int32_t *sel_ids;
    int32_t sel_index, sel_count;
    // Second output (tensor-parallel kernels only): rows [split_row, rows) of the op go to y2 instead of y
    // (split_row a multiple of 16; 0 = one output). tp_shared bit 0 / bit 1 then say which of the two goes
    // to every GPU's arena.
    float *y2;
    int32_t split_row;
    int32_t pad3_;
};

struct QmFusedArgs {
    QmOp inl[QM_MAX_INLINE_OPS];  // the ops of a single-matvec launch (used when ops is null)
    const QmOp *ops;     // device array of nops ops, or null
    unsigned int *status;    // device status word
    unsigned int *grid_bar;  // grid barrier counter, zero at launch
    int32_t nops, m;
    int32_t consumers, depth;
    int32_t max_units;   // largest K units over the ops: sizes the activation planes
    int32_t cpm;         // mma columns per activation row: 4 (m <= 2) or 2 (m <= 4, or 8 with two column tiles)
    int32_t debug;       // 0 in production
    int32_t debug_slot;
    int32_t img_units;   // K units an activation image has room for (>= units_total of every op that reads one)
    int32_t ngroups;     // CTA groups, each with its own copy of the op list (ops + g*nops); 0 or 1 = one list
    int64_t wait_cycles; // SM clock cycles after which a device-side wait gives up and sets QM_STATUS_TIMEOUT
    // Tensor-parallel launch (kernels *_tp): this GPU computes a row slice of every op and stores
    // it into the same place of every peer's activation arena (its own address + peer_delta[p]);
    // the barrier between dependent ops then spans the GPUs: the last CTA of a GPU to arrive
    // writes the barrier's epoch into flag [tp_rank] of every peer, and every CTA waits for the
    // flags of all peers in its own arena.
    int32_t tp_world, tp_rank;       // tp_world <= 1: single GPU
    unsigned int tp_epoch0;          // epoch of the launch's first barrier minus one; grows from launch to launch
    unsigned int tp_counter;         // 1: every CTA adds its arrival to a counter in every arena (NVLink atomics); 0: flags
    unsigned int *tp_flags;          // [tp_world] in this GPU's arena, written by the peers
    int64_t peer_delta[QM_MAX_PEERS];   // bytes from an address in this arena to the same place in peer p's
};

// Prefill GEMM over Q4_K weights (tcgen05): C[m][n] = sum_k A[m][k] * W[n][k].
struct QmGemmArgs {
    alignas(64) CUtensorMap tmap_act;  // activations [m][k] bf16, box 64 x bn, 128-byte swizzle
    const uint8_t *wq;     // tiled Q4_K store
    float *c;              // [m][ldc]
    unsigned int *status;
    int64_t ldc;
    int32_t m, n;
    int32_t units;         // K / 256
    int32_t tiles16;       // 16-row tiles of the store
    int32_t bn;            // tokens per CTA: 64, 128, 256 or 512
    int32_t stages;        // shared-memory stages, 2..8
    int32_t splitk;        // K shares (blockIdx.z) of a single matmul; 1 in grouped launches
    // Grouped launch over the experts of a mixture-of-experts layer (blockIdx.z = expert): the
    // activations are the rows [offsets[e], offsets[e+1]) of one gathered matrix, the weights
    // of expert e start at wq_list[e]; CTAs beyond an expert's rows leave at once.
    int32_t grouped;
    const uint8_t *const *wq_list;   // device array of the experts' stores
    const int32_t *offsets;          // device array [experts + 1]
    // SwiGLU epilogue (256-row kernel only): sub-tile 0 holds gate rows n, sub-tile 1 the up rows
    // n + up_offset; the CTA stores bf16 silu(gate) * up to h[row][n] instead of C.
    int32_t swiglu, up_offset;
    uint16_t *h;           // bf16 [rows][ldh]
    int64_t ldh;
    int32_t debug;         // 0 in production; bits switch off pipeline roles for timing experiments (results are wrong)
    int32_t groups;        // groups of dequantizing warps, each a chunk ahead of the next: 4 (one thread per weight row) or 2
    // Split K: share z of an output tile goes to partials[z][m][n] (plain stores); when all splitk CTAs of
    // the tile have arrived (tickets[2*tile], zero between launches) each adds one band of the tile in order
    // of z and writes C — no atomics on C, the same bits every run. The launch is cooperative.
    float *partials;
    unsigned int *tickets;
    int64_t wait_cycles;
    // Gather folded into the activation load (grouped launches): row p of the grouped order is row
    // gather_list[p] / gather_topk of the tokens' own matrix, which tmap_gather describes with a box of
    // 64 columns x 1 row; the loader warp fetches four rows per tile::gather4 copy.
    const int32_t *gather_list;   // null: the activations are already grouped (tmap_act, tiled loads)
    int32_t gather_topk;
    int32_t box_rows;             // token rows per tiled load of tmap_act
    int32_t plane_rows;           // activation rows of one split-K plane (m, or all grouped rows)
    alignas(64) CUtensorMap tmap_gather;
};

#define QM_MAX_EXPERTS 256    // experts of a layer (router, dispatch lists, grouped matmuls); 64 per GPU in expert-parallel runs

// Mixture-of-experts helpers (qm_moe.cu).
struct QmRouteArgs {
    const float *logits;   // [tokens][ld]
    const float *bias;     // [experts] or null
    int32_t *ids;          // [tokens][topk]
    float *weights;        // [tokens][topk]
    int64_t ld;
    int32_t tokens, experts, topk, pad;
};
struct QmListArgs {
    const int32_t *ids;    // [tokens*topk]
    int32_t *rank;         // scratch [tokens*topk]
    int32_t *counts;       // [experts]
    int32_t *offsets;      // [experts+1]
    int32_t *list;         // [tokens*topk] pair indices grouped by expert
    int32_t *pos;          // [tokens*topk] row of each pair in the grouping
    int32_t tokens, experts, topk, pad;
};
struct QmGatherArgs {
    const uint16_t *x;     // bf16 [tokens][ldx]
    const int32_t *list;
    uint16_t *out;         // bf16 [rows][hidden]
    int64_t ldx;
    int32_t rows, hidden, topk, pad;
};
struct QmCombineArgs {
    const float *y;        // [rows][hidden] expert outputs in grouped order
    const int32_t *pos;
    const float *weights;
    float *out;            // [tokens][ldo]
    int64_t ldo;
    int32_t tokens, hidden, topk, pad;
};

// GEMV over Q2_K / IQ2_XXS weights kept in their GGUF byte layout (qm_gemv_kq.cu).
struct QmKqArgs {
    const uint8_t *wq;       // [rows][units] super-blocks of 84 (Q2_K) or 66 (IQ2_XXS) bytes; selected form: [experts][rows][units]
    const void *x;           // activations [m][ldx] float32, or Q8_1 blocks (_q81 kernels; ldx in blocks)
    float *y;                // outputs [m][ldy]
    int64_t ldx, ldy;
    int64_t rows;            // rows of the matrix (selected form: of one expert)
    int32_t units, m;
    // selected form (ids != nullptr): blockIdx.y = slot, expert = ids[slot]
    const int32_t *ids;
    int32_t experts;
    int32_t depth;           // >= 2: rows go through a per-warp shared-memory ring of this many stages; 0: direct loads
    int64_t x_slot_stride;   // floats (or blocks) between the activations of consecutive slots; 0: one x for all
    int64_t y_slot_stride;   // floats between the outputs of consecutive slots
    int32_t xs_bytes;        // _q81 kernels: > 0: shared-memory bytes (a multiple of 16) that hold the CTA's activations
    int32_t pad_;
};

// RMSNorm -> Q8_1 (qm_q8_1.cu): row r of x (rows ldx floats apart) into cols/32 blocks of 36 bytes.
struct QmNormQ81Args {
    const float *x;
    const float *weight;     // nullptr: unweighted
    uint8_t *out;            // [rows][cols/32] blocks
    unsigned int *status;
    int64_t ldx;
    int32_t cols;
    float eps;
};

// SwiGLU -> Q8_1: `slots` vectors of `width` gate and up values laid end to end, one weight per slot.
struct QmSwigluQ81Args {
    const float *gate, *up, *weights;
    uint8_t *out;            // ceil(width*slots/32) blocks
    int32_t width, slots;
};

// Q8_1 -> float32.
struct QmQ81ExpandArgs {
    const uint8_t *xq;       // [m][ldx] blocks
    float *out;              // [m][ld_out]
    int64_t ldx, ld_out;
    int32_t cols, m;
};

// out[t][c] = sum_k weights[t*topk+k] * y[t*topk+k][c] (decode-time MoE: one output vector per (token, slot)
// pair); a token with an id outside [0, experts) gets the NaN 0x7fffffff.
struct QmDecodeCombineArgs {
    const float *y;          // [tokens*topk][hidden]
    const int32_t *ids;
    const float *weights;
    float *out;
    int64_t ldo;
    int32_t tokens, topk, experts, hidden;
};

// Expert-parallel MoE over peer memory (qm_ep_* kernels in qm_moe.cu). Every rank owns `eloc` consecutive
// experts and an arena of the same layout; a rank stores into the arenas of its peers (its own address plus
// peer_delta[p]) and reads only its own.
struct QmEpArgs {
    // this rank's step
    const uint16_t *x;        // bf16 tokens [tokens][ldx]
    const int32_t *ids;       // [tokens*topk] global expert of every (token, slot) pair
    const int32_t *list;      // pairs grouped by global expert (qm_moe_lists)
    const int32_t *offsets;   // [experts + 1] starts of those groups
    const int32_t *pos;       // [tokens*topk] place of every pair in the grouping, -1: none
    const float *weights;     // [tokens*topk]
    float *out;               // [tokens][ldo]
    int64_t ldx, ldo;
    // this rank as an owner of experts
    uint16_t *compact;        // [world*cap][hidden] bf16: the rows received, grouped by local expert
    int32_t *back;            // [world*cap] source rank << 24 | place in that rank's segment, per compact row
    int32_t *loff;            // [eloc + 1] starts of the local experts' groups in `compact`
    const float *y;           // [world*cap][hidden] outputs of the experts, in `compact` order
    unsigned int *done;       // [2] CTA arrival counters (push, return), zero at the start of a step
    unsigned int *status;
    // the arena
    unsigned int *flags;      // [2][QM_MAX_PEERS] epochs: [0][s] rank s has pushed its rows, [1][o] owner o has returned its results
    int32_t *counts_in;       // [world][eloc] rows from rank s for local expert e
    uint16_t *rows_in;        // [world][cap][hidden] bf16 rows from rank s, grouped by local expert
    float *ret_in;            // [world][cap][hidden] results from owner o for the rows this rank sent it, in sending order
    int64_t peer_delta[QM_MAX_PEERS];
    int32_t tokens, topk, hidden, experts, eloc, world, rank, cap;
    unsigned int epoch;
    int32_t pad_;
    int64_t wait_cycles;
};

// h[j][r] = c_j * sum over parts of parts[k*part_stride + j*ld_in + r], c_j = rsqrt(mean square + eps)
// from the per-part sums of squares ssq[k*8 + j] (qm_sum_parts: the last matvec of a step that ran in K parts).
struct QmSumPartsArgs {
    const float *parts;
    const float *ssq;
    float *out;
    int64_t part_stride, ld_in, ld_out;
    int32_t nparts, m, n;
    float inv_cols, eps;
};

// Part-major copy of a tiled Q4_K store (qm_repack_parts): ups = K units per part.
struct QmPartsArgs {
    const uint8_t *src;
    uint8_t *dst;
    int32_t tiles, units, ups, pad;
};

struct QmDequantArgs {
    const uint8_t *wq;
    const uint16_t *wd;
    float *out;              // [rows][cols]
    int64_t rows;
    int32_t cols, units;
};

struct QmRepackArgs {
    const uint8_t *src;      // GGUF bytes of `nrows` rows
    uint8_t *wq;
    uint16_t *wd;
    int64_t row_offset, nrows;
    int32_t cols, units;
};
