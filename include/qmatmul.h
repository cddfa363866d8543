/*
 * qmatmul.h — C ABI of libqmatmul.so: fused dequantize-and-multiply over GGUF
 * block-quantized weights on NVIDIA B200 (sm_100a).
 *
 * The library is meant to be bound without cgo (dlopen + dlsym, positional
 * integer/pointer arguments, no variadics, no struct by value): the calling
 * constraints of the reference's purego funnel (nvidia/internal/ffi/ffi.go:67-86).
 * Every entry point returns an int32 status: 0 = success, negative = one of the
 * QM_ERR_* codes below, positive = a CUresult of the CUDA driver, passed
 * through unchanged (the convention of nvidia/driver/result.gen.go:207-212).
 * No entry point aborts, traps or leaves a device-side wait unbounded.
 *
 * Kernels are sm_100a cubins that the library loads with cuModuleLoadData, the
 * call behind the reference's cudakernel.Artifact.Load
 * (nvidia/x/cudakernel/artifact.go:303-340). The same cubins and a JSON
 * description of each kernel's parameters sit next to the library so that a Go
 * caller may also load them directly through nvidia/driver.
 *
 * Threading: a qm_ctx binds one device's primary context and one stream. Each
 * call makes that context current for its own duration (the discipline of
 * nvidia/x/cuda/context.go:35-59), so calls may come from any OS thread, one at
 * a time per qm_ctx.
 */
#ifndef QMATMUL_H
#define QMATMUL_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define QM_VERSION 100
#define QM_API __attribute__((visibility("default")))

/* Weight formats: the GGUF tensor type ids of gguf/gguf.go:273-282. */
#define QM_FMT_Q4_0 2  /* lm/quant/quant.go:30-34  BlockQ4_0, 18 bytes / 32 elements  */
#define QM_FMT_Q8_0 8  /* lm/quant/quant.go:36-40  BlockQ8_0, 34 bytes / 32 elements  */
#define QM_FMT_Q2_K 10 /* lm/quant/kquant.go:29-34 BlockQ2_K, 84 bytes / 256 elements */
#define QM_FMT_Q4_K 12 /* gguf/gguf.go:276         type 12, 144 bytes / 256 elements  */
#define QM_FMT_IQ2_XXS 16 /* lm/quant/kquant.go:36-40 BlockIQ2_XXS, 66 bytes / 256 elements */

#define QM_OK 0
#define QM_ERR_COUNT (-1)    /* element count negative or not a multiple of the block (quant.go:45) */
#define QM_ERR_BUFFER (-2)   /* byte buffer shorter than the blocks need (quant.go:49)              */
#define QM_ERR_FORMAT (-3)   /* unknown or unsupported weight format                                */
#define QM_ERR_SHAPE (-4)    /* rows/cols/m/ld out of range for the operation                       */
#define QM_ERR_ARG (-5)      /* NULL pointer or invalid handle                                      */
#define QM_ERR_NO_DRIVER (-6)/* libcuda could not be loaded or lacks a required symbol              */
#define QM_ERR_NO_KERNEL (-7)/* a kernel image failed to load: the library cannot run               */
#define QM_ERR_TIMEOUT (-8)  /* a bounded device-side wait expired; see qm_last_status              */
#define QM_ERR_NOMEM (-9)    /* host allocation failed                                              */
#define QM_ERR_STATE (-10)   /* call not valid in the object's current state                        */
#define QM_ERR_LIMIT (-11)   /* size beyond a documented fixed maximum                              */
#define QM_ERR_DOMAIN (-12)  /* Q8_1 producer: nonfinite input/weight/value or zero denominator
                                (the data refusals of cudaquant.RMSNormQ8_1, quant.go:56-68,76-90)  */

/* Input transforms applied to the activation vector while it is staged
 * (qm_matvec flags, bits 0..3). */
#define QM_XOP_NONE 0u
#define QM_XOP_RMSNORM 1u     /* x * rsqrt(mean(x^2)+eps), the form of the reference's fused
                                 RMSNorm+GEMV (nvidia/x/egraph/codegen.go:395-414), no gain    */
#define QM_XOP_ADD_RMSNORM 2u /* rmsnorm(x + x2)                                               */
#define QM_XOP_SWIGLU 3u      /* silu(x) * x2 (nvidia/x/egraph/codegen.go:328-374)             */
#define QM_FLAG_PDL 0x100u    /* launch with programmatic stream serialization                 */
#define QM_FLAG_X_Q8_1 0x200u /* qm_matvec_selected: x holds Q8_1 blocks, not float32          */

typedef struct qm_ctx qm_ctx;
typedef uint64_t qm_weight; /* opaque handle of one device-resident weight matrix */

QM_API int32_t qm_version(void);
/* Static, NUL-terminated description of a status code (driver codes included
 * once a context exists). Mirrors cuGetErrorString as used by
 * nvidia/driver/result.gen.go:21. */
QM_API const char *qm_error_string(int32_t code);

/* Context: loads libcuda, retains the primary context of `device`, loads the
 * kernel images, creates a stream. Replaces the reference's
 * cuda.NewDevice + nvrtcx Compile/Load chain (nvidia/x/cuda/device.go:22-41,
 * nvidia/x/nvrtcx/load.go:26-71). */
QM_API int32_t qm_init(int32_t device, qm_ctx **out);
QM_API int32_t qm_destroy(qm_ctx *ctx);
/* Use the caller's CUstream (0 = the library's own stream) for all later work. */
QM_API int32_t qm_set_stream(qm_ctx *ctx, uint64_t cu_stream);
QM_API int32_t qm_sync(qm_ctx *ctx);
/* Device status word of the most recent launches (0 = clean); cleared on read. */
QM_API int32_t qm_last_status(qm_ctx *ctx, uint32_t *status);
/* Number of kernel launches issued through this context since qm_init. The
 * counter the reference keeps in cudalaunch.TotalLaunches
 * (nvidia/x/cudalaunch/launch.go:46-48). */
QM_API int64_t qm_launch_count(qm_ctx *ctx);

/* Plain device memory for callers without an allocator of their own
 * (driver.MemAllocBytes / DevicePtr.CopyFromHostPtr / CopyToHostPtr,
 * nvidia/driver/funcs.gen.go:12837, device_ptr.gen.go:679,597). */
QM_API int32_t qm_malloc(qm_ctx *ctx, int64_t bytes, uint64_t *dptr);
QM_API int32_t qm_free(qm_ctx *ctx, uint64_t dptr);
QM_API int32_t qm_memcpy_h2d(qm_ctx *ctx, uint64_t dst, const void *src, int64_t bytes);
QM_API int32_t qm_memcpy_d2h(qm_ctx *ctx, void *dst, uint64_t src, int64_t bytes);

/* Weight store. `host_bytes` are the tensor's bytes exactly as the GGUF file
 * holds them at DataOffset+Tensor.Offset (gguf/gguf.go:108-113,285-306):
 * `rows` rows of `cols` elements, row-major blocks. `cols` is
 * Tensor.Dimensions[0] and must be block aligned (gguf.go:290-292). Only rows
 * [row_lo,row_hi) are kept on the device (tensor-parallel row shard);
 * pass 0,rows for all. The bytes are copied before the call returns; nothing
 * is retained (nvidia/internal/ffi/call_funnel.go:100-126). */
QM_API int32_t qm_store_upload(qm_ctx *ctx, int32_t fmt, int64_t rows, int64_t cols, const void *host_bytes,
                        int64_t len, int64_t row_lo, int64_t row_hi, qm_weight *out);
/* A store entry assembled from several tensors stacked by rows (q|k|v,
 * gate|up): create with the total row count, then write row ranges. */
QM_API int32_t qm_store_create(qm_ctx *ctx, int32_t fmt, int64_t rows, int64_t cols, qm_weight *out);
QM_API int32_t qm_store_write_rows(qm_ctx *ctx, qm_weight w, int64_t row_offset, int64_t nrows,
                            const void *host_bytes, int64_t len);
/* Same, with the GGUF bytes already in device memory (not retained). */
QM_API int32_t qm_store_write_rows_device(qm_ctx *ctx, qm_weight w, int64_t row_offset, int64_t nrows,
                                   uint64_t dev_bytes, int64_t len);
QM_API int32_t qm_store_free(qm_ctx *ctx, qm_weight w);
/* info[0]=fmt, [1]=rows, [2]=cols, [3]=device bytes held, [4]=GGUF bytes represented */
QM_API int32_t qm_store_info(qm_ctx *ctx, qm_weight w, int64_t *info5);

/* Dequantize a stored matrix to float32 [rows][cols] in device memory.
 * Bit-exact with quant.DequantizeQ4_0/Q8_0/Q2_K (lm/quant/quant.go:44,72,
 * lm/quant/kquant.go:49). */
QM_API int32_t qm_dequantize(qm_ctx *ctx, qm_weight w, uint64_t out_f32_dev);
/* quant.Dequantize*(data []byte, numElements int) ([]float32, error) on the
 * GPU with host buffers: same validation order and error cases
 * (lm/quant/quant.go:44-91, kquant.go:49-77). */
QM_API int32_t qm_dequantize_host(qm_ctx *ctx, int32_t fmt, const void *data, int64_t len, int64_t num_elements,
                           float *out_host);

/* y[j][r] = sum_c x[j][c] * W[r][c] for j < m (1 <= m <= 8), float32 in and
 * out, device pointers; x rows are ldx floats apart, y rows ldy floats apart.
 * `x2_dev` is the second operand of QM_XOP_ADD_RMSNORM / QM_XOP_SWIGLU (0
 * otherwise). Supersedes the reference's one-warp-per-row kernels
 * (nvidia/x/egraph/codegen.go:443-482, 674-735). */
QM_API int32_t qm_matvec(qm_ctx *ctx, qm_weight w, uint64_t x_dev, uint64_t x2_dev, int32_t m, int64_t ldx,
                  uint64_t y_dev, int64_t ldy, uint32_t flags);
/* Same through host buffers: x is copied to the device, y copied back and the
 * stream synchronized before the call returns. */
QM_API int32_t qm_matvec_host(qm_ctx *ctx, qm_weight w, const float *x_host, int32_t m, int64_t ldx,
                       float *y_host, int64_t ldy, uint32_t flags);

/* ---- Q8_1 activation ABI ----------------------------------------------------------------------
 * An activation vector as blocks of 36 bytes per 32 elements: fp16 d, fp16 sum field, 32 signed
 * quants; element i = d * q[i] (cudaquant.BlockQ8_1, nvidia/x/cudaquant/quant.go:35-40;
 * block_q8_1 and q8_1_at of nvidia/x/egraph/codegen.go:114-128). Block pointers must be 4-byte
 * aligned. All calls are asynchronous on the context's stream unless they take host buffers.
 *
 * qm_rmsnorm_q8_1: row r of x (rows ldx floats apart) -> blocks [r][cols/32] at out_dev, bytes as
 * cudaquant.RMSNormQ8_1 produces them (quant.go:46-118; weight_dev = 0: unweighted). Replaces the
 * one-thread-per-row kernel rms_quant_q8_1 (quant.go:129-155). What the reference refuses by
 * looking at the data (nonfinite input or weight, zero denominator, nonfinite normalised value)
 * sets a status bit: qm_last_status then returns QM_ERR_DOMAIN.
 * qm_rmsnorm_q8_1_host: the reference's signature over host slices (lengths in elements), its
 * refusals in its order: dimensions/epsilon -> QM_ERR_SHAPE, length mismatches -> QM_ERR_BUFFER,
 * data refusals -> QM_ERR_DOMAIN with out_blocks left untouched. */
QM_API int32_t qm_rmsnorm_q8_1(qm_ctx *ctx, uint64_t x_dev, int64_t ldx, uint64_t weight_dev, int64_t rows,
                               int64_t cols, float eps, uint64_t out_dev);
QM_API int32_t qm_rmsnorm_q8_1_host(qm_ctx *ctx, const float *input, int64_t n_input, const float *weight,
                                    int64_t n_weight, int64_t rows, int64_t cols, float eps, int32_t weighted,
                                    void *out_blocks);
/* fused_swiglu_q8_1 (nvidia/x/egraph/codegen.go:513-552): `slots` vectors of `width` gate and up
 * values laid end to end, v = silu(min(gate, 10)) * clamp(up, -10, 10) * weights[slot], into
 * ceil(width*slots/32) blocks: d = fp16(max|v|/127), sum field = fp16(sum v), q = round(v/d). */
QM_API int32_t qm_swiglu_q8_1(qm_ctx *ctx, uint64_t gate_dev, uint64_t up_dev, uint64_t weights_dev, int32_t width,
                              int32_t slots, uint64_t out_dev);
/* out[j][i] = d * q of row j's blocks (rows ldx_blocks blocks apart), float32, exact. */
QM_API int32_t qm_q8_1_dequantize(qm_ctx *ctx, uint64_t xq_dev, int32_t m, int64_t ldx_blocks, int64_t cols,
                                  uint64_t out_dev, int64_t ld_out);
/* qm_matvec with Q8_1 activations (the *_matvec_q8_1 kernels, codegen.go:443-482 with ACT_LOAD =
 * q8_1_at, :674-809): y[j][r] = sum_c (d*q)[j][c] * W[r][c]. flags: QM_FLAG_PDL only. */
QM_API int32_t qm_matvec_q8_1(qm_ctx *ctx, qm_weight w, uint64_t xq_dev, int32_t m, int64_t ldx_blocks,
                              uint64_t y_dev, int64_t ldy, uint32_t flags);
/* Matvec over selected experts for decode-time MoE (q2_k_selected_matvec_q8_1, codegen.go:554-583;
 * iq2_xxs_selected_matvec_q8_1, :585-616): `w` holds `experts` equally sized matrices stacked by
 * rows (a GGUF 3-D expert tensor as it lies in the file), ids_dev[slot] (int32) names the expert of
 * each of `slots` slots, y_dev = float32 [slot][rows of one expert]. x is one vector for all slots
 * (x_slot_stride = 0, as in the reference) or one per slot, x_slot_stride floats (blocks) apart;
 * float32, or Q8_1 blocks with QM_FLAG_X_Q8_1. An id outside [0, experts) fills that slot's
 * outputs with the NaN 0x7fffffff. Formats: Q2_K, IQ2_XXS. */
QM_API int32_t qm_matvec_selected(qm_ctx *ctx, qm_weight w, int32_t experts, uint64_t ids_dev, int32_t slots,
                                  uint64_t x_dev, int64_t x_slot_stride, uint64_t y_dev, uint32_t flags);

/* Batched / prefill product over a stored Q4_K matrix on the tcgen05 tensor cores:
 * c[j][r] = sum_k a[j][k] * W[r][k] for j < m, a bf16 [m][lda] (16-byte aligned, lda a multiple
 * of 8), c float32 [m][ldc], device pointers. Weights are dequantized into shared memory as
 * bf16, accumulation is fp32 in tensor memory. Supersedes the reference's fp16 wmma prefill
 * GEMM (nvidia/x/cudamoe/prefill.go:97-121). Asynchronous on the context's stream. */
QM_API int32_t qm_matmul_bf16(qm_ctx *ctx, qm_weight w, uint64_t a_dev, int32_t m, int64_t lda, uint64_t c_dev,
                              int64_t ldc);

/* GroupedTopKRouter.Route (lm/moe/moe.go:73-141) for `tokens` tokens at once: experts ranked by
 * logit + bias (descending, ties to the lower index), weights = softmax over the selected
 * experts' UNBIASED logits (exp in double, rounded to float32, float32 sum in selection order).
 * logits float32 [tokens][ld], bias float32 [experts] or 0, ids int32 [tokens][topk],
 * weights float32 [tokens][topk]; experts <= 256 (the 256 routed experts of the reference's
 * MoEConfig, lm/moe/moe.go). Device pointers, asynchronous. */
QM_API int32_t qm_moe_route(qm_ctx *ctx, uint64_t logits_dev, int32_t tokens, int64_t ld, int32_t experts,
                            int32_t topk, uint64_t bias_dev, uint64_t ids_dev, uint64_t weights_dev);
/* Grouped expert matmul over routed token lists (SwiGLU experts, Q4_K weights):
 * out[t] = sum_s weights[t][s] * down_e( silu(gate_e x_t) * (up_e x_t) ), e = ids[t][s].
 * gate_up[e] is a stored [2*ffn][hidden] matrix (gate rows, then up rows), down[e] a stored
 * [hidden][ffn] matrix; x bf16 [tokens][ldx], out float32 [tokens][ldo]. Tokens are grouped per
 * expert on the device, each expert runs the tcgen05 matmul over its list, and the combine
 * adds a token's expert outputs in slot order. New API of this path: the reference's lm/moe
 * routes and caches experts but has no matmul; its device gather is nvidia/x/cudamoe/moe.go:72-96.
 * All experts run in two grouped launches (gate|up with the SwiGLU in its epilogue, then
 * down); ffn must be a multiple of 128. The list lengths are read back to the host once (one
 * stream synchronization inside the call) to size those launches; with QM_MOE_NOSYNC=1 in the
 * environment nothing is read back and the call is fully asynchronous (slower: the launches
 * then cover the longest possible lists). With QM_MOE_FOLD=1 the gate|up matmul gathers the
 * tokens' rows itself (tile::gather4 copies that follow the dispatch list; needs x 16-byte aligned
 * and ldx a multiple of 8) and no gathered copy is written: the same bits, no 2*pairs*hidden bytes
 * of scratch traffic, but slower on large token tiles. */
QM_API int32_t qm_moe_grouped(qm_ctx *ctx, const qm_weight *gate_up, const qm_weight *down, int32_t experts,
                              uint64_t x_bf16_dev, int32_t tokens, int64_t ldx, uint64_t ids_dev,
                              uint64_t weights_dev, int32_t topk, uint64_t out_dev, int64_t ldo);

/* The three stages of qm_moe_grouped, for expert-parallel runs where an exchange of rows
 * between GPUs sits between them (token dispatch, nvidia/x/cudamoe/moe.go:72-96 gathers rows
 * the same way; the exchange itself is the caller's NCCL all-to-all).
 * qm_moe_dispatch: groups the (token, slot) pairs of ids[tokens][topk] by expert (ascending
 *   token inside an expert), copies the bf16 row of each pair's token to rows[pairs][hidden] in
 *   that order, writes pos[pair] = row of the pair in the grouping, and returns the list
 *   lengths in counts_host[experts] (the call synchronizes the stream once to read them).
 * qm_moe_experts: y[p] = down_e( silu(gate_e r_p) * (up_e r_p) ) over rows grouped by expert
 *   (counts_host[e] consecutive rows per expert e, in order); y float32 [rows][hidden]. Two
 *   grouped launches for all experts; asynchronous.
 * qm_moe_combine: out[t] = sum_s weights[t][s] * y[pos[t*topk+s]], slots in order. */
QM_API int32_t qm_moe_dispatch(qm_ctx *ctx, uint64_t ids_dev, int32_t tokens, int32_t topk, int32_t experts,
                               uint64_t x_bf16_dev, int64_t ldx, int32_t hidden, uint64_t rows_dev,
                               uint64_t pos_dev, int32_t *counts_host);
QM_API int32_t qm_moe_experts(qm_ctx *ctx, const qm_weight *gate_up, const qm_weight *down, int32_t experts,
                              uint64_t rows_bf16_dev, const int32_t *counts_host, uint64_t y_dev);
QM_API int32_t qm_moe_combine(qm_ctx *ctx, uint64_t y_dev, uint64_t pos_dev, uint64_t weights_dev, int32_t tokens,
                              int32_t topk, int32_t hidden, uint64_t out_dev, int64_t ldo);

/* Decode-time MoE over selected Q4_K experts (1..few tokens): for every (token, slot) pair the
 * gate|up matvec of expert ids[t*topk+s] on the token's float32 x, then the down matvec on
 * silu(gate) * up, then out[t] = sum_s weights[t*topk+s] * down output, slots in order. The whole
 * batch is ONE persistent launch of the decode GEMV kernels plus a small combine; which expert a
 * pair uses is read on the device, so ids and weights can come straight from qm_moe_route. The
 * reference's counterparts are q2_k_selected_matvec_q8_1 / iq2_xxs_selected_matvec_q8_1
 * (nvidia/x/egraph/codegen.go:554-616), one launch per projection. Experts must be Q4_K stores
 * of one shape (gate|up: [2*ffn][hidden] rows stacked, down: [hidden][ffn]);
 * max_tokens * topk <= 32. A token with an id outside [0, experts) gets NaN outputs. Pairs are
 * independent matvecs: two tokens that choose the same expert each stream it — for larger
 * batches use qm_moe_grouped. x_dev/ids_dev changes between runs rebuild a small device list
 * (a synchronizing copy); steady-state callers keep their buffers. Asynchronous otherwise. */
typedef struct qm_moe_decode qm_moe_decode;
QM_API int32_t qm_moe_decode_create(qm_ctx *ctx, const qm_weight *gate_up, const qm_weight *down, int32_t experts,
                                    int32_t topk, int32_t max_tokens, qm_moe_decode **out);
QM_API int32_t qm_moe_decode_run(qm_ctx *ctx, qm_moe_decode *md, uint64_t x_dev, int32_t tokens, int64_t ldx,
                                 uint64_t ids_dev, uint64_t weights_dev, uint64_t out_dev, int64_t ldo);
QM_API int32_t qm_moe_decode_destroy(qm_ctx *ctx, qm_moe_decode *md);

/* Expert-parallel MoE layer behind the C ABI: rank `rank` of `world` (<= 8, one rank per GPU) owns
 * experts [rank*experts_local, (rank+1)*experts_local) of experts_total and calls qm_ep_moe with
 * its own tokens; the routed rows travel to the ranks that own their experts and the results back
 * through peer memory (plain stores into the peers' arenas, one flag per rank and direction, every
 * wait bounded: QM_ERR_TIMEOUT from qm_last_status) — no collective library is involved. The
 * reference's model for such an exchange is ncclGroupStart + ncclSend/ncclRecv pairs
 * (nvidia/nccl/comm.gen.go:401,288; nvidia/x/nccltest/run.go:595-603).
 * Set-up mirrors the tensor-parallel stack: qm_ep_create on every rank (max_tokens = the most
 * tokens ANY rank passes in one step; it sizes the arena: world * max_tokens * topk rows in both
 * directions), then either qm_ep_ipc_handle + exchange of the 64-byte handles + qm_ep_set_peers
 * (one process per GPU) or qm_ep_arena + qm_ep_set_peer_pointers (one process, peer access
 * enabled by the caller). world == 1 needs neither.
 * A step: x bf16 [tokens][ldx], ids int32 and weights float32 [tokens][topk] as qm_moe_route
 * writes them (ids outside [0, experts_total) contribute nothing), out float32 [tokens][ldo].
 * Every rank must run the same number of steps, also with zero tokens. qm_ep_moe is
 * qm_ep_begin (lists + push) + qm_ep_run (collect, grouped expert matmuls, return) + qm_ep_end
 * (combine); a process that drives several ranks calls each phase for all its ranks before the
 * next phase. Asynchronous on the context's stream. */
typedef struct qm_ep qm_ep;
QM_API int32_t qm_ep_create(qm_ctx *ctx, const qm_weight *gate_up, const qm_weight *down, int32_t experts_local,
                            int32_t experts_total, int32_t topk, int32_t max_tokens, int32_t rank, int32_t world,
                            qm_ep **out);
QM_API int32_t qm_ep_arena(qm_ctx *ctx, qm_ep *ep, uint64_t *base, int64_t *bytes);
QM_API int32_t qm_ep_ipc_handle(qm_ctx *ctx, qm_ep *ep, void *handle64);
QM_API int32_t qm_ep_set_peers(qm_ctx *ctx, qm_ep *ep, const void *handles /* world x 64 bytes */);
QM_API int32_t qm_ep_set_peer_pointers(qm_ctx *ctx, qm_ep *ep, const uint64_t *bases /* [world] */);
QM_API int32_t qm_ep_moe(qm_ctx *ctx, qm_ep *ep, uint64_t x_bf16_dev, int32_t tokens, int64_t ldx, uint64_t ids_dev,
                         uint64_t weights_dev, uint64_t out_dev, int64_t ldo);
QM_API int32_t qm_ep_begin(qm_ctx *ctx, qm_ep *ep, uint64_t x_bf16_dev, int32_t tokens, int64_t ldx, uint64_t ids_dev,
                           uint64_t weights_dev, uint64_t out_dev, int64_t ldo);
QM_API int32_t qm_ep_run(qm_ctx *ctx, qm_ep *ep);
QM_API int32_t qm_ep_end(qm_ctx *ctx, qm_ep *ep);
QM_API int32_t qm_ep_destroy(qm_ctx *ctx, qm_ep *ep);

/* No counterpart in the reference. The Q4_0 / Q8_0 matvec of qm_matvec for callers that may
 * not allocate device memory at the point of the call: a server whose memory plan is frozen
 * once it starts serving, a latency-critical loop where an allocation would stall the device,
 * or a host framework that owns the allocator and forbids allocations by the libraries it
 * calls. The split-K scratch (partial sums, arrival tickets, status word) lives in a fixed
 * 4 MiB array inside the library image, held by every GPU that loads the library until the
 * process exits; nothing is allocated or freed by this call, ever.
 *   w        a stored Q4_0 or Q8_0 matrix (its device memory was allocated when it was stored)
 *   x_dev    float32 [m][ldx], 16-byte aligned, ldx a multiple of 4; y_dev float32 [m][ldy]
 *   m        1..8 activation rows
 *   cu_stream  the CUstream to launch on (0 = the default stream); the call does not wait
 * The pointers belong to the current device's primary context, and the current device must be
 * the one the weights were stored on (QM_ERR_ARG otherwise). Returns QM_ERR_LIMIT when the
 * matrix needs more scratch than the array holds (scratch = 512 bytes per 16-row tile, per K
 * slice, per warp group sharing a tile, plus 4 bytes per tile), QM_ERR_FORMAT for other
 * formats. The first call on a device resolves the array's device address and raises the
 * kernels' shared-memory limit: make it outside any stream capture. All calls on a device
 * share the array; each clears the words it needs at zero, and calls whose kernels overlap on
 * the GPU race on it — order them on one stream or with events. */
QM_API int32_t qm_matvec_noalloc(qm_weight w, uint64_t x_dev, int32_t m, int64_t ldx, uint64_t y_dev,
                                 int64_t ldy, uint64_t cu_stream);
/* Status word of the most recent qm_matvec_noalloc on the current device: 0 = clean,
 * bit 0 = a bounded wait inside the kernel ran out (y is then incomplete; the call returns
 * QM_ERR_TIMEOUT). The word sits in the same fixed array, so reading it allocates nothing (a
 * 4-byte device-to-host copy). Synchronize the matvec's stream first, and read before the next
 * qm_matvec_noalloc on the device, which clears the word. Like qm_matvec_noalloc it has no
 * counterpart in the reference. */
QM_API int32_t qm_noalloc_status(uint32_t *status);

/* Decode step over a stack of layers whose matrices are stored weights of one
 * format: per layer q|k|v [hidden+2*kv_dim][hidden], o [hidden][hidden],
 * gate|up [2*ffn][hidden] and down [hidden][ffn], each matvec reading the RMS
 * normalised output of its producer (down reads rmsnorm(gate + up)). The
 * launches are captured once per batch size and replayed as one graph with
 * programmatic dependent launch. New API of this path (the reference has no
 * model runner above lm/quant); shapes as in Llama-3-8B: 32 layers, hidden
 * 4096, kv_dim 1024, ffn 14336. */
typedef struct qm_stack qm_stack;
QM_API int32_t qm_stack_create(qm_ctx *ctx, int32_t layers, int32_t hidden, int32_t kv_dim, int32_t ffn,
                               int32_t m_max, qm_stack **out);
QM_API int32_t qm_stack_destroy(qm_ctx *ctx, qm_stack *stack);
QM_API int32_t qm_stack_set_layer(qm_ctx *ctx, qm_stack *stack, int32_t layer, qm_weight qkv, qm_weight o,
                                  qm_weight gate_up, qm_weight down);
/* x_dev [m][ldx] -> h_out_dev [m][ldh] (last down-projection output), asynchronous. */
QM_API int32_t qm_stack_step(qm_ctx *ctx, qm_stack *stack, uint64_t x_dev, int32_t m, int64_t ldx,
                             uint64_t h_out_dev, int64_t ldh);
/* Host buffers: x [m][hidden] in; h [m][hidden] and, if kv_host is not NULL, every layer's k|v
 * outputs [layers][m][2*kv_dim] out; returns after the stream has drained. */
QM_API int32_t qm_stack_step_host(qm_ctx *ctx, qm_stack *stack, const float *x_host, int32_t m, float *h_host,
                                  float *kv_host);
/* Activation buffers for per-matvec checks: [0] input, [1] q|k|v of every layer, [2] o,
 * [3] gate|up, [4] down (of the last layer run). */
QM_API int32_t qm_stack_buffers(qm_ctx *ctx, qm_stack *stack, uint64_t *ptrs5);
/* info2[0] = K parts the most recent step cut the o projection into (1 = whole), info2[1] = floats
 * between its partial vectors: ptrs5[2] of qm_stack_buffers then holds partial sums. */
QM_API int32_t qm_stack_parts(qm_ctx *ctx, qm_stack *stack, int64_t *info2);
/* 0 = issue the launches one by one; 1 = replay them as a captured graph; 2 (default) = the
 * whole step as one persistent launch where format and shapes allow it, else as 1. */
QM_API int32_t qm_stack_use_graph(qm_ctx *ctx, qm_stack *stack, int32_t on);

/* Tensor-parallel decode stack over the GPUs of one box, one process per GPU (config "row
 * sharding at 1/2/4/8 GPUs"). Rank `rank` of `world` (<= 8) holds rows [rank*R/world,
 * (rank+1)*R/world) of EVERY matrix — q|k|v, o, gate|up, down — (R/world a multiple of 16)
 * and hands those slices to qm_stack_set_layer. The whole step is one persistent launch per
 * GPU: a GPU's slice of an output is stored straight into every peer's activation arena over
 * NVLink (peer memory mapped through CUDA IPC, or plain pointers in a one-process caller) and
 * consumers poll their own arena for the words they read; one barrier over the GPUs ends the
 * launch (flags in peer memory, every wait bounded: QM_ERR_TIMEOUT from qm_last_status) — the
 * all-gather of the reference's plan (nvidia/x/nccltest/run.go:375-391,584) fused into the
 * matvec kernel. */
QM_API int32_t qm_stack_create_tp(qm_ctx *ctx, int32_t layers, int32_t hidden, int32_t kv_dim, int32_t ffn,
                                  int32_t m_max, int32_t rank, int32_t world, qm_stack **out);
/* The paired form of the same step, the usual pairing of transformer matrices: q|k|v and gate|up sliced by
 * rows, o and down by K over the rank's OWN slice of their inputs, so that only two of a layer's four
 * hand-overs cross the GPUs. Rank r holds: of q|k|v the rows of q slice r followed by the rows of k|v slice r;
 * of gate|up the rows of gate slice r followed by those of up slice r (slice r of N rows = [r*N/world,
 * (r+1)*N/world)); of o and of down ALL rows of the K columns [r*K/world, (r+1)*K/world) — a column shard
 * is, for every row, the blocks of that column range, in row order. An o or down part leaves a partial
 * output vector per GPU in every arena; the consumer adds them in rank order (the same bits on every GPU).
 * This departs from "rows of every matrix": it is the same product, summed over K in `world` pieces
 * instead of one. hidden and ffn must be multiples of 256*world, 2*kv_dim of 16*world; m_max <= 4.
 * Everything else (handles, peers, steps, results, bounded waits) is as for qm_stack_create_tp. */
QM_API int32_t qm_stack_create_tp_paired(qm_ctx *ctx, int32_t layers, int32_t hidden, int32_t kv_dim, int32_t ffn,
                                         int32_t m_max, int32_t rank, int32_t world, qm_stack **out);
QM_API int32_t qm_stack_ipc_handle(qm_ctx *ctx, qm_stack *stack, void *handle64);
QM_API int32_t qm_stack_set_peers(qm_ctx *ctx, qm_stack *stack, const void *handles);
/* The same for a caller that drives all GPUs from one process (the reference's nccltest model,
 * nvidia/x/nccltest/run.go:375-391, with Context.EnablePeerAccess, nvidia/driver/context.gen.go:98):
 * qm_stack_arena returns this rank's arena, qm_stack_set_peer_pointers takes the `world` arena
 * base addresses as this process addresses them (entry `rank` ignored). */
QM_API int32_t qm_stack_arena(qm_ctx *ctx, qm_stack *stack, uint64_t *base, int64_t *bytes);
QM_API int32_t qm_stack_set_peer_pointers(qm_ctx *ctx, qm_stack *stack, const uint64_t *bases);

/* GGUF file -> weight store. qm_gguf_open parses header, metadata and tensor directory of a GGUF v3
 * file by the rules of gguf.Read (gguf/gguf.go:116-250; QM_ERR_FORMAT for a malformed or
 * unsupported file, QM_ERR_COUNT for a row that is not block aligned, QM_ERR_STATE if the file
 * cannot be opened) and keeps what gguf.File.Tensors holds: name, TypeID, Dimensions, Offset.
 * qm_gguf_tensor_info: info6 = {type id, ndims, dims[4]}, offs2 = {DataOffset + Offset, Bytes()}.
 * qm_gguf_load_tensor / qm_gguf_load_rows stream rows [row_lo, row_hi) of a tensor (rows = product
 * of Dimensions[1:], row length Dimensions[0]; row_hi = 0 means all) from the file through two
 * pinned staging buffers into a store entry, reading the next chunk while the previous one is
 * copied and permuted on the device; load_rows writes into an existing entry (q|k|v or gate|up
 * stacked by rows). No GPU is needed to open and inspect a file. */
typedef struct qm_gguf qm_gguf;
QM_API int32_t qm_gguf_open(const char *path, qm_gguf **out);
QM_API int32_t qm_gguf_close(qm_gguf *file);
QM_API int32_t qm_gguf_tensor_count(qm_gguf *file);
QM_API int32_t qm_gguf_tensor_info(qm_gguf *file, int32_t index, char *name, int32_t name_cap, int64_t *info6,
                                   int64_t *offs2);
QM_API int32_t qm_gguf_find(qm_gguf *file, const char *name);
QM_API int32_t qm_gguf_load_tensor(qm_ctx *ctx, qm_gguf *file, int32_t index, int64_t row_lo, int64_t row_hi,
                                   qm_weight *out);
QM_API int32_t qm_gguf_load_rows(qm_ctx *ctx, qm_gguf *file, int32_t index, int64_t row_lo, int64_t row_hi,
                                 qm_weight w, int64_t dst_row);

/* Host-side residency manager for expert weight blobs, the behaviour of moe.ExpertCacheManager
 * (lm/moe/moe.go:143-287): at most max_hot experts stay in host memory, admitting one more
 * spills the least recently used one (never the one just touched) to <dir>/expert_<id>.bin, a
 * cold expert is read back on demand. dir NULL or "" = $TMPDIR/lm-expert-cache. max_hot <= 0 is
 * refused (QM_ERR_ARG), an unknown expert is QM_ERR_ARG, file errors are QM_ERR_STATE.
 * qm_expert_cache_get with out = NULL only returns the size (and pages the expert in); with a
 * buffer it copies the bytes (QM_ERR_BUFFER if capacity is short). The bytes are what
 * qm_store_upload takes. Thread-safe; no GPU involved. */
typedef struct qm_expert_cache qm_expert_cache;
QM_API int32_t qm_expert_cache_create(const char *dir, int32_t max_hot, qm_expert_cache **out);   /* NewExpertCacheManager */
QM_API int32_t qm_expert_cache_register(qm_expert_cache *cache, int64_t expert, const void *bytes, int64_t n); /* RegisterExpert */
QM_API int32_t qm_expert_cache_get(qm_expert_cache *cache, int64_t expert, void *out, int64_t capacity,
                                   int64_t *size);                                               /* GetExpert */
QM_API int32_t qm_expert_cache_hot(qm_expert_cache *cache);                                      /* HotExperts */
QM_API int32_t qm_expert_cache_evict(qm_expert_cache *cache, int64_t expert);                    /* EvictColdExpert */
QM_API int32_t qm_expert_cache_close(qm_expert_cache *cache);                                    /* Close */

/* Device-side residency over such a host cache, for models whose experts do not all fit in HBM:
 * `max_resident` store entries of one shape (fmt, rows, cols) are allocated once;
 * qm_expert_pool_get returns the entry that holds `expert`, first overwriting the least recently
 * used entry (never the one just touched) with the expert's bytes from the host cache (memory or
 * spill file) when it is not resident. A returned handle names an ENTRY: it stays valid, but a
 * later get that misses may give the entry to another expert — fetch the handles of all experts
 * of a step (max_resident >= their number) before launching it. No counterpart in the
 * reference, whose ExpertCacheManager stops at host memory (lm/moe/moe.go:143-287).
 * qm_expert_pool_info: [0] experts resident, [1] entries, [2] hits, [3] misses. */
typedef struct qm_expert_pool qm_expert_pool;
QM_API int32_t qm_expert_pool_create(qm_ctx *ctx, qm_expert_cache *host, int32_t fmt, int64_t rows, int64_t cols,
                                     int32_t max_resident, qm_expert_pool **out);
QM_API int32_t qm_expert_pool_get(qm_ctx *ctx, qm_expert_pool *pool, int64_t expert, qm_weight *out);
QM_API int32_t qm_expert_pool_info(qm_expert_pool *pool, int64_t *info4);
QM_API int32_t qm_expert_pool_evict(qm_expert_pool *pool, int64_t expert);
QM_API int32_t qm_expert_pool_close(qm_ctx *ctx, qm_expert_pool *pool);

#ifdef __cplusplus
}
#endif
#endif /* QMATMUL_H */
