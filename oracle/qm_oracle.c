/*
 * qm_oracle.c — CPU restatement of the reference's quantized-weight algorithms.
 *
 * TEST INFRASTRUCTURE ONLY. Nothing in the product path (the CUDA library and
 * its host bindings) links, loads or calls this file. It is the checker the
 * parity tests compare the CUDA kernels against, and the timed "port" CPU
 * baseline of the benchmark.
 *
 * Each function names the reference file:line it follows (paths are relative
 * to the tmc/lib repository root).
 *
 * Pinning status:
 *   Q4_0, Q8_0, fp16->fp32 : pinned by the reference's known-answer tests
 *                            (lm/quant/quant_test.go:12-43).
 *   Q2_K                   : pinned bit-exactly by the reference's golden
 *                            vectors (lm/quant/testdata/ds4_golden.txt).
 *   router                 : pinned by lm/moe/moe_test.go:12-32 and
 *                            lm/moe/routing_test.go:21-130.
 *   Q4_K                   : PARITY UNPINNED. The reference holds no decoder,
 *                            test or vector for GGUF type 12 — only its block
 *                            geometry (256 elements / 144 bytes,
 *                            gguf/gguf.go:276). The decoder below restates
 *                            the public GGUF type-12 field layout with the
 *                            arithmetic form of the sibling Q2_K decoder
 *                            (lm/quant/kquant.go:73) and is cross-checked
 *                            against an independently written numpy decoder.
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define QO_OK 0
#define QO_ERR_COUNT (-1)  /* element count negative or not a block multiple */
#define QO_ERR_SHORT (-2)  /* buffer shorter than the blocks need */
#define QO_ERR_FORMAT (-3) /* unknown format id */
#define QO_ERR_TYPE (-4)   /* unknown GGUF tensor type */
#define QO_ERR_ALIGN (-5)  /* GGUF row not block aligned */
#define QO_ERR_OVERFLOW (-6)

/* Format ids shared with the CUDA library (include/qmatmul.h). */
enum { QO_Q4_0 = 2, QO_Q8_0 = 8, QO_Q2_K = 10, QO_Q4_K = 12 };

/* lm/quant/quant.go:94-116 — IEEE binary16 bits to float32, bit for bit:
 * subnormals are normalised by the shift loop, inf/NaN keep the mantissa
 * payload shifted by 13 (signalling NaNs are NOT quieted). */
float qo_f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (uint32_t)(h & 0x7C00u) >> 10;
    uint32_t mant = (uint32_t)(h & 0x03FFu);
    uint32_t bits;
    if (exp == 0) {
        if (mant == 0) {
            bits = sign;
            goto done;
        }
        while ((mant & 0x0400u) == 0) {
            mant <<= 1;
            exp--; /* wraps below zero exactly like the Go uint32 */
        }
        exp++;
        mant &= 0x03FFu;
    } else if (exp == 0x1F) {
        bits = sign | 0x7F800000u | (mant << 13);
        goto done;
    }
    exp = exp + (127 - 15);
    mant = mant << 13;
    bits = sign | (exp << 23) | mant;
done:;
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

uint32_t qo_f16_to_f32_bits(uint16_t h) {
    float f = qo_f16_to_f32(h);
    uint32_t b;
    memcpy(&b, &f, 4);
    return b;
}

static inline uint16_t rd16(const uint8_t *p) { return (uint16_t)(p[0] | (p[1] << 8)); }

/* Shared argument validation: lm/quant/quant.go:45-51, kquant.go:50-56.
 * A trailing surplus of bytes is accepted, as in lm/quant. */
static int check(int64_t len, int64_t n, int64_t block, int64_t bytes) {
    if (n < 0 || n % block != 0) return QO_ERR_COUNT;
    if (len < (n / block) * bytes) return QO_ERR_SHORT;
    return QO_OK;
}

/* lm/quant/quant.go:44-68 — Q4_0: 18-byte blocks, low nibbles are elements
 * 0..15 and high nibbles elements 16..31, value = (nibble-8)*scale. */
int qo_dequantize_q4_0(const uint8_t *data, int64_t len, int64_t n, float *out) {
    int rc = check(len, n, 32, 18);
    if (rc) return rc;
    for (int64_t b = 0; b < n / 32; b++) {
        const uint8_t *blk = data + b * 18;
        float scale = qo_f16_to_f32(rd16(blk));
        for (int i = 0; i < 16; i++) {
            uint8_t v = blk[2 + i];
            int lo = (int)(v & 0x0F) - 8;
            int hi = (int)(v >> 4) - 8;
            out[b * 32 + i] = (float)lo * scale;
            out[b * 32 + 16 + i] = (float)hi * scale;
        }
    }
    return QO_OK;
}

/* lm/quant/quant.go:72-91 — Q8_0: 34-byte blocks, value = int8*scale. */
int qo_dequantize_q8_0(const uint8_t *data, int64_t len, int64_t n, float *out) {
    int rc = check(len, n, 32, 34);
    if (rc) return rc;
    for (int64_t b = 0; b < n / 32; b++) {
        const uint8_t *blk = data + b * 34;
        float scale = qo_f16_to_f32(rd16(blk));
        for (int i = 0; i < 32; i++) out[b * 32 + i] = (float)(int8_t)blk[2 + i] * scale;
    }
    return QO_OK;
}

/* lm/quant/kquant.go:49-77 — Q2_K: 84-byte super-blocks laid out as
 * scales[16] | qs[64] | d | dmin; element value d*(sc&15)*q - dmin*(sc>>4),
 * evaluated left to right in float32 without contraction. */
int qo_dequantize_q2_k(const uint8_t *data, int64_t len, int64_t n, float *out) {
    int rc = check(len, n, 256, 84);
    if (rc) return rc;
    for (int64_t b = 0; b < n / 256; b++) {
        const uint8_t *blk = data + b * 84;
        const uint8_t *scales = blk, *quants = blk + 16;
        float d = qo_f16_to_f32(rd16(blk + 80));
        float dmin = qo_f16_to_f32(rd16(blk + 82));
        for (int i = 0; i < 256; i++) {
            int group = i / 16, l = i - group * 16;
            int base = 32 * (group / 8) + 16 * (group & 1);
            int shift = ((group / 2) & 3) * 2;
            int q = (quants[base + l] >> shift) & 3;
            uint8_t sc = scales[group];
            float t1 = d * (float)(sc & 0x0f);
            float t2 = t1 * (float)q;
            float t3 = dmin * (float)(sc >> 4);
            out[b * 256 + i] = t2 - t3;
        }
    }
    return QO_OK;
}

/* Q4_K scale/min unpacking for sub-block j of one super-block. S is the
 * 12-byte field at bytes 4..15. Public GGUF type-12 convention (the reference
 * pins only the 144-byte size, gguf/gguf.go:276):
 *   j<4 : sc = S[j]&63,                     m = S[j+4]&63
 *   j>=4: sc = (S[j+4]&15) | (S[j-4]>>6)<<4, m = (S[j+4]>>4) | (S[j]>>6)<<4 */
static inline void q4k_scale_min(const uint8_t *S, int j, int *sc, int *m) {
    if (j < 4) {
        *sc = S[j] & 63;
        *m = S[j + 4] & 63;
    } else {
        *sc = (S[j + 4] & 0x0F) | ((S[j - 4] >> 6) << 4);
        *m = (S[j + 4] >> 4) | ((S[j] >> 6) << 4);
    }
}

/* Q4_K: 144-byte super-blocks d | dmin | S[12] | qs[128]. The 32 bytes
 * qs[32p..32p+31] carry sub-block 2p in their low nibbles and sub-block 2p+1
 * in their high nibbles. Value = (d*sc)*q - dmin*m in float32, the arithmetic
 * form of lm/quant/kquant.go:73. */
int qo_dequantize_q4_k(const uint8_t *data, int64_t len, int64_t n, float *out) {
    int rc = check(len, n, 256, 144);
    if (rc) return rc;
    for (int64_t b = 0; b < n / 256; b++) {
        const uint8_t *blk = data + b * 144;
        float d = qo_f16_to_f32(rd16(blk));
        float dmin = qo_f16_to_f32(rd16(blk + 2));
        const uint8_t *S = blk + 4, *qs = blk + 16;
        for (int j = 0; j < 8; j++) {
            int sc, m;
            q4k_scale_min(S, j, &sc, &m);
            float t1 = d * (float)sc;
            float t3 = dmin * (float)m;
            const uint8_t *g = qs + 32 * (j / 2);
            for (int i = 0; i < 32; i++) {
                int q = (j & 1) ? (g[i] >> 4) : (g[i] & 0x0F);
                float t2 = t1 * (float)q;
                out[b * 256 + j * 32 + i] = t2 - t3;
            }
        }
    }
    return QO_OK;
}

int64_t qo_block_elems(int fmt) {
    switch (fmt) {
    case QO_Q4_0: case QO_Q8_0: return 32;
    case QO_Q2_K: case QO_Q4_K: return 256;
    }
    return 0;
}

int64_t qo_block_bytes(int fmt) {
    switch (fmt) {
    case QO_Q4_0: return 18;
    case QO_Q8_0: return 34;
    case QO_Q2_K: return 84;
    case QO_Q4_K: return 144;
    }
    return 0;
}

int qo_dequantize(int fmt, const uint8_t *data, int64_t len, int64_t n, float *out) {
    switch (fmt) {
    case QO_Q4_0: return qo_dequantize_q4_0(data, len, n, out);
    case QO_Q8_0: return qo_dequantize_q8_0(data, len, n, out);
    case QO_Q2_K: return qo_dequantize_q2_k(data, len, n, out);
    case QO_Q4_K: return qo_dequantize_q4_k(data, len, n, out);
    }
    return QO_ERR_FORMAT;
}

/* gguf/gguf.go:273-306 — byte size of a tensor: dims[0] is the row length and
 * must be block aligned; the remaining dims multiply; overflow is an error. */
int qo_tensor_bytes(uint32_t type_id, const uint64_t *dims, int nd, uint64_t *out) {
    static const struct { uint32_t id; uint64_t block, bytes; } T[] = {
        {0, 1, 4},     {1, 1, 2},     {2, 32, 18},   {3, 32, 20},   {6, 32, 22},   {7, 32, 24},
        {8, 32, 34},   {9, 32, 40},   {10, 256, 84}, {11, 256, 110}, {12, 256, 144}, {13, 256, 176},
        {14, 256, 210}, {15, 256, 292}, {16, 256, 66}, {17, 256, 74}, {18, 256, 98}, {19, 256, 110},
        {20, 256, 50}, {21, 256, 110}, {22, 256, 82}, {23, 256, 136}, {24, 1, 1},   {25, 1, 2},
        {26, 1, 4},    {27, 1, 8},    {28, 1, 8},    {29, 256, 56}, {30, 1, 2},    {39, 32, 17},
    };
    for (size_t i = 0; i < sizeof T / sizeof T[0]; i++) {
        if (T[i].id != type_id) continue;
        if (nd < 1 || dims[0] % T[i].block != 0) return QO_ERR_ALIGN;
        unsigned __int128 n = (unsigned __int128)(dims[0] / T[i].block) * T[i].bytes;
        if (n >> 64) return QO_ERR_OVERFLOW;
        for (int d = 1; d < nd; d++) {
            n *= dims[d];
            if (n >> 64) return QO_ERR_OVERFLOW;
        }
        *out = (uint64_t)n;
        return QO_OK;
    }
    return QO_ERR_TYPE;
}

/* lm/moe/moe.go:73-141 — GroupedTopKRouter.Route for one token.
 * Ranking key is logit+bias (descending, ties to the lower index); weights are
 * the softmax of the UNBIASED logits of the selected experts, with exp taken
 * in float64 and rounded to float32, summed in float32 in selection order.
 * Returns k, the number of experts selected. */
int qo_route(const float *logits, int n_logits, int n_experts, int topk, const float *biases,
             int32_t *ids, float *weights) {
    int n = n_experts;
    if (n_logits < n) n = n_logits;
    if (n < 0) n = 0;
    int k = topk;
    if (k > n) k = n;
    if (k < 0) k = 0;
    if (k == 0) return 0;
    int *idx = (int *)malloc(sizeof(int) * (size_t)n);
    float *score = (float *)malloc(sizeof(float) * (size_t)n);
    for (int i = 0; i < n; i++) {
        idx[i] = i;
        float s = logits[i] + (biases ? biases[i] : 0.0f);
        score[i] = s;
    }
    /* selection of the k best under the total order (score desc, index asc);
     * equivalent to the reference's full sort with the same comparator */
    for (int a = 0; a < k; a++) {
        int best = a;
        for (int b = a + 1; b < n; b++) {
            int ib = idx[b], ibest = idx[best];
            if (score[ib] != score[ibest] ? score[ib] > score[ibest] : ib < ibest) best = b;
        }
        int t = idx[a];
        idx[a] = idx[best];
        idx[best] = t;
    }
    float max_logit = logits[idx[0]];
    for (int i = 0; i < k; i++) {
        ids[i] = idx[i];
        if (logits[idx[i]] > max_logit) max_logit = logits[idx[i]];
    }
    float sum = 0.0f;
    for (int i = 0; i < k; i++) {
        float diff = logits[idx[i]] - max_logit;
        float e = (float)exp((double)diff);
        weights[i] = e;
        sum += e;
    }
    if (sum > 0) {
        for (int i = 0; i < k; i++) {
            float w = weights[i] / sum;
            weights[i] = w;
        }
    }
    free(idx);
    free(score);
    return k;
}

/* Output oracle: y[m][r] = sum_c x[m][c] * dequant(W)[r][c], composed from the
 * reference's dequantizer and a float64 accumulator rounded once, the
 * construction the reference's own device tests use
 * (nvidia/x/egraph/q2k_cuda_test.go:81-96, nvidia/x/cudaref/ref.go:28-44).
 * W is rows x cols in GGUF row-major block layout. */
int qo_matvec(int fmt, const uint8_t *w, int64_t wlen, int64_t rows, int64_t cols, const float *x,
              int m, int64_t ldx, float *y, int64_t ldy) {
    int64_t be = qo_block_elems(fmt), bb = qo_block_bytes(fmt);
    if (!be) return QO_ERR_FORMAT;
    if (rows < 0 || cols < 0 || cols % be != 0) return QO_ERR_COUNT;
    int64_t row_bytes = cols / be * bb;
    if (wlen < rows * row_bytes) return QO_ERR_SHORT;
    float *wr = (float *)malloc(sizeof(float) * (size_t)(cols ? cols : 1));
    for (int64_t r = 0; r < rows; r++) {
        qo_dequantize(fmt, w + r * row_bytes, row_bytes, cols, wr);
        for (int j = 0; j < m; j++) {
            double acc = 0.0;
            const float *xr = x + (int64_t)j * ldx;
            for (int64_t c = 0; c < cols; c++) acc += (double)wr[c] * (double)xr[c];
            y[(int64_t)j * ldy + r] = (float)acc;
        }
    }
    free(wr);
    return QO_OK;
}

/* Timed CPU baseline: the same dequantize-then-dot in float32 arithmetic,
 * rows split over `threads` POSIX threads. With threads=1 and a whole-matrix
 * dequantize it mirrors what a single goroutine calling the reference's
 * Dequantize* followed by a dot loop would execute. */
typedef struct {
    int fmt;
    const uint8_t *w;
    int64_t r0, r1, cols, row_bytes, ldx, ldy;
    const float *x;
    int m;
    float *y;
} mv_job;

static void *mv_worker(void *p) {
    mv_job *j = (mv_job *)p;
    float *wr = (float *)malloc(sizeof(float) * (size_t)(j->cols ? j->cols : 1));
    for (int64_t r = j->r0; r < j->r1; r++) {
        qo_dequantize(j->fmt, j->w + r * j->row_bytes, j->row_bytes, j->cols, wr);
        for (int k = 0; k < j->m; k++) {
            const float *xr = j->x + (int64_t)k * j->ldx;
            float acc = 0.0f;
            for (int64_t c = 0; c < j->cols; c++) acc += wr[c] * xr[c];
            j->y[(int64_t)k * j->ldy + r] = acc;
        }
    }
    free(wr);
    return NULL;
}

int qo_matvec_f32_threaded(int fmt, const uint8_t *w, int64_t wlen, int64_t rows, int64_t cols,
                           const float *x, int m, int64_t ldx, float *y, int64_t ldy, int threads) {
    int64_t be = qo_block_elems(fmt), bb = qo_block_bytes(fmt);
    if (!be) return QO_ERR_FORMAT;
    if (rows < 0 || cols < 0 || cols % be != 0) return QO_ERR_COUNT;
    int64_t row_bytes = cols / be * bb;
    if (wlen < rows * row_bytes) return QO_ERR_SHORT;
    if (threads < 1) threads = 1;
    if (threads > 256) threads = 256;
    pthread_t tid[256];
    mv_job jobs[256];
    for (int t = 0; t < threads; t++) {
        jobs[t] = (mv_job){fmt, w, rows * t / threads, rows * (t + 1) / threads, cols, row_bytes,
                           ldx, ldy, x, m, y};
        if (threads == 1) mv_worker(&jobs[t]);
        else pthread_create(&tid[t], NULL, mv_worker, &jobs[t]);
    }
    if (threads > 1)
        for (int t = 0; t < threads; t++) pthread_join(tid[t], NULL);
    return QO_OK;
}

/* RMS normalisation used between the matvecs of the synthetic decode chain:
 * out = x * 1/sqrt(mean(x^2) + eps); the form of the reference's fused
 * RMSNorm+GEMV kernel without a gain vector
 * (nvidia/x/egraph/codegen.go:395-414). Accumulates in float64. */
void qo_rmsnorm(const float *x, int64_t n, float eps, float *out) {
    double s = 0.0;
    for (int64_t i = 0; i < n; i++) s += (double)x[i] * (double)x[i];
    float scale = (float)(1.0 / sqrt(s / (double)n + (double)eps));
    for (int64_t i = 0; i < n; i++) out[i] = x[i] * scale;
}
