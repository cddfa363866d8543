// Kernel parameter blocks shared by the device code and the host launcher.
// Every kernel takes ONE pointer-free-of-padding POD struct by value, made of
// 8-byte pointers, 8-byte and 4-byte integers and floats only — the parameter
// kinds the reference's ABI schema can describe
// (nvidia/x/cudakernel/abi.go:43-100).
#pragma once
#include <stdint.h>

#define QM_K_UNIT 256          // columns covered by one K unit (one Q4_K super-block)
#define QM_GEMV_MAX_THREADS 512  // up to 16 warps per CTA
#define QM_GEMV_TILE_ROWS 16   // rows of one mma tile
#define QM_STATUS_TIMEOUT 1u
#define QM_STATUS_BOUNDS 2u

// Device layouts held by the weight store.
//   Q4_K : the GGUF bytes unchanged, [rows][units][144].
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
