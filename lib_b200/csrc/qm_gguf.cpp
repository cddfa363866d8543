// qm_gguf.cpp — GGUF file -> device weight store.
//
// qm_gguf_open parses the header, the metadata and the tensor directory of a GGUF v3 file with the
// rules of the reference's reader (gguf/gguf.go:116-250: magic, version 3 only, bounded counts and
// string lengths, no duplicate keys or tensor names, 1..4 non-zero dimensions, `general.alignment`
// a uint32 multiple of 8, tensors contiguous and aligned from DataOffset on, every tensor inside the
// file) and keeps what a loader needs: name, type id, dimensions and file offset of each tensor.
// Metadata values are validated and skipped; only `general.alignment` is interpreted.
//
// qm_gguf_load_tensor streams one tensor's rows into a store entry: the file is read in chunks
// into two pinned host buffers used alternately, each chunk goes to the device with an
// asynchronous copy and is permuted into the store's layout by the repack kernels, so reading chunk
// i+1 from the file overlaps the copy and repack of chunk i. Row ranges [row_lo, row_hi) load a
// tensor-parallel rank's slice without touching the rest of the file.
#include <fcntl.h>
#include <stdio.h>
#include <string.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <new>
#include <set>
#include <string>
#include <vector>

#include "qm_internal.h"

#define QM_GGUF_MAGIC 0x46554747u  // "GGUF" little-endian

namespace {

// bounds of gguf/gguf.go:15-20
constexpr uint64_t kMaxMetadata = 1 << 20, kMaxTensors = 1 << 20, kMaxString = 1 << 24, kMaxArray = 1 << 20;

struct GgufTensor {
    std::string name;
    uint32_t type_id;
    int ndims;
    uint64_t dims[4];
    uint64_t offset;   // relative to the data block
    uint64_t bytes;
};

bool block_geometry(uint32_t type_id, uint64_t *block, uint64_t *bytes) {   // gguf/gguf.go:273-282
    static const struct { uint32_t id; uint64_t block, bytes; } T[] = {
        {0, 1, 4},     {1, 1, 2},     {2, 32, 18},   {3, 32, 20},   {6, 32, 22},   {7, 32, 24},
        {8, 32, 34},   {9, 32, 40},   {10, 256, 84}, {11, 256, 110}, {12, 256, 144}, {13, 256, 176},
        {14, 256, 210}, {15, 256, 292}, {16, 256, 66}, {17, 256, 74}, {18, 256, 98}, {19, 256, 110},
        {20, 256, 50}, {21, 256, 110}, {22, 256, 82}, {23, 256, 136}, {24, 1, 1},   {25, 1, 2},
        {26, 1, 4},    {27, 1, 8},    {28, 1, 8},    {29, 256, 56}, {30, 1, 2},    {39, 32, 17},
    };
    for (const auto &t : T)
        if (t.id == type_id) {
            *block = t.block;
            *bytes = t.bytes;
            return true;
        }
    return false;
}

struct Reader {
    int fd;
    uint64_t size, off;
    bool ok;
    bool read(void *dst, uint64_t n) {
        if (!ok || n > size - off) return ok = false;
        uint8_t *p = static_cast<uint8_t *>(dst);
        uint64_t done = 0;
        while (done < n) {
            const ssize_t r = pread(fd, p + done, (size_t)std::min<uint64_t>(n - done, 1 << 30), (off_t)(off + done));
            if (r <= 0) return ok = false;
            done += (uint64_t)r;
        }
        off += n;
        return true;
    }
    bool skip(uint64_t n) {
        if (!ok || n > size - off) return ok = false;
        off += n;
        return true;
    }
    uint32_t u32() { uint32_t v = 0; read(&v, 4); return v; }
    uint64_t u64() { uint64_t v = 0; read(&v, 8); return v; }
    bool str(std::string *out) {
        const uint64_t n = u64();
        if (!ok || n > kMaxString) return ok = false;
        out->resize((size_t)n);
        return n == 0 || read(&(*out)[0], n);
    }
    // skips one metadata value of type t (arrays nest at most as deep as the reference allows)
    bool value(uint32_t t, int depth, uint32_t *as_u32) {
        static const int fixed[13] = {1, 1, 2, 2, 4, 4, 4, 1, -1, -1, 8, 8, 8};
        if (t > 12) return ok = false;
        if (t == 8) {
            std::string s;
            return str(&s);
        }
        if (t == 9) {
            if (depth >= 4) return ok = false;
            const uint32_t et = u32();
            const uint64_t n = u64();
            if (!ok || n > kMaxArray) return ok = false;
            for (uint64_t i = 0; i < n; i++)
                if (!value(et, depth + 1, nullptr)) return false;
            return true;
        }
        if (t == 4 && as_u32) {
            *as_u32 = u32();
            return ok;
        }
        return skip((uint64_t)fixed[t]);
    }
};

}  // namespace

struct qm_gguf {
    uint32_t magic;
    int fd;
    uint64_t size, data_offset, alignment;
    std::vector<GgufTensor> tensors;
    void *pinned[2];
    CUdeviceptr stage[2];
    CUevent done[2];
    size_t chunk_bytes;
    qm_ctx *staging_ctx;
};

static void free_staging(qm_gguf *g) {
    if (!g->staging_ctx) return;
    qm_ctx *c = g->staging_ctx;
    CtxGuard guard(c);
    if (guard.rc == CUDA_SUCCESS) {
        c->drv->cuStreamSynchronize(c->stream);
        for (int k = 0; k < 2; k++) {
            if (g->pinned[k]) c->drv->cuMemFreeHost(g->pinned[k]);
            if (g->stage[k]) c->drv->cuMemFree_v2(g->stage[k]);
            if (g->done[k]) c->drv->cuEventDestroy_v2(g->done[k]);
            g->pinned[k] = nullptr;
            g->stage[k] = 0;
            g->done[k] = nullptr;
        }
    }
    g->staging_ctx = nullptr;
}

extern "C" int32_t qm_gguf_open(const char *path, qm_gguf **out) {
    if (!path || !out) return QM_ERR_ARG;
    *out = nullptr;
    const int fd = open(path, O_RDONLY);
    if (fd < 0) return QM_ERR_STATE;
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size < 0) {
        close(fd);
        return QM_ERR_STATE;
    }
    qm_gguf *g = new (std::nothrow) qm_gguf();
    if (!g) {
        close(fd);
        return QM_ERR_NOMEM;
    }
    g->magic = QM_GGUF_MAGIC;
    g->fd = fd;
    g->size = (uint64_t)st.st_size;
    g->alignment = 32;
    g->pinned[0] = g->pinned[1] = nullptr;
    g->stage[0] = g->stage[1] = 0;
    g->done[0] = g->done[1] = nullptr;
    g->staging_ctx = nullptr;
    Reader r{fd, g->size, 0, true};
    auto fail = [&](int32_t code) {
        close(fd);
        delete g;
        return code;
    };
    if (r.u32() != QM_GGUF_MAGIC || !r.ok) return fail(QM_ERR_FORMAT);   // bad magic
    if (r.u32() != 3 || !r.ok) return fail(QM_ERR_FORMAT);               // only version 3 (gguf.go:132)
    const uint64_t ntensors = r.u64(), nmeta = r.u64();
    if (!r.ok || ntensors > kMaxTensors || nmeta > kMaxMetadata) return fail(QM_ERR_FORMAT);
    if (nmeta * 13 > r.size - r.off) return fail(QM_ERR_FORMAT);
    std::set<std::string> keys;
    for (uint64_t i = 0; i < nmeta; i++) {
        std::string key;
        if (!r.str(&key) || key.size() > 65535 || !keys.insert(key).second) return fail(QM_ERR_FORMAT);
        const uint32_t t = r.u32();
        const bool is_align = key == "general.alignment";
        uint32_t v = 0;
        if (is_align && t != 4) return fail(QM_ERR_FORMAT);   // alignment must be a uint32 (gguf.go:213)
        if (!r.value(t, 0, is_align ? &v : nullptr)) return fail(QM_ERR_FORMAT);
        if (is_align) {
            if (v == 0 || v > (1u << 20) || v % 8 != 0) return fail(QM_ERR_FORMAT);
            g->alignment = v;
        }
    }
    if (ntensors * 32 > r.size - r.off) return fail(QM_ERR_FORMAT);
    std::set<std::string> names;
    g->tensors.reserve((size_t)ntensors);
    for (uint64_t i = 0; i < ntensors; i++) {
        GgufTensor t;
        if (!r.str(&t.name) || t.name.size() > 64 || !names.insert(t.name).second) return fail(QM_ERR_FORMAT);
        const uint32_t nd = r.u32();
        if (!r.ok || nd == 0 || nd > 4) return fail(QM_ERR_FORMAT);
        t.ndims = (int)nd;
        for (uint32_t d = 0; d < 4; d++) t.dims[d] = 1;
        for (uint32_t d = 0; d < nd; d++) {
            t.dims[d] = r.u64();
            if (!r.ok || t.dims[d] == 0) return fail(QM_ERR_FORMAT);
        }
        t.type_id = r.u32();
        t.offset = r.u64();
        if (!r.ok) return fail(QM_ERR_FORMAT);
        g->tensors.push_back(t);
    }
    const uint64_t A = g->alignment;
    g->data_offset = ntensors ? (r.off + A - 1) / A * A : r.off;
    if (g->data_offset > g->size) return fail(QM_ERR_FORMAT);
    uint64_t expected = 0;
    for (GgufTensor &t : g->tensors) {
        uint64_t block, bbytes;
        if (!block_geometry(t.type_id, &block, &bbytes)) return fail(QM_ERR_FORMAT);
        if (t.dims[0] % block != 0) return fail(QM_ERR_COUNT);            // row not block aligned (gguf.go:290)
        unsigned __int128 n = (unsigned __int128)(t.dims[0] / block) * bbytes;
        for (int d = 1; d < t.ndims; d++) {
            n *= t.dims[d];
            if (n >> 64) return fail(QM_ERR_FORMAT);
        }
        t.bytes = (uint64_t)n;
        if (t.offset % A != 0 || t.offset != expected) return fail(QM_ERR_FORMAT);
        if (t.bytes > g->size - g->data_offset || t.offset > g->size - g->data_offset - t.bytes) return fail(QM_ERR_FORMAT);
        expected = (t.offset + t.bytes + A - 1) / A * A;
    }
    *out = g;
    return QM_OK;
}

extern "C" int32_t qm_gguf_close(qm_gguf *g) {
    if (!g || g->magic != QM_GGUF_MAGIC) return QM_ERR_ARG;
    free_staging(g);
    close(g->fd);
    g->magic = 0;
    delete g;
    return QM_OK;
}

extern "C" int32_t qm_gguf_tensor_count(qm_gguf *g) {
    if (!g || g->magic != QM_GGUF_MAGIC) return QM_ERR_ARG;
    return (int32_t)g->tensors.size();
}

// info6: [0] type id, [1] number of dimensions, [2..5] dimensions (1 beyond the last); offs2: [0] file offset of
// the tensor's bytes (DataOffset + Tensor.Offset), [1] byte count (Tensor.Bytes). name may be NULL.
extern "C" int32_t qm_gguf_tensor_info(qm_gguf *g, int32_t index, char *name, int32_t name_cap, int64_t *info6,
                                       int64_t *offs2) {
    if (!g || g->magic != QM_GGUF_MAGIC || index < 0 || (size_t)index >= g->tensors.size()) return QM_ERR_ARG;
    const GgufTensor &t = g->tensors[(size_t)index];
    if (name && name_cap > 0) {
        const size_t n = std::min<size_t>(t.name.size(), (size_t)name_cap - 1);
        memcpy(name, t.name.data(), n);
        name[n] = 0;
    }
    if (info6) {
        info6[0] = t.type_id;
        info6[1] = t.ndims;
        for (int d = 0; d < 4; d++) info6[2 + d] = (int64_t)t.dims[d];
    }
    if (offs2) {
        offs2[0] = (int64_t)(g->data_offset + t.offset);
        offs2[1] = (int64_t)t.bytes;
    }
    return QM_OK;
}

// Index of the tensor called `name`, or QM_ERR_ARG.
extern "C" int32_t qm_gguf_find(qm_gguf *g, const char *name) {
    if (!g || g->magic != QM_GGUF_MAGIC || !name) return QM_ERR_ARG;
    for (size_t i = 0; i < g->tensors.size(); i++)
        if (g->tensors[i].name == name) return (int32_t)i;
    return QM_ERR_ARG;
}

// Rows [row_lo, row_hi) of tensor `index` (rows = product of the dimensions after the first, the row
// length is Dimensions[0]) into rows [dst_row, dst_row + row_hi - row_lo) of the store entry `w`,
// which must have the tensor's format and row length.
extern "C" int32_t qm_gguf_load_rows(qm_ctx *c, qm_gguf *g, int32_t index, int64_t row_lo, int64_t row_hi, qm_weight w,
                                     int64_t dst_row) {
    CHECK_CTX(c);
    if (!g || g->magic != QM_GGUF_MAGIC || index < 0 || (size_t)index >= g->tensors.size()) return QM_ERR_ARG;
    const GgufTensor &t = g->tensors[(size_t)index];
    int64_t info[5];
    int32_t rc = qm_store_info(c, w, info);
    if (rc) return rc;
    const int64_t rows = (int64_t)(t.dims[1] * t.dims[2] * t.dims[3]);
    if ((int64_t)t.type_id != info[0] || (int64_t)t.dims[0] != info[2]) return QM_ERR_SHAPE;
    if (row_lo < 0 || row_hi > rows || row_lo > row_hi || dst_row < 0 || dst_row + (row_hi - row_lo) > info[1])
        return QM_ERR_SHAPE;
    if (row_lo == row_hi) return QM_OK;
    const int64_t row_bytes = (int64_t)(t.bytes / (uint64_t)rows);
    CtxGuard guard(c);
    DRV(guard.rc);
    QmDriver *d = c->drv;
    // staging: two pinned buffers and two device buffers of 32 MiB (at least one row), made on first use
    const size_t want = (size_t)std::max<int64_t>(32ll << 20, row_bytes);
    if (g->staging_ctx != c || g->chunk_bytes < want) {
        free_staging(g);
        g->staging_ctx = c;
        g->chunk_bytes = want;
        for (int k = 0; k < 2; k++) {
            CUresult r = d->cuMemHostAlloc(&g->pinned[k], want, 0);
            if (r == CUDA_SUCCESS) r = d->cuMemAlloc_v2(&g->stage[k], want + 64);
            if (r == CUDA_SUCCESS) r = d->cuEventCreate(&g->done[k], CU_EVENT_DISABLE_TIMING);
            if (r != CUDA_SUCCESS) {
                free_staging(g);
                return (int32_t)r;
            }
        }
    }
    const int64_t chunk_rows = std::max<int64_t>(1, (int64_t)g->chunk_bytes / row_bytes);
    bool used[2] = {false, false};
    int k = 0;
    for (int64_t r0 = row_lo; r0 < row_hi; r0 += chunk_rows, k ^= 1) {
        const int64_t nr = std::min(chunk_rows, row_hi - r0);
        if (used[k]) DRV(d->cuEventSynchronize(g->done[k]));   // the copy and repack that last used this pair are done
        const uint64_t off = g->data_offset + t.offset + (uint64_t)(r0 * row_bytes);
        uint64_t done = 0, n = (uint64_t)(nr * row_bytes);
        while (done < n) {
            const ssize_t got = pread(g->fd, (uint8_t *)g->pinned[k] + done, (size_t)(n - done), (off_t)(off + done));
            if (got <= 0) return QM_ERR_STATE;
            done += (uint64_t)got;
        }
        DRV(d->cuMemcpyHtoDAsync_v2(g->stage[k], g->pinned[k], (size_t)n, c->stream));
        rc = qm_store_write_rows_device(c, w, dst_row + (r0 - row_lo), nr, (uint64_t)g->stage[k], (int64_t)n);
        if (rc) return rc;
        DRV(d->cuEventRecord(g->done[k], c->stream));
        used[k] = true;
    }
    DRV(d->cuStreamSynchronize(c->stream));
    return QM_OK;
}

// A whole store entry from rows [row_lo, row_hi) of one tensor (row_hi = 0: all rows).
extern "C" int32_t qm_gguf_load_tensor(qm_ctx *c, qm_gguf *g, int32_t index, int64_t row_lo, int64_t row_hi,
                                       qm_weight *out) {
    CHECK_CTX(c);
    if (!out || !g || g->magic != QM_GGUF_MAGIC || index < 0 || (size_t)index >= g->tensors.size()) return QM_ERR_ARG;
    *out = 0;
    const GgufTensor &t = g->tensors[(size_t)index];
    const int64_t rows = (int64_t)(t.dims[1] * t.dims[2] * t.dims[3]);
    if (row_hi == 0) row_hi = rows;
    if (row_lo < 0 || row_hi > rows || row_lo >= row_hi) return QM_ERR_SHAPE;
    qm_weight w = 0;
    int32_t rc = qm_store_create(c, (int32_t)t.type_id, row_hi - row_lo, (int64_t)t.dims[0], &w);
    if (rc) return rc;
    rc = qm_gguf_load_rows(c, g, index, row_lo, row_hi, w, 0);
    if (rc) {
        qm_store_free(c, w);
        return rc;
    }
    *out = w;
    return QM_OK;
}
