// qm_expert_pool.cpp — device-side residency of experts over the host cache of
// qm_expert_cache.cpp: at most max_resident experts hold a device store entry, a request for
// another one overwrites the least recently used entry (never the one just touched) with the
// expert's bytes, which the host cache hands out from memory or from its spill file. The
// reference keeps experts in host memory and files only (moe.ExpertCacheManager,
// lm/moe/moe.go:143-287); this is the same policy one level further down, for models whose
// experts do not all fit in HBM.
//
// The entries are allocated once, so paging an expert in is a copy and a repack on the context's
// stream (qm_store_write_rows, which waits for the stream: kernels launched earlier have read the
// old contents by then, kernels launched later read the new ones) and nothing is allocated or freed.
#include <stdint.h>
#include <string.h>

#include <map>
#include <new>
#include <vector>

#include "qm_internal.h"

struct qm_expert_pool {
    uint32_t magic;
    qm_expert_cache *host;
    int32_t fmt;
    int64_t rows, cols, blob_bytes;
    std::vector<qm_weight> slot;        // device store entries, all of one shape
    std::vector<int64_t> slot_expert;   // expert held by each entry, -1: none
    std::vector<uint64_t> slot_used;    // access clock at last use
    std::map<int64_t, int> where;       // expert -> entry
    std::vector<uint8_t> staging;       // one expert's GGUF bytes on their way to the device
    uint64_t clock;
    int64_t hits, misses;
};
#define QM_POOL_MAGIC 0x514D504Cu   // "QMPL"

extern "C" int32_t qm_expert_pool_close(qm_ctx *c, qm_expert_pool *p) {
    CHECK_CTX(c);
    if (!p || p->magic != QM_POOL_MAGIC) return QM_ERR_ARG;
    int32_t rc = qm_sync(c);   // the entries may still be read
    for (qm_weight w : p->slot)
        if (w) {
            const int32_t r = qm_store_free(c, w);
            if (r && !rc) rc = r;
        }
    p->magic = 0;
    delete p;
    return rc;
}

extern "C" int32_t qm_expert_pool_create(qm_ctx *c, qm_expert_cache *host, int32_t fmt, int64_t rows, int64_t cols,
                                         int32_t max_resident, qm_expert_pool **out) {
    CHECK_CTX(c);
    if (!out) return QM_ERR_ARG;
    *out = nullptr;
    if (!host || max_resident <= 0) return QM_ERR_ARG;   // "maxHot must be positive" (lm/moe/moe.go:160-162)
    qm_expert_pool *p = new (std::nothrow) qm_expert_pool();
    if (!p) return QM_ERR_NOMEM;
    p->magic = QM_POOL_MAGIC;
    p->host = host;
    p->fmt = fmt;
    p->rows = rows;
    p->cols = cols;
    p->clock = 0;
    p->hits = p->misses = 0;
    for (int i = 0; i < max_resident; i++) {
        qm_weight w = 0;
        const int32_t rc = qm_store_create(c, fmt, rows, cols, &w);   // also checks format and shape
        if (rc) {
            qm_expert_pool_close(c, p);
            return rc;
        }
        p->slot.push_back(w);
        p->slot_expert.push_back(-1);
        p->slot_used.push_back(0);
    }
    int64_t info[5];
    const int32_t rc = qm_store_info(c, p->slot[0], info);
    if (rc) {
        qm_expert_pool_close(c, p);
        return rc;
    }
    p->blob_bytes = info[4];
    p->staging.resize((size_t)p->blob_bytes);
    *out = p;
    return QM_OK;
}

// The device entry that holds `expert`, paging it in first if need be. QM_ERR_ARG when the host cache does not
// know the expert, QM_ERR_BUFFER when its blob is not rows x cols of the pool's format.
extern "C" int32_t qm_expert_pool_get(qm_ctx *c, qm_expert_pool *p, int64_t expert, qm_weight *out) {
    CHECK_CTX(c);
    if (!p || p->magic != QM_POOL_MAGIC || !out || expert < 0) return QM_ERR_ARG;
    *out = 0;
    auto it = p->where.find(expert);
    if (it != p->where.end()) {
        p->slot_used[it->second] = ++p->clock;
        p->hits++;
        *out = p->slot[it->second];
        return QM_OK;
    }
    int64_t size = 0;
    int32_t rc = qm_expert_cache_get(p->host, expert, p->staging.data(), p->blob_bytes, &size);
    if (rc) return rc;
    if (size != p->blob_bytes) return QM_ERR_BUFFER;
    int victim = 0;   // an empty entry, else the least recently used one
    for (int i = 0; i < (int)p->slot.size(); i++) {
        if (p->slot_expert[i] < 0) { victim = i; break; }
        if (p->slot_used[i] < p->slot_used[victim]) victim = i;
    }
    // qm_store_write_rows copies from pageable memory: the bytes have left `staging` when it returns
    rc = qm_store_write_rows(c, p->slot[victim], 0, p->rows, p->staging.data(), p->blob_bytes);
    if (rc) return rc;
    if (p->slot_expert[victim] >= 0) p->where.erase(p->slot_expert[victim]);
    p->slot_expert[victim] = expert;
    p->slot_used[victim] = ++p->clock;
    p->where[expert] = victim;
    p->misses++;
    *out = p->slot[victim];
    return QM_OK;
}

// info[0] = experts resident, [1] = entries, [2] = hits, [3] = misses (= experts paged in)
extern "C" int32_t qm_expert_pool_info(qm_expert_pool *p, int64_t *info4) {
    if (!p || p->magic != QM_POOL_MAGIC || !info4) return QM_ERR_ARG;
    info4[0] = (int64_t)p->where.size();
    info4[1] = (int64_t)p->slot.size();
    info4[2] = p->hits;
    info4[3] = p->misses;
    return QM_OK;
}

// Drops an expert from the device (its entry becomes free); unknown or absent experts are not an error, as
// EvictColdExpert's are not (lm/moe/moe.go:229-248).
extern "C" int32_t qm_expert_pool_evict(qm_expert_pool *p, int64_t expert) {
    if (!p || p->magic != QM_POOL_MAGIC) return QM_ERR_ARG;
    auto it = p->where.find(expert);
    if (it == p->where.end()) return QM_OK;
    p->slot_expert[it->second] = -1;
    p->slot_used[it->second] = 0;
    p->where.erase(it);
    return QM_OK;
}
