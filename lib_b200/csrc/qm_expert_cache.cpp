// qm_expert_cache.cpp — host-side residency manager for expert weight blobs: at most
// max_hot experts stay in memory, the least recently used one is spilled to a file
// "expert_<id>.bin" when an admission exceeds that, and a cold expert is paged back in on
// demand. Same behaviour as moe.ExpertCacheManager (lm/moe/moe.go:143-287: RegisterExpert,
// GetExpert, HotExperts, EvictColdExpert, Close; the most recently touched expert is never the
// victim, lm/moe/moe.go:229-248). It is the host source of the bytes that qm_store_upload
// turns into device-resident experts; nothing here touches the GPU.
#include <errno.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/stat.h>
#include <unistd.h>

#include <map>
#include <mutex>
#include <new>
#include <string>
#include <vector>

#include "../../include/qmatmul.h"

struct qm_expert_cache {
    std::string dir;
    int max_hot;
    std::map<int64_t, std::vector<uint8_t>> hot;   // expert -> weight bytes
    std::map<int64_t, std::string> cold;           // expert -> spill file
    std::map<int64_t, uint64_t> last_used;         // expert -> access clock at last use
    uint64_t clock;
    std::mutex mu;
};

namespace {

int mkdirs(const std::string &path) {
    std::string cur;
    for (size_t i = 0; i <= path.size(); i++) {
        if (i == path.size() || path[i] == '/') {
            if (!cur.empty() && mkdir(cur.c_str(), 0700) != 0 && errno != EEXIST) return -1;
        }
        if (i < path.size()) cur.push_back(path[i]);
    }
    return 0;
}

void touch(qm_expert_cache *m, int64_t id) { m->last_used[id] = ++m->clock; }

int32_t evict(qm_expert_cache *m, int64_t id) {
    auto it = m->hot.find(id);
    if (it == m->hot.end()) return QM_OK;
    const std::string path = m->dir + "/expert_" + std::to_string((long long)id) + ".bin";
    FILE *f = fopen(path.c_str(), "wb");
    if (!f) return QM_ERR_STATE;
    const size_t n = it->second.size();
    const bool ok = (n == 0 || fwrite(it->second.data(), 1, n, f) == n);
    if (fclose(f) != 0 || !ok) return QM_ERR_STATE;
    chmod(path.c_str(), 0600);
    m->hot.erase(it);
    m->cold[id] = path;
    return QM_OK;
}

// Spills least recently used experts until at most max_hot are resident.
int32_t trim(qm_expert_cache *m) {
    while ((int)m->hot.size() > m->max_hot) {
        int64_t victim = 0;
        uint64_t oldest = UINT64_MAX;
        bool found = false;
        for (const auto &kv : m->hot) {
            const uint64_t use = m->last_used[kv.first];
            if (use < oldest) {
                oldest = use;
                victim = kv.first;
                found = true;
            }
        }
        if (!found) return QM_OK;
        const int32_t rc = evict(m, victim);
        if (rc) return rc;
    }
    return QM_OK;
}

}  // namespace

extern "C" int32_t qm_expert_cache_create(const char *dir, int32_t max_hot, qm_expert_cache **out) {
    if (!out) return QM_ERR_ARG;
    *out = nullptr;
    if (max_hot <= 0) return QM_ERR_ARG;   // "maxHot must be positive" (lm/moe/moe.go:160-162)
    std::string d = (dir && *dir) ? dir : "";
    if (d.empty()) {
        const char *tmp = getenv("TMPDIR");
        d = std::string(tmp && *tmp ? tmp : "/tmp") + "/lm-expert-cache";
    }
    if (mkdirs(d) != 0) return QM_ERR_STATE;
    qm_expert_cache *m = new (std::nothrow) qm_expert_cache();
    if (!m) return QM_ERR_NOMEM;
    m->dir = d;
    m->max_hot = max_hot;
    m->clock = 0;
    *out = m;
    return QM_OK;
}

extern "C" int32_t qm_expert_cache_register(qm_expert_cache *m, int64_t expert, const void *bytes, int64_t n) {
    if (!m || n < 0 || (n > 0 && !bytes)) return QM_ERR_ARG;
    std::lock_guard<std::mutex> g(m->mu);
    const uint8_t *p = static_cast<const uint8_t *>(bytes);
    m->hot[expert] = std::vector<uint8_t>(p, p + n);
    touch(m, expert);
    return trim(m);
}

// Size of an expert's blob, paging it in if it is cold (so that a following qm_expert_cache_get
// with a buffer of that size cannot be surprised). QM_ERR_ARG when the expert is unknown.
extern "C" int32_t qm_expert_cache_get(qm_expert_cache *m, int64_t expert, void *out, int64_t capacity,
                                       int64_t *size) {
    if (!m || !size) return QM_ERR_ARG;
    std::lock_guard<std::mutex> g(m->mu);
    auto it = m->hot.find(expert);
    if (it == m->hot.end()) {
        auto c = m->cold.find(expert);
        if (c == m->cold.end()) return QM_ERR_ARG;   // "not found in memory or disk"
        FILE *f = fopen(c->second.c_str(), "rb");
        if (!f) return QM_ERR_STATE;
        std::vector<uint8_t> data;
        uint8_t buf[65536];
        size_t got;
        while ((got = fread(buf, 1, sizeof buf, f)) > 0) data.insert(data.end(), buf, buf + got);
        const bool bad = ferror(f) != 0;
        fclose(f);
        if (bad) return QM_ERR_STATE;
        m->hot[expert] = std::move(data);
        touch(m, expert);
        const int32_t rc = trim(m);
        if (rc) return rc;
        it = m->hot.find(expert);
    } else {
        touch(m, expert);
    }
    *size = (int64_t)it->second.size();
    if (out) {
        if (capacity < *size) return QM_ERR_BUFFER;
        if (*size) memcpy(out, it->second.data(), (size_t)*size);
    }
    return QM_OK;
}

extern "C" int32_t qm_expert_cache_hot(qm_expert_cache *m) {
    if (!m) return QM_ERR_ARG;
    std::lock_guard<std::mutex> g(m->mu);
    return (int32_t)m->hot.size();
}

extern "C" int32_t qm_expert_cache_evict(qm_expert_cache *m, int64_t expert) {
    if (!m) return QM_ERR_ARG;
    std::lock_guard<std::mutex> g(m->mu);
    return evict(m, expert);
}

// Removes the spilled files and frees the cache.
extern "C" int32_t qm_expert_cache_close(qm_expert_cache *m) {
    if (!m) return QM_ERR_ARG;
    int32_t rc = QM_OK;
    {
        std::lock_guard<std::mutex> g(m->mu);
        for (const auto &kv : m->cold)
            if (unlink(kv.second.c_str()) != 0 && errno != ENOENT && rc == QM_OK) rc = QM_ERR_STATE;
        m->cold.clear();
    }
    delete m;
    return rc;
}
