// See cache.hpp.
#include "cache.hpp"

#include <cuda_runtime.h>

#include <algorithm>
#include <set>

#include "device.hpp"

namespace fg {

PagedKVCache::PagedKVCache(const std::map<int, CacheRequest> &requests, int64_t max_tokens, int max_seq_len_, int n_slots_,
                           int page_size_)
    : page_size(page_size_), n_slots(n_slots_), max_seq_len(max_seq_len_) {
    if (page_size <= 0 || max_tokens <= 0 || n_slots <= 0)
        fail(FG_E_USAGE, "page_size, max_tokens and n_slots must be positive");
    int64_t n_pages = (max_tokens + page_size - 1) / page_size + 1;      // + the reserved page 0
    if (n_pages > 0x7fffffff) fail(FG_E_USAGE, "max_tokens is too large for 32-bit page ids");
    for (auto &kv : requests) {                                          // std::map: ascending entries
        bool placed = false;
        for (size_t gi = 0; gi < groups.size(); gi++) {
            if (groups[gi].request == kv.second) {
                groups[gi].entries.push_back(kv.first);
                group_of_entry[kv.first] = (int)gi;
                placed = true;
                break;
            }
        }
        if (!placed) {
            CacheGroup g;
            g.request = kv.second;
            g.entries.push_back(kv.first);
            g.n_pages = (int)n_pages;
            groups.push_back(std::move(g));
            group_of_entry[kv.first] = (int)groups.size() - 1;
        }
    }
    for (auto &g : groups) {
        g.free.reserve((size_t)g.n_pages);
        for (int p = g.n_pages - 1; p >= 1; p--) g.free.push_back(p);   // pop_back hands out low ids first
        for (int e : g.entries) g.k_pools[e] = g.v_pools[e] = nullptr;
    }
    slots_.resize((size_t)n_slots);
    for (auto &s : slots_) s.pages.resize(groups.size());
    for (int s = n_slots - 1; s >= 0; s--) free_slots_.push_back(s);
}

PagedKVCache::~PagedKVCache() {
    if (storage_) cudaFree(storage_);
}

static int64_t pool_elems(const CacheGroup &g, int page_size) {
    return (int64_t)g.n_pages * g.request.n_kv_heads * page_size * g.request.head_dim;
}

int64_t PagedKVCache::pool_bytes(int dtype) const {
    int64_t total = 0;
    for (auto &g : groups) {
        int64_t one = (pool_elems(g, page_size) * elem_size(dtype) + 255) / 256 * 256;
        total += 2 * one * (int64_t)g.entries.size();
    }
    return total;
}

int64_t PagedKVCache::bytes_per_token(int dtype) const {
    int64_t b = 0;
    for (auto &g : groups) b += 2LL * g.request.n_kv_heads * g.request.head_dim * elem_size(dtype) * (int64_t)g.entries.size();
    return b;
}

void PagedKVCache::allocate(int dtype) {
    if (storage_) fail(FG_E_INTERNAL, "the cache is allocated already");
    int64_t need = pool_bytes(dtype);
    dtype_ = dtype;
    if (need == 0) return;
    size_t free_b = 0, total_b = 0;
    FG_CUDA(cudaMemGetInfo(&free_b, &total_b));
    if ((uint64_t)need > free_b)
        fail(FG_E_DEVICE, format("the cache does not fit: %lld pages of %d tokens at %lld bytes a token need %.1f MiB, "
                                 "%.1f MiB of device memory are free (lower max_tokens)",
                                 groups.empty() ? 0LL : (long long)groups[0].n_pages - 1, page_size,
                                 (long long)bytes_per_token(dtype), need / 1048576.0, free_b / 1048576.0));
    cudaError_t e = cudaMalloc(&storage_, (size_t)need);
    if (e != cudaSuccess) {
        cudaGetLastError();
        storage_ = nullptr;
        fail(FG_E_DEVICE, format("the cache does not fit: cudaMalloc of %.1f MiB failed (%s)", need / 1048576.0,
                                 cudaGetErrorString(e)));
    }
    FG_CUDA(cudaMemset(storage_, 0, (size_t)need));
    char *p = (char *)storage_;
    for (auto &g : groups) {
        int64_t one = (pool_elems(g, page_size) * elem_size(dtype) + 255) / 256 * 256;
        for (int entry : g.entries) {
            g.k_pools[entry] = p; p += one;
            g.v_pools[entry] = p; p += one;
        }
    }
}

// ------------------------------------------------------------------------------------ slots
int PagedKVCache::acquire() {
    if (free_slots_.empty()) fail(FG_E_CAPACITY, format("all %d sequence slots are in use", n_slots));
    int s = free_slots_.back();
    free_slots_.pop_back();
    Slot &sl = slots_[(size_t)s];
    bool clean = !sl.live && sl.length == 0;
    for (auto &p : sl.pages) clean = clean && p.empty();
    if (!clean) fail(FG_E_INTERNAL, format("slot %d was on the free list but is not empty", s));
    sl.live = true;
    return s;
}

void PagedKVCache::release(int s) {
    Slot &sl = slot(s);
    for (size_t gi = 0; gi < groups.size(); gi++) {
        for (auto &kv : sl.pages[gi]) groups[gi].free.push_back(kv.second);
        sl.pages[gi].clear();
    }
    sl.length = 0;
    sl.live = false;
    free_slots_.push_back(s);
}

PagedKVCache::Slot &PagedKVCache::slot(int s) {
    if (s < 0 || s >= n_slots) fail(FG_E_CACHE, format("slot %d does not exist (there are %d)", s, n_slots));
    Slot &sl = slots_[(size_t)s];
    if (!sl.live) fail(FG_E_CACHE, format("slot %d is not held by a sequence (released twice, or never acquired)", s));
    return sl;
}
const PagedKVCache::Slot &PagedKVCache::slot(int s) const { return const_cast<PagedKVCache *>(this)->slot(s); }

int PagedKVCache::length(int s) const { return slot(s).length; }

std::vector<int> PagedKVCache::live_slots() const {
    std::vector<int> out;
    for (int i = 0; i < n_slots; i++)
        if (slots_[(size_t)i].live) out.push_back(i);
    return out;
}

// ------------------------------------------------------------------------------------ pages
// Index (within a sequence) of the first page that a sequence of `new_length` still reads: the oldest
// position any row of the NEXT step can see is new_length - window + 1 at the least, and pages are dropped
// at commit, by the length after the step.
int PagedKVCache::first_needed_page(const CacheGroup &g, int new_length) const {
    if (g.request.window <= 0) return 0;
    return std::max(0, new_length - g.request.window) / page_size;
}

std::vector<int> PagedKVCache::pages_needed(int s, int n_new) const {
    const Slot &sl = slot(s);
    std::vector<int> out;
    for (size_t gi = 0; gi < groups.size(); gi++) {
        int first = sl.length / page_size, last = (sl.length + n_new - 1) / page_size, n = 0;
        for (int p = first; p <= last; p++)
            if (!sl.pages[gi].count(p)) n++;
        out.push_back(n);
    }
    return out;
}

void PagedKVCache::reserve(const std::vector<std::pair<int, int>> &steps) {
    std::vector<int> need(groups.size(), 0);
    std::set<int> seen;
    for (auto &st : steps) {
        int s = st.first, n_new = st.second;
        if (seen.count(s)) fail(FG_E_CACHE, format("slot %d appears twice in one step", s));
        seen.insert(s);
        const Slot &sl = slot(s);
        if (n_new <= 0) fail(FG_E_CACHE, format("slot %d: a step must bring at least one token", s));
        if ((int64_t)sl.length + n_new > max_seq_len)
            fail(FG_E_CAPACITY, format("slot %d: %d + %d tokens exceed the longest sequence the cache was sized for (%d)", s,
                                       sl.length, n_new, max_seq_len));
        std::vector<int> pn = pages_needed(s, n_new);
        for (size_t gi = 0; gi < groups.size(); gi++) need[gi] += pn[gi];
    }
    for (size_t gi = 0; gi < groups.size(); gi++)
        if (need[gi] > (int)groups[gi].free.size())
            fail(FG_E_CAPACITY, format("cache group %zu needs %d more pages of %d tokens, %zu are free", gi, need[gi], page_size,
                                       groups[gi].free.size()));
    for (auto &st : steps) {
        Slot &sl = slots_[(size_t)st.first];
        for (size_t gi = 0; gi < groups.size(); gi++) {
            int first = sl.length / page_size, last = (sl.length + st.second - 1) / page_size;
            for (int p = first; p <= last; p++) {
                if (!sl.pages[gi].count(p)) {
                    sl.pages[gi][p] = groups[gi].free.back();
                    groups[gi].free.pop_back();
                }
            }
        }
    }
}

void PagedKVCache::commit(const std::vector<std::pair<int, int>> &steps) {
    for (auto &st : steps) {
        Slot &sl = slot(st.first);
        sl.length += st.second;
        for (size_t gi = 0; gi < groups.size(); gi++) {
            if (groups[gi].request.window <= 0) continue;
            int keep_from = first_needed_page(groups[gi], sl.length);
            for (auto it = sl.pages[gi].begin(); it != sl.pages[gi].end() && it->first < keep_from;) {
                groups[gi].free.push_back(it->second);
                it = sl.pages[gi].erase(it);
            }
        }
    }
}

void PagedKVCache::block_table(int gi, int s, int width, int *out) const {
    if (gi < 0 || gi >= (int)groups.size()) fail(FG_E_USAGE, format("cache group %d does not exist", gi));
    if (s < 0 || s >= n_slots) fail(FG_E_CACHE, format("slot %d does not exist (there are %d)", s, n_slots));
    for (int i = 0; i < width; i++) out[i] = 0;
    for (auto &kv : slots_[(size_t)s].pages[(size_t)gi])
        if (kv.first < width) out[kv.first] = kv.second;
}

int PagedKVCache::free_pages(int gi) const {
    if (gi < 0 || gi >= (int)groups.size()) fail(FG_E_USAGE, format("cache group %d does not exist", gi));
    return (int)groups[(size_t)gi].free.size();
}

void PagedKVCache::check() const {
    for (size_t gi = 0; gi < groups.size(); gi++) {
        const CacheGroup &g = groups[gi];
        std::vector<int> all(g.free.begin(), g.free.end());
        size_t held = 0;
        for (int si = 0; si < n_slots; si++) {
            const Slot &sl = slots_[(size_t)si];
            if (!sl.live && !sl.pages[gi].empty())
                fail(FG_E_CACHE, format("slot %d is free but still holds pages of group %zu", si, gi));
            for (auto &kv : sl.pages[gi]) { all.push_back(kv.second); held++; }
        }
        std::sort(all.begin(), all.end());
        bool ok = (int)all.size() == g.n_pages - 1;
        for (size_t i = 0; ok && i < all.size(); i++) ok = all[i] == (int)i + 1;
        if (!ok)
            fail(FG_E_CACHE, format("group %zu: pages are lost or duplicated (%zu held + %zu free of %d)", gi, held, g.free.size(),
                                    g.n_pages - 1));
    }
    std::vector<int> all(free_slots_);
    for (int i = 0; i < n_slots; i++)
        if (slots_[(size_t)i].live) all.push_back(i);
    std::sort(all.begin(), all.end());
    bool ok = (int)all.size() == n_slots;
    for (size_t i = 0; ok && i < all.size(); i++) ok = all[i] == (int)i;
    if (!ok) fail(FG_E_CACHE, "a slot is lost, or both free and live");
}

Json PagedKVCache::info() const {
    Json j = Json::object();
    j.set("page_size", page_size);
    j.set("n_slots", n_slots);
    j.set("max_seq_len", max_seq_len);
    Json gs = Json::array();
    for (auto &g : groups) {
        Json o = Json::object();
        o.set("n_kv_heads", g.request.n_kv_heads);
        o.set("head_dim", g.request.head_dim);
        o.set("window", g.request.window > 0 ? Json(g.request.window) : Json());
        Json es = Json::array();
        for (int e : g.entries) es.push(Json(e));
        o.set("entries", es);
        o.set("pages", g.n_pages - 1);
        o.set("free_pages", (long long)g.free.size());
        gs.push(o);
    }
    j.set("groups", gs);
    Json live = Json::array();
    for (int s : live_slots()) live.push(Json(s));
    j.set("live_slots", live);
    return j;
}

// ------------------------------------------------------------------------------------ state
StatePool::StatePool(const std::map<int, int64_t> &bytes_of_entry, int n_slots_, bool allocate) : n_slots(n_slots_) {
    int64_t total = 0;
    for (auto &kv : bytes_of_entry) {
        int64_t b = (kv.second + 15) / 16 * 16;
        bytes_[kv.first] = b;
        total += (b * (n_slots + 1) + 255) / 256 * 256;
    }
    if (!allocate || total == 0) return;
    FG_CUDA(cudaMalloc(&storage_, (size_t)total));
    FG_CUDA(cudaMemset(storage_, 0, (size_t)total));
    char *p = (char *)storage_;
    for (auto &kv : bytes_) {
        ptr_[kv.first] = p;
        p += (kv.second * (n_slots + 1) + 255) / 256 * 256;
    }
}
StatePool::~StatePool() {
    if (storage_) cudaFree(storage_);
}
void StatePool::reset(int slot, void *stream) {
    for (auto &kv : ptr_) {
        int64_t b = bytes_[kv.first];
        FG_CUDA(cudaMemsetAsync((char *)kv.second + b * slot, 0, (size_t)b, (cudaStream_t)stream));
    }
}
void *StatePool::of(int entry) const {
    auto it = ptr_.find(entry);
    return it == ptr_.end() ? nullptr : it->second;
}
int64_t StatePool::bytes_of(int entry) const {
    auto it = bytes_.find(entry);
    return it == bytes_.end() ? 0 : it->second;
}
int64_t StatePool::total_bytes() const {
    int64_t t = 0;
    for (auto &kv : bytes_) t += kv.second * (n_slots + 1);
    return t;
}

std::map<int, CacheRequest> cache_requests_from_json(const Json &j) {
    if (!j.is_array()) fail(FG_E_USAGE, "cache requests must be a list of {entry, n_kv_heads, head_dim, window}");
    std::map<int, CacheRequest> out;
    for (auto &r : j.items()) {
        if (!r.is_object() || !r.get("entry").is_int() || !r.get("n_kv_heads").is_int() || !r.get("head_dim").is_int())
            fail(FG_E_USAGE, "a cache request needs integer entry, n_kv_heads and head_dim");
        CacheRequest c;
        c.n_kv_heads = (int)r.get("n_kv_heads").as_int();
        c.head_dim = (int)r.get("head_dim").as_int();
        c.window = r.get("window").is_int() ? (int)r.get("window").as_int() : 0;
        out[(int)r.get("entry").as_int()] = c;
    }
    return out;
}

}  // namespace fg
