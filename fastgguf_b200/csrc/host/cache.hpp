// The cache: a slot per sequence, pages of keys and values per layer group, and per-sequence state of
// fixed size.
//
// The reference keeps, per layer that owns a cache, two float arrays [capacity][kv_dim] written at
// pos % capacity (fastgguf.c:4114-4115, :4449-4450, :4720), for ONE sequence per model; sliding-window
// layers get a short ring of their own while global layers get the full context (:4427-4436), shared-KV
// layers own nothing and read a donor's arrays (:4745-4751), and it prints the cache's size at load
// (:4561-4565).  Per-sequence scalars (position, RNG) are scattered over locals and structs (:5243, :3974).
//
// Here many sequences share the storage:
//   * a slot per live sequence holds its length and, per cache group, the pages it owns;
//   * a cache group is the set of schedule entries whose mixers asked for the same (KV heads, head size,
//     window); it has storage of its own - one pool per entry, [pages, kv_heads, page_size, head_dim] -
//     and one page table per sequence, so a full-attention group and a windowed group never share pages;
//   * a windowed group gives pages back as soon as every position in them has left the window;
//   * page 0 of every group is never handed out: padded rows of a fixed-shape step write there;
//   * StatePool keeps [n_slots + 1, bytes] per schedule entry that asked for fixed-size state; a slot's
//     rows are zeroed when a sequence takes the slot, and the last row is a spare for padded rows.
// All bookkeeping is on the host and checked: a page or a slot can neither be lost, held twice nor freed
// twice (check() proves it).
#pragma once
#include <cstdint>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "errors.hpp"
#include "json.hpp"

namespace fg {

struct CacheRequest {
    int n_kv_heads = 0, head_dim = 0;
    int window = 0;                           // 0 keeps every position; w keeps the last w
    bool operator==(const CacheRequest &o) const {
        return n_kv_heads == o.n_kv_heads && head_dim == o.head_dim && window == o.window;
    }
};

struct CacheGroup {
    CacheRequest request;
    std::vector<int> entries;                 // schedule entries that own a pool in this group
    int n_pages = 0;                          // pages in each pool, the reserved page 0 included
    std::vector<int> free;
    std::map<int, void *> k_pools, v_pools;   // entry -> device pointer (null without device memory)
};

class PagedKVCache {
public:
    // requests: schedule entry -> what its mixer keeps.  max_tokens: most tokens held by live sequences at
    // any time, each sequence counted rounded up to a page.
    PagedKVCache(const std::map<int, CacheRequest> &requests, int64_t max_tokens, int max_seq_len, int n_slots,
                 int page_size);
    ~PagedKVCache();
    PagedKVCache(const PagedKVCache &) = delete;

    // bytes the pools take in `dtype`; nothing is allocated
    int64_t pool_bytes(int dtype) const;
    int64_t bytes_per_token(int dtype) const;
    // ONE device allocation for every pool, zeroed; throws FG_E_DEVICE naming need and free memory if it
    // does not fit (checked BEFORE allocating)
    void allocate(int dtype);
    int dtype() const { return dtype_; }

    int acquire();
    void release(int slot);
    int length(int slot) const;
    std::vector<int> live_slots() const;
    std::vector<int> pages_needed(int slot, int n_new) const;
    void reserve(const std::vector<std::pair<int, int>> &steps);      // all or nothing
    void commit(const std::vector<std::pair<int, int>> &steps);
    // table[gi][slot, 0 .. width): page ids, 0 where none
    void block_table(int gi, int slot, int width, int *out) const;
    int free_pages(int gi) const;
    void check() const;
    Json info() const;

    int page_size, n_slots, max_seq_len;
    std::vector<CacheGroup> groups;
    std::map<int, int> group_of_entry;

private:
    struct Slot {
        int length = 0;
        bool live = false;
        std::vector<std::map<int, int>> pages;   // per group: page index in the sequence -> page id
    };
    Slot &slot(int s);
    const Slot &slot(int s) const;
    int first_needed_page(const CacheGroup &g, int new_length) const;
    std::vector<Slot> slots_;
    std::vector<int> free_slots_;
    void *storage_ = nullptr;
    int dtype_ = -1;
};

// Fixed-size per-sequence state: [n_slots + 1, bytes] per schedule entry that asked for it.
class StatePool {
public:
    StatePool(const std::map<int, int64_t> &bytes_of_entry, int n_slots, bool allocate);
    ~StatePool();
    StatePool(const StatePool &) = delete;
    void reset(int slot, void *stream);           // zero the slot's row of every entry
    void *of(int entry) const;
    int64_t bytes_of(int entry) const;
    int64_t total_bytes() const;
    int n_slots;

private:
    std::map<int, int64_t> bytes_;
    std::map<int, void *> ptr_;
    void *storage_ = nullptr;
};

std::map<int, CacheRequest> cache_requests_from_json(const Json &j);

}  // namespace fg
