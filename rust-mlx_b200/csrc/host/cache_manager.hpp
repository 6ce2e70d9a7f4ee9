// The cache manager: pages of keys and values with a block table per request, one pool
// per group of layers with the same needs, and slots for per-request state of fixed size.
//
// The reference keeps one growing contiguous K and V per request and layer
// (src/dense.rs:27-111, optionally in 256-position blocks, src/kv_blocks.rs:19) and a
// per-layer enum of cache kinds for its hybrid model (src/hybrid.rs:510-514).  Here a
// token at position p of a request lives in page table[p / page_size], slot
// p % page_size, of its group's pool.  The manager only does the bookkeeping: which
// page ids and which state slot a request holds; the tensors live with the engine.
#pragma once
#include <cstdint>
#include <unordered_map>
#include <vector>

namespace rmx {

struct GroupConfig {
    int num_pages;
    int page_size;
    int window;  // 0: every key is kept; > 0: positions below len - window + 1 are never read again
};

enum Status : int {
    OK = 0,
    NO_PAGES = -1,
    NO_SLOT = -2,
    UNKNOWN_REQUEST = -3,
    BAD_LENGTH = -4,
    DUPLICATE_REQUEST = -5,
    BAD_ARGUMENT = -6,
    INVARIANT_BROKEN = -7,
};

class CacheManager {
public:
    CacheManager(const std::vector<GroupConfig>& groups, int max_requests);

    int num_groups() const { return (int)groups_.size(); }
    const GroupConfig& group(int g) const { return groups_[g]; }
    int free_pages(int g) const { return (int)free_[g].size(); }
    int free_slots() const { return (int)free_slots_.size(); }
    int live() const { return (int)requests_.size(); }
    bool has(int64_t id) const { return requests_.count(id) != 0; }

    // Take a state slot for a new request: the slot index, or NO_SLOT / DUPLICATE_REQUEST.
    int open(int64_t id);
    // Make room for positions len .. new_len - 1 in every group, all or nothing.
    int reserve(int64_t id, int new_len);
    // The largest length <= want that reserve() would accept now.
    int max_reservable(int64_t id, int want) const;
    // The request now holds new_len tokens (<= what was reserved).  Pages that a window has
    // passed are given back; returns how many.
    int commit(int64_t id, int new_len);
    // Give back everything the request holds; returns the number of pages freed.
    int close(int64_t id);
    // Give back what was reserved beyond the committed length (a step that did not run).
    int release_reserved(int64_t id);

    int length(int64_t id) const;
    int reserved(int64_t id) const;
    int slot(int64_t id) const;
    // Copy the block table of group g: entry i is the page of positions i*page_size ..,
    // or -1 where the request holds none.  Returns the number of entries, or an error.
    int table(int64_t id, int g, int32_t* out, int capacity) const;
    int pages_held(int64_t id, int g) const;
    // Pages a request of `len` tokens needs at most in group g at one time when it is fed
    // in portions of at most `portion` tokens.
    int peak_pages(int g, int len, int portion) const;

    // 0 if every page of every group is either free once or held once, else INVARIANT_BROKEN.
    int check() const;

private:
    struct Request {
        int slot = -1;
        int len = 0;        // committed tokens
        int reserved = 0;   // tokens there is room for
        std::vector<std::vector<int32_t>> tables;  // per group: logical page -> page id or -1
        std::vector<int> first_live;               // per group: first logical page still held
    };
    std::vector<GroupConfig> groups_;
    std::vector<std::vector<int32_t>> free_;  // per group, used as a stack: last freed is reused first
    std::vector<int> free_slots_;
    std::unordered_map<int64_t, Request> requests_;
};

}  // namespace rmx
