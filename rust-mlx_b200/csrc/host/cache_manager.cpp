#include "cache_manager.hpp"

#include <algorithm>

namespace rmx {

static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

CacheManager::CacheManager(const std::vector<GroupConfig>& groups, int max_requests) : groups_(groups) {
    free_.resize(groups_.size());
    for (size_t g = 0; g < groups_.size(); ++g) {
        // page 0 on top of the stack, so a fresh pool hands out 0, 1, 2, ...
        for (int p = groups_[g].num_pages - 1; p >= 0; --p) free_[g].push_back(p);
    }
    for (int s = max_requests - 1; s >= 0; --s) free_slots_.push_back(s);
}

int CacheManager::open(int64_t id) {
    if (requests_.count(id)) return DUPLICATE_REQUEST;
    if (free_slots_.empty()) return NO_SLOT;
    Request r;
    r.slot = free_slots_.back();
    free_slots_.pop_back();
    r.tables.resize(groups_.size());
    r.first_live.assign(groups_.size(), 0);
    requests_.emplace(id, std::move(r));
    return requests_[id].slot;
}

int CacheManager::max_reservable(int64_t id, int want) const {
    auto it = requests_.find(id);
    if (it == requests_.end()) return UNKNOWN_REQUEST;
    const Request& r = it->second;
    int best = want;
    for (size_t g = 0; g < groups_.size(); ++g) {
        const long long room = ((long long)r.tables[g].size() + (long long)free_[g].size()) * groups_[g].page_size;
        if (room < best) best = (int)room;
    }
    return std::max(best, r.reserved);
}

int CacheManager::reserve(int64_t id, int new_len) {
    auto it = requests_.find(id);
    if (it == requests_.end()) return UNKNOWN_REQUEST;
    Request& r = it->second;
    if (new_len < r.len) return BAD_LENGTH;
    if (new_len <= r.reserved) return OK;
    for (size_t g = 0; g < groups_.size(); ++g) {
        const int need = ceil_div(new_len, groups_[g].page_size) - (int)r.tables[g].size();
        if (need > (int)free_[g].size()) return NO_PAGES;
    }
    for (size_t g = 0; g < groups_.size(); ++g) {
        const int want = ceil_div(new_len, groups_[g].page_size);
        while ((int)r.tables[g].size() < want) {
            r.tables[g].push_back(free_[g].back());
            free_[g].pop_back();
        }
    }
    r.reserved = new_len;
    return OK;
}

int CacheManager::commit(int64_t id, int new_len) {
    auto it = requests_.find(id);
    if (it == requests_.end()) return UNKNOWN_REQUEST;
    Request& r = it->second;
    if (new_len < r.len || new_len > r.reserved) return BAD_LENGTH;
    r.len = new_len;
    int freed = 0;
    for (size_t g = 0; g < groups_.size(); ++g) {
        const int w = groups_[g].window;
        if (w <= 0) continue;
        // the next query is at position >= len and reads keys from len - w + 1 on
        const int first_needed = std::max(0, new_len - w + 1);
        const int dead_pages = first_needed / groups_[g].page_size;  // pages wholly below first_needed
        for (int i = r.first_live[g]; i < dead_pages && i < (int)r.tables[g].size(); ++i) {
            if (r.tables[g][i] >= 0) {
                free_[g].push_back(r.tables[g][i]);
                r.tables[g][i] = -1;
                ++freed;
            }
        }
        r.first_live[g] = std::max(r.first_live[g], std::min(dead_pages, (int)r.tables[g].size()));
    }
    return freed;
}

int CacheManager::close(int64_t id) {
    auto it = requests_.find(id);
    if (it == requests_.end()) return UNKNOWN_REQUEST;
    Request& r = it->second;
    int freed = 0;
    for (size_t g = 0; g < groups_.size(); ++g) {
        for (int32_t p : r.tables[g]) {
            if (p >= 0) {
                free_[g].push_back(p);
                ++freed;
            }
        }
    }
    free_slots_.push_back(r.slot);
    requests_.erase(it);
    return freed;
}

int CacheManager::release_reserved(int64_t id) {
    auto it = requests_.find(id);
    if (it == requests_.end()) return UNKNOWN_REQUEST;
    Request& r = it->second;
    int freed = 0;
    for (size_t g = 0; g < groups_.size(); ++g) {
        const int keep = ceil_div(r.len, groups_[g].page_size);
        while ((int)r.tables[g].size() > keep) {
            if (r.tables[g].back() >= 0) {
                free_[g].push_back(r.tables[g].back());
                ++freed;
            }
            r.tables[g].pop_back();
        }
    }
    r.reserved = r.len;
    return freed;
}

int CacheManager::length(int64_t id) const {
    auto it = requests_.find(id);
    return it == requests_.end() ? (int)UNKNOWN_REQUEST : it->second.len;
}

int CacheManager::reserved(int64_t id) const {
    auto it = requests_.find(id);
    return it == requests_.end() ? (int)UNKNOWN_REQUEST : it->second.reserved;
}

int CacheManager::slot(int64_t id) const {
    auto it = requests_.find(id);
    return it == requests_.end() ? (int)UNKNOWN_REQUEST : it->second.slot;
}

int CacheManager::table(int64_t id, int g, int32_t* out, int capacity) const {
    auto it = requests_.find(id);
    if (it == requests_.end()) return UNKNOWN_REQUEST;
    if (g < 0 || g >= (int)groups_.size()) return BAD_ARGUMENT;
    const auto& t = it->second.tables[g];
    if ((int)t.size() > capacity) return BAD_ARGUMENT;
    std::copy(t.begin(), t.end(), out);
    return (int)t.size();
}

int CacheManager::pages_held(int64_t id, int g) const {
    auto it = requests_.find(id);
    if (it == requests_.end()) return UNKNOWN_REQUEST;
    if (g < 0 || g >= (int)groups_.size()) return BAD_ARGUMENT;
    int n = 0;
    for (int32_t p : it->second.tables[g]) n += p >= 0;
    return n;
}

int CacheManager::peak_pages(int g, int len, int portion) const {
    const GroupConfig& c = groups_[g];
    if (c.window <= 0 || len <= c.window) return ceil_div(len, c.page_size);
    // during a step the request holds the window before the portion and the portion itself
    const int span = std::min(len, c.window - 1 + std::max(1, portion));
    return std::min(ceil_div(len, c.page_size), ceil_div(span, c.page_size) + 1);
}

int CacheManager::check() const {
    for (size_t g = 0; g < groups_.size(); ++g) {
        std::vector<int> seen(groups_[g].num_pages, 0);
        for (int32_t p : free_[g]) {
            if (p < 0 || p >= groups_[g].num_pages || seen[p]++) return INVARIANT_BROKEN;
        }
        for (const auto& kv : requests_) {
            const Request& r = kv.second;
            for (size_t i = 0; i < r.tables[g].size(); ++i) {
                const int32_t p = r.tables[g][i];
                if (p == -1) continue;
                if (p < 0 || p >= groups_[g].num_pages || seen[p]++) return INVARIANT_BROKEN;
            }
            if (ceil_div(r.reserved, groups_[g].page_size) != (int)r.tables[g].size()) return INVARIANT_BROKEN;
        }
        for (int s : seen)
            if (s != 1) return INVARIANT_BROKEN;
    }
    std::vector<int> slots(free_slots_.size() + requests_.size(), 0);
    for (int s : free_slots_) {
        if (s < 0 || s >= (int)slots.size() || slots[s]++) return INVARIANT_BROKEN;
    }
    for (const auto& kv : requests_) {
        const int s = kv.second.slot;
        if (s < 0 || s >= (int)slots.size() || slots[s]++) return INVARIANT_BROKEN;
    }
    return OK;
}

}  // namespace rmx
