// The C interface of the cache manager and the scheduler (called from Python via ctypes).
#include <cstring>

#include "cache_manager.hpp"
#include "scheduler.hpp"

#define RMX_API extern "C" __attribute__((visibility("default")))

using rmx::CacheManager;
using rmx::Scheduler;

RMX_API void* rmx_cm_create(int n_groups, const int* num_pages, const int* page_sizes, const int* windows,
                            int max_requests) {
    if (n_groups < 0 || max_requests <= 0) return nullptr;
    std::vector<rmx::GroupConfig> groups;
    for (int g = 0; g < n_groups; ++g) {
        if (num_pages[g] < 0 || page_sizes[g] <= 0 || windows[g] < 0) return nullptr;
        groups.push_back({num_pages[g], page_sizes[g], windows[g]});
    }
    return new CacheManager(groups, max_requests);
}
RMX_API void rmx_cm_destroy(void* h) { delete (CacheManager*)h; }
RMX_API int rmx_cm_open(void* h, long long id) { return ((CacheManager*)h)->open(id); }
RMX_API int rmx_cm_reserve(void* h, long long id, int new_len) { return ((CacheManager*)h)->reserve(id, new_len); }
RMX_API int rmx_cm_max_reservable(void* h, long long id, int want) { return ((CacheManager*)h)->max_reservable(id, want); }
RMX_API int rmx_cm_commit(void* h, long long id, int new_len) { return ((CacheManager*)h)->commit(id, new_len); }
RMX_API int rmx_cm_close(void* h, long long id) { return ((CacheManager*)h)->close(id); }
RMX_API int rmx_cm_release_reserved(void* h, long long id) { return ((CacheManager*)h)->release_reserved(id); }
RMX_API int rmx_cm_length(void* h, long long id) { return ((CacheManager*)h)->length(id); }
RMX_API int rmx_cm_reserved(void* h, long long id) { return ((CacheManager*)h)->reserved(id); }
RMX_API int rmx_cm_slot(void* h, long long id) { return ((CacheManager*)h)->slot(id); }
RMX_API int rmx_cm_table(void* h, long long id, int g, int* out, int capacity) {
    return ((CacheManager*)h)->table(id, g, out, capacity);
}
RMX_API int rmx_cm_pages_held(void* h, long long id, int g) { return ((CacheManager*)h)->pages_held(id, g); }
RMX_API int rmx_cm_peak_pages(void* h, int g, int len, int portion) { return ((CacheManager*)h)->peak_pages(g, len, portion); }
RMX_API int rmx_cm_free_pages(void* h, int g) { return ((CacheManager*)h)->free_pages(g); }
RMX_API int rmx_cm_free_slots(void* h) { return ((CacheManager*)h)->free_slots(); }
RMX_API int rmx_cm_live(void* h) { return ((CacheManager*)h)->live(); }
RMX_API int rmx_cm_has(void* h, long long id) { return ((CacheManager*)h)->has(id) ? 1 : 0; }
RMX_API int rmx_cm_check(void* h) { return ((CacheManager*)h)->check(); }

RMX_API void* rmx_sched_create(void* cm, int max_seqs, int max_batch_tokens, int prefill_chunk, int max_context) {
    if (!cm || max_seqs <= 0 || max_batch_tokens <= 0 || prefill_chunk <= 0) return nullptr;
    return new Scheduler((CacheManager*)cm, max_seqs, max_batch_tokens, prefill_chunk, max_context);
}
RMX_API void rmx_sched_destroy(void* h) { delete (Scheduler*)h; }
RMX_API int rmx_sched_add(void* h, long long id, int prompt_len, int max_new) {
    return ((Scheduler*)h)->add(id, prompt_len, max_new);
}
// Fills ids/start/count/wants (capacity entries each); returns the number of entries, or -1 if more than capacity.
RMX_API int rmx_sched_next(void* h, long long* ids, int* start, int* count, int* wants, int capacity) {
    const auto& b = ((Scheduler*)h)->next();
    if ((int)b.size() > capacity) return -1;
    for (size_t i = 0; i < b.size(); ++i) {
        ids[i] = b[i].id;
        start[i] = b[i].start;
        count[i] = b[i].count;
        wants[i] = b[i].wants_logits;
    }
    return (int)b.size();
}
RMX_API int rmx_sched_step_done(void* h) { return ((Scheduler*)h)->step_done(); }
RMX_API int rmx_sched_append_token(void* h, long long id) { return ((Scheduler*)h)->append_token(id); }
RMX_API int rmx_sched_finish(void* h, long long id) { return ((Scheduler*)h)->finish(id); }
RMX_API int rmx_sched_waiting(void* h) { return ((Scheduler*)h)->waiting(); }
RMX_API int rmx_sched_running(void* h) { return ((Scheduler*)h)->running(); }
RMX_API int rmx_sched_computed(void* h, long long id) { return ((Scheduler*)h)->computed(id); }
RMX_API int rmx_sched_total(void* h, long long id) { return ((Scheduler*)h)->total(id); }
RMX_API int rmx_sched_take_preempted(void* h, long long* out, int capacity) {
    auto v = ((Scheduler*)h)->take_preempted();
    const int n = (int)v.size() < capacity ? (int)v.size() : capacity;
    for (int i = 0; i < n; ++i) out[i] = v[i];
    return n;
}
