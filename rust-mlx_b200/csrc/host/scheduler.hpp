// The scheduler: admits requests, cuts prompts into portions under a token budget,
// lets every running request past its prompt decode one token a step, finishes and
// frees.  Portions of some requests run beside decoded tokens of others in one batch.
//
// The reference's only scheduler (src/bin/server/batch.rs:240-323) admits up to eight
// rows from a bounded queue, prefills a whole prompt at admission, and then runs the rows
// at the smallest cache offset; it has no pages and no token budget.
//
// A request is a count of known tokens (`total`: prompt plus what was generated) and a
// count of tokens whose keys are in the cache (`computed`).  Each step feeds tokens
// computed .. computed + n - 1; when that reaches `total` the step's last logits are
// wanted and the caller appends the chosen token (or finishes the request).
//
// When pages run out: portions of prompts shrink or wait; if a decoding request cannot
// get the page for its next token, the running request admitted last gives up all its
// pages and goes back to the head of the queue, to be computed again (prompt and
// generated tokens) when there is room.  A request that could never fit is refused when
// it is added.  All decisions are in order of admission, so a run is reproducible.
#pragma once
#include <cstdint>
#include <deque>
#include <vector>

#include "cache_manager.hpp"

namespace rmx {

enum SchedStatus : int {
    SCHED_OK = 0,
    SCHED_EMPTY_PROMPT = -10,
    SCHED_TOO_LONG = -11,      // prompt + max_new_tokens exceeds the context limit
    SCHED_NEVER_FITS = -12,    // needs more pages than a pool has
    SCHED_DUPLICATE = -13,
    SCHED_UNKNOWN = -14,
    SCHED_BAD_STATE = -15,
};

struct Entry {
    int64_t id;
    int start;        // position of the first token fed
    int count;        // tokens fed this step
    int wants_logits; // 1 if the last of them is the request's last known token
};

class Scheduler {
public:
    Scheduler(CacheManager* cache, int max_seqs, int max_batch_tokens, int prefill_chunk, int max_context);

    int add(int64_t id, int prompt_len, int max_new_tokens);
    // Build the next batch.  Pages for it are reserved.  Returns the entries (possibly none).
    const std::vector<Entry>& next();
    // The batch ran: its tokens are in the cache.
    int step_done();
    // The caller chose a token for a request whose logits were wanted.
    int append_token(int64_t id);
    int finish(int64_t id);

    int waiting() const { return (int)waiting_.size(); }
    int running() const { return (int)running_.size(); }
    bool idle() const { return waiting_.empty() && running_.empty(); }
    // Requests preempted since the last call (they are waiting again).
    std::vector<int64_t> take_preempted();
    int computed(int64_t id) const;
    int total(int64_t id) const;

private:
    struct Req {
        int64_t id;
        int total;      // tokens known
        int computed;   // tokens in the cache
        int limit;      // prompt + max_new_tokens
        int64_t order;  // admission counter (for "admitted last")
    };
    Req* find_running(int64_t id);
    bool preempt_last(int64_t protect);
    bool schedule(Req& r, int want, int& budget);

    CacheManager* cache_;
    int max_seqs_, max_batch_tokens_, prefill_chunk_, max_context_;
    int64_t order_ = 0;
    std::deque<Req> waiting_;
    std::vector<Req> running_;  // in order of admission
    std::vector<Entry> batch_;
    std::vector<int64_t> preempted_;
    bool in_flight_ = false;
};

}  // namespace rmx
