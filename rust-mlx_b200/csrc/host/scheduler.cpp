#include "scheduler.hpp"

#include <algorithm>

namespace rmx {

Scheduler::Scheduler(CacheManager* cache, int max_seqs, int max_batch_tokens, int prefill_chunk, int max_context)
    : cache_(cache), max_seqs_(max_seqs), max_batch_tokens_(max_batch_tokens), prefill_chunk_(prefill_chunk),
      max_context_(max_context) {}

int Scheduler::add(int64_t id, int prompt_len, int max_new_tokens) {
    if (prompt_len <= 0) return SCHED_EMPTY_PROMPT;
    if (max_new_tokens < 0) max_new_tokens = 0;
    const long long limit = (long long)prompt_len + max_new_tokens;
    if (max_context_ > 0 && limit > max_context_) return SCHED_TOO_LONG;
    for (const Req& r : waiting_)
        if (r.id == id) return SCHED_DUPLICATE;
    for (const Req& r : running_)
        if (r.id == id) return SCHED_DUPLICATE;
    // the cache holds at most limit - 1 tokens: the last generated token is never fed
    const int held = (int)std::max<long long>(1, limit - 1);
    for (int g = 0; g < cache_->num_groups(); ++g) {
        if (cache_->peak_pages(g, held, std::min(prefill_chunk_, max_batch_tokens_)) > cache_->group(g).num_pages)
            return SCHED_NEVER_FITS;
    }
    waiting_.push_back(Req{id, prompt_len, 0, (int)limit, -1});
    return SCHED_OK;
}

Scheduler::Req* Scheduler::find_running(int64_t id) {
    for (Req& r : running_)
        if (r.id == id) return &r;
    return nullptr;
}

// The running request admitted last (other than `protect`, unless it is the only one)
// gives up its pages and waits again at the head of the queue.
bool Scheduler::preempt_last(int64_t protect) {
    int victim = -1;
    for (int i = (int)running_.size() - 1; i >= 0; --i) {
        if (running_[i].id != protect) {
            victim = i;
            break;
        }
    }
    if (victim < 0) return false;
    Req r = running_[victim];
    // drop it from the batch being built, if it is there
    batch_.erase(std::remove_if(batch_.begin(), batch_.end(), [&](const Entry& e) { return e.id == r.id; }),
                 batch_.end());
    cache_->close(r.id);
    running_.erase(running_.begin() + victim);
    r.computed = 0;
    waiting_.push_front(r);
    preempted_.push_back(r.id);
    return true;
}

// Give `r` up to `want` tokens of this step; false if not even one fits.
bool Scheduler::schedule(Req& r, int want, int& budget) {
    want = std::min(want, budget);
    if (want <= 0) return false;
    const int fit = cache_->max_reservable(r.id, r.computed + want) - r.computed;
    const int n = std::min(want, fit);
    if (n <= 0) return false;
    if (cache_->reserve(r.id, r.computed + n) != OK) return false;
    batch_.push_back(Entry{r.id, r.computed, n, r.computed + n == r.total ? 1 : 0});
    budget -= n;
    return true;
}

const std::vector<Entry>& Scheduler::next() {
    batch_.clear();
    if (in_flight_) return batch_;
    int budget = max_batch_tokens_;

    auto in_batch = [&](int64_t id) {
        return std::any_of(batch_.begin(), batch_.end(), [&](const Entry& e) { return e.id == id; });
    };
    bool preempted_now = false;

    // 1. decoding requests, one token each, in order of admission
    for (size_t i = 0; i < running_.size() && budget > 0;) {
        Req& r = running_[i];
        if (r.total - r.computed != 1 || in_batch(r.id) || schedule(r, 1, budget)) {
            ++i;
            continue;
        }
        // no page for its next token: the request admitted last makes room
        preempted_now = true;
        if (!preempt_last(r.id)) {
            preempt_last(-1);  // it is alone: it waits to be computed again (add() made sure it can fit)
            break;
        }
        i = 0;  // positions moved; entries already made are skipped
    }

    // 2. running requests still in their prompt (or being computed again), in order of admission
    for (Req& r : running_) {
        if (r.total - r.computed <= 1) continue;
        if (in_batch(r.id)) continue;
        schedule(r, std::min(r.total - r.computed, prefill_chunk_), budget);
    }

    // 3. admit from the queue while there is room
    while (!preempted_now && !waiting_.empty() && (int)running_.size() < max_seqs_ && budget > 0 && cache_->free_slots() > 0) {
        Req r = waiting_.front();
        if (cache_->open(r.id) < 0) break;
        r.order = order_++;
        const int want = std::min(r.total - r.computed, prefill_chunk_);
        // admit only if its whole first portion (or what the budget leaves of it) fits
        const int need = std::min(want, budget);
        if (cache_->max_reservable(r.id, need) < need) {
            cache_->close(r.id);
            break;
        }
        waiting_.pop_front();
        running_.push_back(r);
        schedule(running_.back(), want, budget);
    }

    // 4. a request has tokens to feed, nothing could run, and others hold pages: the one admitted last steps back.
    // (Requests that merely wait for their next token to be chosen hold pages too, but they are not stuck.)
    if (batch_.empty() && !running_.empty()) {
        bool starving = !waiting_.empty() && (int)running_.size() < max_seqs_ && cache_->free_slots() > 0;
        bool anyone_idle = false;
        for (const Req& r : running_) {
            if (r.total > r.computed) starving = true;
            else anyone_idle = true;
        }
        if (starving && !anyone_idle && (running_.size() > 1 || !waiting_.empty())) {
            preempt_last(-1);
            return next();
        }
    }
    in_flight_ = !batch_.empty();
    return batch_;
}

int Scheduler::step_done() {
    if (!in_flight_) return SCHED_BAD_STATE;
    for (const Entry& e : batch_) {
        Req* r = find_running(e.id);
        if (!r) continue;
        r->computed = e.start + e.count;
        cache_->commit(e.id, r->computed);
    }
    in_flight_ = false;
    return SCHED_OK;
}

int Scheduler::append_token(int64_t id) {
    Req* r = find_running(id);
    if (!r) return SCHED_UNKNOWN;
    if (r->computed != r->total) return SCHED_BAD_STATE;
    r->total += 1;
    return SCHED_OK;
}

int Scheduler::finish(int64_t id) {
    for (size_t i = 0; i < running_.size(); ++i) {
        if (running_[i].id == id) {
            cache_->close(id);
            running_.erase(running_.begin() + i);
            batch_.erase(std::remove_if(batch_.begin(), batch_.end(), [&](const Entry& e) { return e.id == id; }),
                         batch_.end());
            return SCHED_OK;
        }
    }
    for (size_t i = 0; i < waiting_.size(); ++i) {
        if (waiting_[i].id == id) {
            waiting_.erase(waiting_.begin() + i);
            return SCHED_OK;
        }
    }
    return SCHED_UNKNOWN;
}

std::vector<int64_t> Scheduler::take_preempted() {
    std::vector<int64_t> out;
    out.swap(preempted_);
    return out;
}

int Scheduler::computed(int64_t id) const {
    for (const Req& r : running_)
        if (r.id == id) return r.computed;
    for (const Req& r : waiting_)
        if (r.id == id) return r.computed;
    return SCHED_UNKNOWN;
}

int Scheduler::total(int64_t id) const {
    for (const Req& r : running_)
        if (r.id == id) return r.total;
    for (const Req& r : waiting_)
        if (r.id == id) return r.total;
    return SCHED_UNKNOWN;
}

}  // namespace rmx
