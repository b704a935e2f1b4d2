// Scheduler: decides which tokens of which requests run in the next step.
//
// The reference batches only decode tokens (one per live request and engine iteration,
// src/serve/vllm_batch.c:199-229) and runs a whole prompt under the engine lock in between
// (vllm_batch.c:320-350); it refuses work at admission (src/serve/vllm_server.c:82-101) and
// has no answer to a cache that fills up.  This scheduler builds mixed steps:
//
//   1. every running request that has exactly one token left to compute (a decode token)
//      gets it, oldest first;
//   2. what is left of the step's token budget goes to prompt portions of running requests,
//      oldest first, each at most `prefill_chunk` tokens;
//   3. then waiting requests are admitted in arrival order while a state slot is free, the
//      live-request limit is not reached and free pages exist for all the tokens they have so
//      far (their prompt, and what they had generated if they were preempted): a request that
//      only its first portion fits would be preempted again a few steps later.  A request is not
//      admitted by the same call that preempted it.
//
// When pages run out for a running request, the youngest running request (the last one
// admitted) gives back everything it holds and returns to the FRONT of the waiting queue;
// all its tokens, prompt and generated, are computed again later, so its output is the one it
// would have produced undisturbed.  A request that could never fit the pool alone is refused
// when it is added.
//
// The scheduler counts tokens; the token values and the sampling live with the caller.
#include <stdint.h>

#include <algorithm>
#include <deque>
#include <unordered_map>
#include <vector>

#include "../../include/kestrel.h"

namespace {

struct Req {
    long long id = 0;
    int known = 0;        // tokens whose values exist (prompt + generated so far)
    int computed = 0;     // tokens in the cache
    int max_total = 0;    // prompt + max_new_tokens
    int scheduled = 0;    // tokens of the step in flight
    long long order = 0;  // admission order among running requests
};

struct Sched {
    void *cache = nullptr;
    int max_step_tokens = 0, prefill_chunk = 0, batch_max = 0, max_queued = 0, max_model_len = 0;
    std::deque<Req> waiting;
    std::vector<Req> running;          // admission order
    std::vector<long long> preempted;  // ids preempted by the last schedule() call
    long long admissions = 0;
    long long n_preemptions = 0;
    bool step_in_flight = false;
};

int min_pool_tokens(Sched &s) {
    int n = kcache_num_groups(s.cache), best = INT32_MAX;
    for (int g = 0; g < n; ++g) best = std::min(best, kcache_num_pages(s.cache, g));
    if (n == 0) return INT32_MAX;
    long long t = (long long)best * kcache_page_size(s.cache);
    return t > INT32_MAX ? INT32_MAX : (int)t;
}

// the youngest running request leaves the cache and goes to the front of the waiting queue
bool preempt_youngest(Sched &s, std::vector<int> &entry_of_running, std::vector<long long> &ids,
                      std::vector<int> &starts, std::vector<int> &counts) {
    if (s.running.empty()) return false;
    size_t vi = s.running.size() - 1;
    Req victim = s.running[vi];
    // drop the victim's entry of this step, if it has one
    for (size_t e = 0; e < ids.size(); ++e)
        if (ids[e] == victim.id) {
            ids.erase(ids.begin() + e);
            starts.erase(starts.begin() + e);
            counts.erase(counts.begin() + e);
            break;
        }
    kcache_release(s.cache, victim.id);
    victim.computed = 0;
    victim.scheduled = 0;
    s.running.pop_back();
    entry_of_running.resize(s.running.size());
    s.waiting.push_front(victim);
    s.preempted.push_back(victim.id);
    s.n_preemptions++;
    return true;
}

}  // namespace

KESTREL_API void *ksched_create(void *cache, int max_step_tokens, int prefill_chunk, int batch_max,
                         int max_queued, int max_model_len) {
    if (!cache || max_step_tokens <= 0 || prefill_chunk <= 0 || batch_max <= 0 || max_model_len <= 0) return nullptr;
    Sched *s = new Sched();
    s->cache = cache;
    s->max_step_tokens = max_step_tokens;
    s->prefill_chunk = prefill_chunk;
    s->batch_max = batch_max;
    s->max_queued = max_queued;
    s->max_model_len = max_model_len;
    return s;
}

KESTREL_API void ksched_destroy(void *h) { delete (Sched *)h; }

// 0 = queued; -1 = waiting queue full; -2 = prompt + max_new_tokens exceeds max_model_len or
// what the page pool can ever hold; -3 = empty prompt or duplicate id
KESTREL_API int ksched_add(void *h, long long id, int prompt_len, int max_new_tokens) {
    Sched &s = *(Sched *)h;
    if (prompt_len <= 0 || max_new_tokens < 0) return -3;
    for (const Req &r : s.running) if (r.id == id) return -3;
    for (const Req &r : s.waiting) if (r.id == id) return -3;
    if ((int)s.waiting.size() >= s.max_queued) return -1;
    long long total = (long long)prompt_len + max_new_tokens;
    if (total > s.max_model_len || total > min_pool_tokens(s)) return -2;
    Req r;
    r.id = id;
    r.known = prompt_len;
    r.max_total = (int)total;
    s.waiting.push_back(r);
    return 0;
}

// Builds the next step.  Entry e runs tokens [starts[e], starts[e] + counts[e]) of request
// ids[e]; wants[e] = 1 if the entry ends with the request's last known token, whose logits
// pick the next token.  Pages for every entry are reserved.  Returns the number of entries
// (0 = nothing to do), or -7 if the previous step was not completed.
KESTREL_API int ksched_schedule(void *h, long long *ids_out, int *starts_out, int *counts_out, int *wants_out, int cap) {
    Sched &s = *(Sched *)h;
    if (s.step_in_flight) return -7;
    s.preempted.clear();
    std::vector<long long> ids;
    std::vector<int> starts, counts;
    std::vector<int> dummy;
    int budget = s.max_step_tokens;

    // 1. decode tokens, oldest first; on a page shortage the youngest running request yields
    for (size_t i = 0; i < s.running.size();) {
        Req &r = s.running[i];
        if (r.known - r.computed != 1 || budget <= 0) { ++i; continue; }
        int rc = kcache_reserve(s.cache, r.id, 1);
        if (rc == 0) {
            ids.push_back(r.id); starts.push_back(r.computed); counts.push_back(1);
            r.scheduled = 1;
            --budget;
            ++i;
        } else if (rc == -1) {
            bool self = (i == s.running.size() - 1);
            preempt_youngest(s, dummy, ids, starts, counts);
            if (self) break;            // the request that needed the page was the youngest
        } else {
            return rc;
        }
    }
    // 2. prompt portions of running requests
    for (size_t i = 0; i < s.running.size() && budget > 0; ++i) {
        Req &r = s.running[i];
        int left = r.known - r.computed;
        if (left <= 1 || r.scheduled) continue;
        int n = std::min(std::min(left, s.prefill_chunk), budget);
        while (n > 0 && kcache_can_reserve(s.cache, r.id, n) == 0) n /= 2;   // a shorter portion may fit
        if (n <= 0) continue;
        int rc = kcache_reserve(s.cache, r.id, n);
        if (rc != 0) return rc == -1 ? -8 : rc;
        ids.push_back(r.id); starts.push_back(r.computed); counts.push_back(n);
        r.scheduled = n;
        budget -= n;
    }
    // 3. admissions
    while (!s.waiting.empty() && budget > 0 && (int)s.running.size() < s.batch_max &&
           kcache_free_slots(s.cache) > 0) {
        Req r = s.waiting.front();
        if (std::find(s.preempted.begin(), s.preempted.end(), r.id) != s.preempted.end()) break;
        int left = r.known - r.computed;
        int n = std::min(std::min(left, s.prefill_chunk), budget);
        if (kcache_admit(s.cache, r.id) < 0) break;
        if (kcache_can_reserve(s.cache, r.id, left) != 1) {
            kcache_release(s.cache, r.id);
            break;                      // arrival order is kept: nobody overtakes the head
        }
        kcache_reserve(s.cache, r.id, n);
        s.waiting.pop_front();
        r.order = s.admissions++;
        r.scheduled = n;
        ids.push_back(r.id); starts.push_back(r.computed); counts.push_back(n);
        budget -= n;
        s.running.push_back(r);
    }
    // Nothing could run although requests are live: prompts hold all pages between them.
    // The youngest yields until the oldest can go on.
    auto work_left = [&]() {
        for (const Req &r : s.running) if (r.known > r.computed) return true;
        return false;
    };
    while (ids.empty() && s.running.size() > 1 && work_left()) {
        preempt_youngest(s, dummy, ids, starts, counts);
        for (size_t i = 0; i < s.running.size() && budget > 0; ++i) {
            Req &r = s.running[i];
            int left = r.known - r.computed;
            if (left <= 0) continue;
            int n = std::min(std::min(left, s.prefill_chunk), budget);
            while (n > 0 && kcache_can_reserve(s.cache, r.id, n) == 0) n /= 2;
            if (n <= 0) continue;
            if (kcache_reserve(s.cache, r.id, n) != 0) continue;
            ids.push_back(r.id); starts.push_back(r.computed); counts.push_back(n);
            r.scheduled = n;
            budget -= n;
        }
    }
    int n_entries = (int)ids.size();
    if (n_entries > cap) return -9;
    for (int e = 0; e < n_entries; ++e) {
        ids_out[e] = ids[e]; starts_out[e] = starts[e]; counts_out[e] = counts[e];
        int want = 0;
        for (const Req &r : s.running)
            if (r.id == ids[e]) want = (starts[e] + counts[e] == r.known) ? 1 : 0;
        wants_out[e] = want;
    }
    s.step_in_flight = n_entries > 0;
    return n_entries;
}

// ids that the last schedule() call sent back to the waiting queue
KESTREL_API int ksched_preempted(void *h, long long *out, int cap) {
    Sched &s = *(Sched *)h;
    int n = std::min(cap, (int)s.preempted.size());
    for (int i = 0; i < n; ++i) out[i] = s.preempted[i];
    return (int)s.preempted.size();
}

// The step that schedule() built has run: its tokens are in the cache.  The caller commits
// the cache manager itself (it owns the device side); this only moves the counters.
KESTREL_API int ksched_step_done(void *h) {
    Sched &s = *(Sched *)h;
    for (Req &r : s.running) {
        r.computed += r.scheduled;
        r.scheduled = 0;
    }
    s.step_in_flight = false;
    return 0;
}

// A token was sampled for the request: it has one more known token.  Returns 1 if the
// request has now reached its token limit (the caller finishes it), 0 otherwise.
KESTREL_API int ksched_on_token(void *h, long long id) {
    Sched &s = *(Sched *)h;
    for (Req &r : s.running)
        if (r.id == id) {
            r.known++;
            return r.known >= r.max_total ? 1 : 0;
        }
    return -3;
}

// The request is over (stop token, token limit or abort): pages and slot are given back.
KESTREL_API int ksched_finish(void *h, long long id) {
    Sched &s = *(Sched *)h;
    for (size_t i = 0; i < s.running.size(); ++i)
        if (s.running[i].id == id) {
            kcache_release(s.cache, id);
            s.running.erase(s.running.begin() + i);
            return 0;
        }
    for (size_t i = 0; i < s.waiting.size(); ++i)
        if (s.waiting[i].id == id) {
            s.waiting.erase(s.waiting.begin() + i);
            return 0;
        }
    return -3;
}

KESTREL_API int ksched_num_running(void *h) { return (int)((Sched *)h)->running.size(); }
KESTREL_API int ksched_num_waiting(void *h) { return (int)((Sched *)h)->waiting.size(); }
KESTREL_API long long ksched_num_preemptions(void *h) { return ((Sched *)h)->n_preemptions; }
KESTREL_API int ksched_known(void *h, long long id) {
    Sched &s = *(Sched *)h;
    for (const Req &r : s.running) if (r.id == id) return r.known;
    for (const Req &r : s.waiting) if (r.id == id) return r.known;
    return -3;
}
