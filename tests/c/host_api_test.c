/* A C11 caller of the engine's host interface, built against include/kestrel.h alone
 * (gcc -std=c11 -Wall -Werror): the cache manager, the scheduler and the packer of a step's
 * description, driven through admission, refusal, prompt portions under a token budget, decode
 * steps, page exhaustion with preempt-and-recompute, and finishing, with a fake step in place
 * of the GPU (it only commits the tokens).  After every step the cache manager's invariants
 * hold, the packed description passes the check the runner's debug guards use, and at the end
 * every page is free again.  The reference's header-level interface is
 * include/model/vllm_safetensors.h:497-670.  Prints OK and exits 0, or names what failed. */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "kestrel.h"

#define CHECK(cond, ...)                                            \
    do {                                                            \
        if (!(cond)) {                                              \
            fprintf(stderr, "FAILED %s:%d: ", __FILE__, __LINE__);  \
            fprintf(stderr, __VA_ARGS__);                           \
            fprintf(stderr, "\n");                                  \
            return 1;                                               \
        }                                                           \
    } while (0)

enum { PAGE = 4, PAGES = 10, MAX_REQ = 3, MAX_BLOCKS = 16, BUDGET = 12, CHUNK = 8, NEW_TOKENS = 6, CAP = 16 };

int main(void) {
    const int windows[1] = {0}, num_pages[1] = {PAGES};
    void *cache = kcache_create(1, windows, num_pages, PAGE, MAX_REQ, MAX_BLOCKS);
    CHECK(cache, "kcache_create");
    void *sched = ksched_create(cache, BUDGET, CHUNK, MAX_REQ, 4, 40);
    CHECK(sched, "ksched_create");

    const int prompt_len[3] = {10, 7, 13};
    int generated[3] = {0, 0, 0}, done[3] = {0, 0, 0}, restarts[3] = {0, 0, 0}, computed[3] = {0, 0, 0};
    for (int r = 0; r < 3; ++r) CHECK(ksched_add(sched, 100 + r, prompt_len[r], NEW_TOKENS) == 0, "add %d", r);
    CHECK(ksched_add(sched, 100, 5, 1) == -3, "a duplicate id must be refused");
    CHECK(ksched_add(sched, 200, 39, 5) == -2, "a request longer than max_model_len must be refused");
    CHECK(ksched_add(sched, 201, 0, 5) == -3, "an empty prompt must be refused");
    CHECK(ksched_num_waiting(sched) == 3 && ksched_num_running(sched) == 0, "queue lengths");

    long long ids[CAP];
    int starts[CAP], counts[CAP], wants[CAP];
    int tokens[64], want_counts[CAP], want_at[CAP], packed[1024], layout[KBATCH_LAYOUT_INTS];
    int steps = 0, saw_portion = 0, saw_mixed = 0;
    while (!(done[0] && done[1] && done[2])) {
        CHECK(++steps < 200, "the scheduler makes no progress");
        int n = ksched_schedule(sched, ids, starts, counts, wants, CAP);
        CHECK(n >= 0, "schedule returned %d", n);
        long long pre[CAP];
        int np = ksched_preempted(sched, pre, CAP);
        for (int i = 0; i < np && i < CAP; ++i) {
            int r = (int)(pre[i] - 100);
            restarts[r]++;
            computed[r] = 0;                /* everything it had is computed again */
            CHECK(kcache_slot(cache, pre[i]) < 0, "a preempted request must hold nothing");
        }
        if (n == 0) continue;
        int total = 0, decodes = 0, portions = 0, n_wants = 0;
        for (int e = 0; e < n; ++e) {
            int r = (int)(ids[e] - 100);
            CHECK(r >= 0 && r < 3 && !done[r], "entry for an unknown or finished request");
            CHECK(starts[e] == computed[r], "request %d: the step starts at %d, %d tokens are in the cache", r, starts[e], computed[r]);
            CHECK(counts[e] >= 1 && counts[e] <= CHUNK, "portion of %d tokens", counts[e]);
            CHECK(kcache_length(cache, ids[e]) == starts[e], "cache length");
            CHECK(kcache_num_blocks(cache, ids[e], 0) * PAGE >= starts[e] + counts[e], "pages were not reserved");
            for (int j = 0; j < counts[e]; ++j) tokens[total + j] = (starts[e] + j) % 50;
            total += counts[e];
            if (counts[e] == 1) decodes++; else portions++;
            want_counts[e] = wants[e] ? 1 : 0;
            if (wants[e]) want_at[n_wants++] = counts[e] - 1;
            CHECK(wants[e] == (starts[e] + counts[e] == prompt_len[r] + generated[r]), "wants_token of request %d", r);
        }
        CHECK(total <= BUDGET, "%d tokens in a step, the budget is %d", total, BUDGET);
        saw_portion |= portions > 0;
        saw_mixed |= portions > 0 && decodes > 0;
        /* the description a GPU step would get, and the guards' check of it */
        int need = kbatch_ints_needed(cache, n, ids, counts, n_wants, 0);
        CHECK(need > 0 && need <= 1024, "kbatch_ints_needed %d", need);
        int wrote = kbatch_pack(cache, n, ids, counts, tokens, want_counts, want_at, 0, packed, 1024, layout);
        CHECK(wrote == need, "kbatch_pack wrote %d of %d", wrote, need);
        CHECK(layout[KB_NUM_TOKENS] == total && layout[KB_NUM_SEQS] == n && layout[KB_NUM_ROWS] == n_wants, "layout counts");
        const int pool[1] = {PAGES + 1};
        CHECK(kbatch_check(packed, layout, 50, PAGE, pool) == 0, "a valid description failed its check");
        /* a description damaged on purpose is caught on the host: no kernel ever sees it */
        int keep = packed[layout[KB_O_TOKEN_IDS]];
        packed[layout[KB_O_TOKEN_IDS]] = 50;
        CHECK((kbatch_check(packed, layout, 50, PAGE, pool) >> 16) == 1, "a token id beyond the vocabulary passed");
        packed[layout[KB_O_TOKEN_IDS]] = keep;
        keep = packed[layout[KB_O_TABLES] + packed[layout[KB_O_POSITIONS]] / PAGE];
        packed[layout[KB_O_TABLES] + packed[layout[KB_O_POSITIONS]] / PAGE] = PAGES + 1;
        CHECK((kbatch_check(packed, layout, 50, PAGE, pool) >> 16) == 5, "a page id beyond the pool passed");
        packed[layout[KB_O_TABLES] + packed[layout[KB_O_POSITIONS]] / PAGE] = keep;
        /* the fake step: the tokens are in the cache now */
        for (int e = 0; e < n; ++e) {
            CHECK(kcache_commit(cache, ids[e], counts[e]) == 0, "commit");
            computed[(int)(ids[e] - 100)] += counts[e];
        }
        CHECK(ksched_step_done(sched) == 0, "step_done");
        CHECK(kcache_check(cache) == 0, "cache invariants broken after step %d (code %d)", steps, kcache_check(cache));
        for (int e = 0; e < n; ++e) {
            if (!wants[e]) continue;
            int r = (int)(ids[e] - 100);
            generated[r]++;
            int at_limit = ksched_on_token(sched, ids[e]);
            CHECK(at_limit == (generated[r] >= NEW_TOKENS), "token limit of request %d", r);
            if (at_limit) {
                CHECK(ksched_finish(sched, ids[e]) == 0, "finish");
                done[r] = 1;
            }
        }
    }
    CHECK(saw_portion && saw_mixed, "no prompt portion beside decode tokens was ever scheduled");
    CHECK(ksched_num_preemptions(sched) > 0 && restarts[0] + restarts[1] + restarts[2] > 0,
          "a pool of %d tokens for 48 must force a preemption", PAGES * PAGE);
    CHECK(restarts[0] == 0, "the oldest request must never be the one that yields");
    CHECK(kcache_live_requests(cache) == 0 && kcache_free_pages(cache, 0) == PAGES && kcache_free_slots(cache) == MAX_REQ,
          "pages or slots were lost");
    CHECK(kcache_pages_handed_out(cache) == kcache_pages_given_back(cache), "pages handed out and given back differ");
    CHECK(kcache_check(cache) == 0, "cache invariants at the end");
    ksched_destroy(sched);
    kcache_destroy(cache);
    printf("OK %d steps, %lld preemptions\n", steps, 0LL + restarts[0] + restarts[1] + restarts[2]);
    return 0;
}
