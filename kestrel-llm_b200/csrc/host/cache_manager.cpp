// Cache manager: pages of keys and values with a block table per request and per group of
// layers, and one slot of fixed-size state per live request.
//
// The reference gives every request a private window of max_seq positions per layer and lets
// the OS fault pages in (src/model/vllm_safetensors.c:9320-9343, 9405-9433); its only
// explicit block tables are in an unused research stack (src/core/vllm_attention.c:100-129).
// Here one pool of pages per group is shared by all requests.  A group is the set of layers
// with the same need: every key ("full", window = 0) or the last `window` keys.  Layers of a
// group share a block table, so page p of the group names the same slot range in each of its
// layers' planes.
//
// Rules:
//  * pages for a step's tokens are reserved before the step runs; a reservation either gets
//    all pages it needs in every group or changes nothing;
//  * commit() advances the request's length and, in windowed groups, gives back pages that
//    no later query can reach (all their positions < length - window + 1);
//  * release() gives back everything the request holds, in every group, and its slot;
//  * free pages are a stack: the page given back last is handed out first.
// The manager only does bookkeeping on the host; device memory is owned by the caller.
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>
#include <unordered_map>
#include <vector>

#include "../../include/kestrel.h"

namespace {

struct Group {
    int window = 0;            // 0 = keep all keys
    int num_pages = 0;
    std::vector<int> free_stack;   // top = back
    std::vector<uint8_t> owned;    // 1 if handed out
};

struct Request {
    long long id = 0;
    int slot = -1;
    int length = 0;            // tokens committed
    int reserved_to = 0;       // positions [0, reserved_to) have pages where still needed
    std::vector<std::vector<int>> table;   // [group][block] -> page or -1
    std::vector<int> first_live;           // [group] first block not yet given back
};

struct Cache {
    int page_size = 0;
    int max_requests = 0;
    int max_blocks = 0;
    std::vector<Group> groups;
    std::vector<int> free_slots;           // stack
    std::unordered_map<long long, Request> live;
    std::vector<std::pair<long long, int>> admitted;   // (id, slot) of admissions not yet taken by the owner of the device state
    long long pages_handed_out = 0, pages_given_back = 0;
};

int blocks_for(int tokens, int page_size) { return (tokens + page_size - 1) / page_size; }

// first block a query at position `pos` (and later ones) can still reach in a group
int first_needed_block(const Group &g, int pos, int page_size) {
    if (g.window <= 0) return 0;
    int lo = pos - g.window + 1;
    return lo <= 0 ? 0 : lo / page_size;
}

// pages a reservation of [req.reserved_to, upto) would take in group gi
int pages_needed(const Cache &c, const Request &r, int gi, int upto) {
    const Group &g = c.groups[gi];
    int last_block = blocks_for(upto, c.page_size);        // blocks [0, last_block)
    int have = (int)r.table[gi].size();                     // blocks ever allocated (some given back)
    int first = std::max(have, first_needed_block(g, r.length, c.page_size));
    return std::max(0, last_block - first);
}

void give_back(Cache &c, int gi, int page) {
    Group &g = c.groups[gi];
    g.owned[page] = 0;
    g.free_stack.push_back(page);
    c.pages_given_back++;
}

}  // namespace

KESTREL_API void *kcache_create(int n_groups, const int *windows, const int *num_pages, int page_size,
                         int max_requests, int max_blocks_per_request) {
    if (n_groups < 0 || page_size <= 0 || max_requests <= 0 || max_blocks_per_request <= 0) return nullptr;
    Cache *c = new Cache();
    c->page_size = page_size;
    c->max_requests = max_requests;
    c->max_blocks = max_blocks_per_request;
    c->groups.resize(n_groups);
    for (int i = 0; i < n_groups; ++i) {
        Group &g = c->groups[i];
        g.window = windows[i];
        g.num_pages = num_pages[i];
        g.owned.assign(g.num_pages, 0);
        g.free_stack.reserve(g.num_pages);
        for (int p = g.num_pages - 1; p >= 0; --p) g.free_stack.push_back(p);   // page 0 first
    }
    for (int s = max_requests - 1; s >= 0; --s) c->free_slots.push_back(s);
    return c;
}

KESTREL_API void kcache_destroy(void *h) { delete (Cache *)h; }

// slot of the new request, -1 if no slot is free, -2 if the id is live already
KESTREL_API int kcache_admit(void *h, long long id) {
    Cache &c = *(Cache *)h;
    if (c.live.count(id)) return -2;
    if (c.free_slots.empty()) return -1;
    Request r;
    r.id = id;
    r.slot = c.free_slots.back();
    c.free_slots.pop_back();
    r.table.resize(c.groups.size());
    r.first_live.assign(c.groups.size(), 0);
    const int slot = r.slot;
    c.live.emplace(id, std::move(r));
    c.admitted.emplace_back(id, slot);
    return slot;
}

// The requests admitted since the last call, whoever admitted them (the caller, or the scheduler
// on its own): whoever owns per-slot state on the device clears those slots before the next
// step runs.  Writes up to cap (id, slot) pairs and forgets all of them; returns how many there were.
KESTREL_API int kcache_take_admitted(void *h, long long *ids, int *slots, int cap) {
    Cache &c = *(Cache *)h;
    int n = (int)c.admitted.size();
    for (int i = 0; i < n && i < cap; ++i) {
        if (ids) ids[i] = c.admitted[i].first;
        if (slots) slots[i] = c.admitted[i].second;
    }
    c.admitted.clear();
    return n;
}

// 1 if reserve(id, n_new) would succeed, 0 if pages are short, negative on misuse
KESTREL_API int kcache_can_reserve(void *h, long long id, int n_new) {
    Cache &c = *(Cache *)h;
    auto it = c.live.find(id);
    if (it == c.live.end()) return -3;
    const Request &r = it->second;
    int upto = r.length + n_new;
    if (blocks_for(upto, c.page_size) > c.max_blocks) return -4;
    for (size_t gi = 0; gi < c.groups.size(); ++gi)
        if (pages_needed(c, r, (int)gi, upto) > (int)c.groups[gi].free_stack.size()) return 0;
    return 1;
}

// Pages for positions [length, length + n_new) in every group.  0 = done, -1 = pages short
// (nothing changed), -3 = unknown request, -4 = longer than max_blocks_per_request allows.
KESTREL_API int kcache_reserve(void *h, long long id, int n_new) {
    Cache &c = *(Cache *)h;
    auto it = c.live.find(id);
    if (it == c.live.end()) return -3;
    Request &r = it->second;
    if (n_new < 0) return -5;
    int upto = r.length + n_new;
    if (blocks_for(upto, c.page_size) > c.max_blocks) return -4;
    for (size_t gi = 0; gi < c.groups.size(); ++gi)
        if (pages_needed(c, r, (int)gi, upto) > (int)c.groups[gi].free_stack.size()) return -1;
    int last_block = blocks_for(upto, c.page_size);
    for (size_t gi = 0; gi < c.groups.size(); ++gi) {
        Group &g = c.groups[gi];
        std::vector<int> &t = r.table[gi];
        int first = first_needed_block(g, r.length, c.page_size);
        while ((int)t.size() < last_block) {
            int b = (int)t.size();
            if (b < first) {            // behind the window already: never allocated
                t.push_back(-1);
                r.first_live[gi] = std::max(r.first_live[gi], b + 1);
                continue;
            }
            int page = g.free_stack.back();
            g.free_stack.pop_back();
            g.owned[page] = 1;
            c.pages_handed_out++;
            t.push_back(page);
        }
    }
    r.reserved_to = std::max(r.reserved_to, upto);
    return 0;
}

// length += n_new (must be reserved); windowed groups give back what fell out of reach
KESTREL_API int kcache_commit(void *h, long long id, int n_new) {
    Cache &c = *(Cache *)h;
    auto it = c.live.find(id);
    if (it == c.live.end()) return -3;
    Request &r = it->second;
    if (n_new < 0 || r.length + n_new > r.reserved_to) return -5;
    r.length += n_new;
    for (size_t gi = 0; gi < c.groups.size(); ++gi) {
        Group &g = c.groups[gi];
        if (g.window <= 0) continue;
        int first = std::min(first_needed_block(g, r.length, c.page_size), (int)r.table[gi].size());
        for (int b = r.first_live[gi]; b < first; ++b) {
            if (r.table[gi][b] >= 0) {
                give_back(c, (int)gi, r.table[gi][b]);
                r.table[gi][b] = -1;
            }
        }
        r.first_live[gi] = std::max(r.first_live[gi], first);
    }
    return 0;
}

KESTREL_API int kcache_release(void *h, long long id) {
    Cache &c = *(Cache *)h;
    auto it = c.live.find(id);
    if (it == c.live.end()) return -3;
    Request &r = it->second;
    for (size_t gi = 0; gi < c.groups.size(); ++gi)
        for (int b = (int)r.table[gi].size() - 1; b >= 0; --b)       // last block first: block 0 is reused first
            if (r.table[gi][b] >= 0) give_back(c, (int)gi, r.table[gi][b]);
    c.free_slots.push_back(r.slot);
    c.live.erase(it);
    return 0;
}

KESTREL_API int kcache_length(void *h, long long id) {
    Cache &c = *(Cache *)h;
    auto it = c.live.find(id);
    return it == c.live.end() ? -3 : it->second.length;
}

KESTREL_API int kcache_slot(void *h, long long id) {
    Cache &c = *(Cache *)h;
    auto it = c.live.find(id);
    return it == c.live.end() ? -3 : it->second.slot;
}

KESTREL_API int kcache_num_blocks(void *h, long long id, int group) {
    Cache &c = *(Cache *)h;
    auto it = c.live.find(id);
    if (it == c.live.end()) return -3;
    if (group < 0 || group >= (int)c.groups.size()) return -6;
    return (int)it->second.table[group].size();
}

// copies min(n, blocks) entries of the request's table in `group` (page id, or -1 where the
// page was given back); pads the rest of `out` with -1; returns the number of blocks
KESTREL_API int kcache_block_table(void *h, long long id, int group, int *out, int n) {
    Cache &c = *(Cache *)h;
    auto it = c.live.find(id);
    if (it == c.live.end()) return -3;
    if (group < 0 || group >= (int)c.groups.size()) return -6;
    const std::vector<int> &t = it->second.table[group];
    int m = std::min(n, (int)t.size());
    if (m > 0) memcpy(out, t.data(), sizeof(int) * m);
    for (int i = m; i < n; ++i) out[i] = -1;
    return (int)t.size();
}

// Describes a step in which each of n requests brings one token, for a batch padded to B rows:
// positions (the length so far), lengths after the step, state slots, and every group's block
// table rows [G][B][W] (-1 beyond a request's pages).  Rows n..B-1 are left untouched.  Returns
// the longest length after the step, or a negative error (then *bad is the request's index).
KESTREL_API int kcache_describe_decode(void *h, const long long *ids, int n, int B, int W, int *pos, int *kv, int *slot,
                                int *tables, int *bad) {
    Cache &c = *(Cache *)h;
    const int G = (int)c.groups.size();
    int longest = 1;
    for (int i = 0; i < n; ++i) {
        auto it = c.live.find(ids[i]);
        if (it == c.live.end()) { if (bad) *bad = i; return -3; }
        const auto &r = it->second;
        pos[i] = r.length;
        kv[i] = r.length + 1;
        slot[i] = r.slot;
        longest = std::max(longest, r.length + 1);
        for (int g = 0; g < G; ++g) {
            const std::vector<int> &t = r.table[g];
            int *row = tables + ((size_t)g * B + i) * W;
            int m = std::min(W, (int)t.size());
            if (m > 0) memcpy(row, t.data(), sizeof(int) * m);
            for (int j = m; j < W; ++j) row[j] = -1;
        }
    }
    return longest;
}

// Puts every group's free pages into a pseudo-random order (a fixed function of `seed`).  A
// fresh pool hands pages out in ascending order, so that a request's pages lie one behind the
// other; after minutes of serving they do not.  Benchmarks and tests call this to get the
// scattered layout from the start.
KESTREL_API int kcache_shuffle_free(void *h, long long seed) {
    Cache &c = *(Cache *)h;
    unsigned long long x = (unsigned long long)seed * 6364136223846793005ull + 1442695040888963407ull;
    for (Group &g : c.groups)
        for (size_t i = g.free_stack.size(); i > 1; --i) {
            x = x * 6364136223846793005ull + 1442695040888963407ull;
            size_t j = (size_t)((x >> 33) % i);
            std::swap(g.free_stack[i - 1], g.free_stack[j]);
        }
    return 0;
}

KESTREL_API int kcache_free_pages(void *h, int group) {
    Cache &c = *(Cache *)h;
    if (group < 0 || group >= (int)c.groups.size()) return -6;
    return (int)c.groups[group].free_stack.size();
}

KESTREL_API int kcache_num_pages(void *h, int group) {
    Cache &c = *(Cache *)h;
    if (group < 0 || group >= (int)c.groups.size()) return -6;
    return c.groups[group].num_pages;
}

KESTREL_API int kcache_num_groups(void *h) { return (int)((Cache *)h)->groups.size(); }
KESTREL_API int kcache_page_size(void *h) { return ((Cache *)h)->page_size; }
KESTREL_API int kcache_max_blocks(void *h) { return ((Cache *)h)->max_blocks; }
KESTREL_API int kcache_live_requests(void *h) { return (int)((Cache *)h)->live.size(); }
KESTREL_API int kcache_free_slots(void *h) { return (int)((Cache *)h)->free_slots.size(); }
KESTREL_API long long kcache_pages_handed_out(void *h) { return ((Cache *)h)->pages_handed_out; }
KESTREL_API long long kcache_pages_given_back(void *h) { return ((Cache *)h)->pages_given_back; }

// Invariants: every page of every group is on the free stack exactly once or in exactly one
// live table exactly once; slots likewise.  0 if they hold, else a negative code that says
// which one broke.
KESTREL_API int kcache_check(void *h) {
    Cache &c = *(Cache *)h;
    for (size_t gi = 0; gi < c.groups.size(); ++gi) {
        const Group &g = c.groups[gi];
        std::vector<int> seen(g.num_pages, 0);
        for (int p : g.free_stack) {
            if (p < 0 || p >= g.num_pages) return -10;
            if (g.owned[p]) return -11;            // free and owned
            if (seen[p]++) return -12;             // on the free stack twice
        }
        for (const auto &kv : c.live)
            for (int p : kv.second.table[gi]) {
                if (p < 0) continue;
                if (p >= g.num_pages) return -10;
                if (!g.owned[p]) return -13;       // held but not marked
                if (seen[p]++) return -14;         // held twice, or held and free
            }
        for (int p = 0; p < g.num_pages; ++p)
            if (!seen[p]) return -15;              // lost
    }
    std::vector<int> slot_seen(c.max_requests, 0);
    for (int s : c.free_slots) {
        if (s < 0 || s >= c.max_requests || slot_seen[s]++) return -16;
    }
    for (const auto &kv : c.live) {
        int s = kv.second.slot;
        if (s < 0 || s >= c.max_requests || slot_seen[s]++) return -17;
    }
    for (int s = 0; s < c.max_requests; ++s)
        if (!slot_seen[s]) return -18;
    return 0;
}
