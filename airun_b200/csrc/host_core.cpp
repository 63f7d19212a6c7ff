// Host-side core of the cache manager and of the step's batch metadata (no CUDA in this file).
//
// Pages of keys and values are handed out from a LIFO free list with a holder count per page;
// every request slot has, per cache group, the list of its page ids by block (position /
// page_size, -1 = given back) and a row of the group's block-table mirror, which a step copies
// to the device.  Groups with a window give pages back as the window passes them.  Pages may be
// shared between requests (fork) and a request's end may be moved back (truncate); a page that
// more than one table holds is never the page a request writes next.  build_batch lays a step's
// flat batch (token ids, positions, request of each token, wanted rows, first row and context
// length of each request, state slots, block-table rows) into the caller's pinned staging buffer.
//
// The reference keeps this bookkeeping in its runtime as well, in Rust: a contiguous cache per
// conversation slot with a position cursor (crates/airun-core/src/runtime.rs:47-57, :2865-2871),
// rewinding by moving the cursor (runtime.rs:3280-3308) and a device table of per-row cache
// pointers rewritten before each step (runtime.rs:3152-3173).  Here the same needs are met with
// pages.  Every function returns a status; the text of the last failure is kept per object.
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#define HOST_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

enum { HC_OK = 0, HC_OUT_OF_PAGES = 1, HC_MISUSE = 2 };

struct PagePool {
    int num_pages;
    std::vector<int> free_list;      // back() is handed out next
    std::vector<int> holders;
    std::string error;

    explicit PagePool(int n) : num_pages(n), holders(n, 0) {
        free_list.reserve(n);
        for (int p = n - 1; p >= 0; --p) free_list.push_back(p);      // page 0 first
    }
    int num_free() const { return (int)free_list.size(); }
    int take(int n, int* out) {
        if (n > num_free()) {
            error = std::to_string(n) + " pages wanted, " + std::to_string(num_free()) + " free of " + std::to_string(num_pages);
            return HC_OUT_OF_PAGES;
        }
        for (int i = 0; i < n; ++i) {
            const int p = free_list.back();
            if (holders[p] != 0) {
                error = "page " + std::to_string(p) + " was on the free list while held";
                return HC_MISUSE;
            }
            free_list.pop_back();
            holders[p] = 1;
            out[i] = p;
        }
        return HC_OK;
    }
    int share(int p) {
        if (p < 0 || p >= num_pages || holders[p] <= 0) {
            error = "page " + std::to_string(p) + " is not held and cannot be shared";
            return HC_MISUSE;
        }
        ++holders[p];
        return HC_OK;
    }
    int give_back(int p) {
        if (p < 0 || p >= num_pages) {
            error = "page " + std::to_string(p) + " is outside the pool";
            return HC_MISUSE;
        }
        if (holders[p] <= 0) {
            error = "page " + std::to_string(p) + " is freed twice";
            return HC_MISUSE;
        }
        if (--holders[p] == 0) free_list.push_back(p);
        return HC_OK;
    }
};

struct Group {
    int window;
    PagePool pool;
    std::vector<int32_t> table;      // [max_requests][max_blocks], -1 where no page
    Group(int w, int pages, size_t cells) : window(w), pool(pages), table(cells, -1) {}
};

struct Req {
    bool live = false;
    long long num_tokens = 0, reserved = 0;
    std::vector<std::vector<int>> blocks;       // per group
};

struct CacheCore {
    int page_size, num_pages, max_requests, max_blocks;
    bool has_state;
    std::vector<Group> groups;
    std::vector<Req> reqs;
    std::vector<int> free_slots;     // back() is handed out next
    std::string error;
    std::vector<int> scratch;

    int fail(int code, const std::string& msg) { error = msg; return code; }
    bool live(int slot) const { return slot >= 0 && slot < max_requests && reqs[slot].live; }
    long long blocks_for(long long n) const { return (n + page_size - 1) / page_size; }
    int32_t* row(int g, int slot) { return groups[g].table.data() + (size_t)slot * max_blocks; }
    void set_cell(int g, int slot, size_t b, int page) { if ((long long)b < max_blocks) row(g, slot)[b] = page; }

    int need(int slot, long long n_new, int g) const {
        const long long want = blocks_for(reqs[slot].num_tokens + n_new);
        return (int)std::max(0LL, want - (long long)reqs[slot].blocks[g].size());
    }
    // takes the pages of one request; the caller has checked that they are free
    int take_for(int slot, long long n_new) {
        Req& r = reqs[slot];
        for (size_t g = 0; g < groups.size(); ++g) {
            const int k = need(slot, n_new, (int)g);
            if (!k) continue;
            scratch.resize(k);
            const int rc = groups[g].pool.take(k, scratch.data());
            if (rc != HC_OK) return fail(rc, groups[g].pool.error);
            for (int i = 0; i < k; ++i) {
                set_cell((int)g, slot, r.blocks[g].size(), scratch[i]);
                r.blocks[g].push_back(scratch[i]);
            }
        }
        r.reserved = std::max(r.reserved, r.num_tokens + n_new);
        return HC_OK;
    }
    int commit(int slot, long long n_new) {
        Req& r = reqs[slot];
        if (r.num_tokens + n_new > r.reserved)
            return fail(HC_MISUSE, std::to_string(n_new) + " tokens committed beyond the reserved pages");
        r.num_tokens += n_new;
        for (size_t g = 0; g < groups.size(); ++g) {
            if (groups[g].window <= 0) continue;
            // the next query sits at position num_tokens and sees keys j > num_tokens - window
            const long long last_dead = r.num_tokens - groups[g].window;
            std::vector<int>& blocks = r.blocks[g];
            for (size_t b = 0; b < blocks.size() && (long long)(b + 1) * page_size - 1 <= last_dead; ++b) {
                if (blocks[b] >= 0) {
                    const int rc = groups[g].pool.give_back(blocks[b]);
                    if (rc != HC_OK) return fail(rc, groups[g].pool.error);
                    blocks[b] = -1;
                    set_cell((int)g, slot, b, -1);
                }
            }
        }
        return HC_OK;
    }
};

}  // namespace

// ------------------------------------------------------------------ page pool
HOST_EXPORT void* airun_pool_create(int num_pages) { return num_pages > 0 ? new PagePool(num_pages) : nullptr; }
HOST_EXPORT void airun_pool_destroy(void* h) { delete static_cast<PagePool*>(h); }
HOST_EXPORT const char* airun_pool_error(void* h) { return static_cast<PagePool*>(h)->error.c_str(); }
HOST_EXPORT int airun_pool_num_pages(void* h) { return static_cast<PagePool*>(h)->num_pages; }
HOST_EXPORT int airun_pool_num_free(void* h) { return static_cast<PagePool*>(h)->num_free(); }
HOST_EXPORT int airun_pool_take(void* h, int n, int* out) { return n < 0 ? HC_MISUSE : static_cast<PagePool*>(h)->take(n, out); }
HOST_EXPORT int airun_pool_share(void* h, int page) { return static_cast<PagePool*>(h)->share(page); }
HOST_EXPORT int airun_pool_give_back(void* h, int page) { return static_cast<PagePool*>(h)->give_back(page); }
HOST_EXPORT int airun_pool_holders(void* h, int page) {
    PagePool* p = static_cast<PagePool*>(h);
    return page >= 0 && page < p->num_pages ? p->holders[page] : -1;
}
HOST_EXPORT int airun_pool_free_list(void* h, int* out, int cap) {
    PagePool* p = static_cast<PagePool*>(h);
    const int n = std::min(cap, p->num_free());
    std::copy(p->free_list.begin(), p->free_list.begin() + n, out);
    return p->num_free();
}

// ------------------------------------------------------------------ cache core
HOST_EXPORT void* airun_cache_create(int n_groups, const int* windows, int page_size, int num_pages, int max_requests,
                                     int max_blocks, int has_state) {
    if (n_groups < 0 || page_size <= 0 || num_pages <= 0 || max_requests <= 0 || max_blocks <= 0) return nullptr;
    CacheCore* c = new CacheCore();
    c->page_size = page_size; c->num_pages = num_pages; c->max_requests = max_requests; c->max_blocks = max_blocks;
    c->has_state = has_state != 0;
    c->groups.reserve(n_groups);
    for (int g = 0; g < n_groups; ++g) c->groups.emplace_back(windows[g], num_pages, (size_t)max_requests * max_blocks);
    c->reqs.resize(max_requests);
    for (int s = max_requests - 1; s >= 0; --s) c->free_slots.push_back(s);
    return c;
}
HOST_EXPORT void airun_cache_destroy(void* h) { delete static_cast<CacheCore*>(h); }
HOST_EXPORT const char* airun_cache_error(void* h) { return static_cast<CacheCore*>(h)->error.c_str(); }
HOST_EXPORT void* airun_cache_pool(void* h, int g) { return &static_cast<CacheCore*>(h)->groups[g].pool; }
HOST_EXPORT int32_t* airun_cache_table(void* h, int g) { return static_cast<CacheCore*>(h)->groups[g].table.data(); }
HOST_EXPORT int airun_cache_has_free_slot(void* h) { return static_cast<CacheCore*>(h)->free_slots.empty() ? 0 : 1; }
HOST_EXPORT int airun_cache_num_live(void* h) {
    CacheCore* c = static_cast<CacheCore*>(h);
    return c->max_requests - (int)c->free_slots.size();
}

HOST_EXPORT int airun_cache_add(void* h) {
    CacheCore* c = static_cast<CacheCore*>(h);
    if (c->free_slots.empty()) return -1;
    const int s = c->free_slots.back();
    c->free_slots.pop_back();
    Req& r = c->reqs[s];
    r.live = true;
    r.num_tokens = r.reserved = 0;
    r.blocks.assign(c->groups.size(), std::vector<int>());
    return s;
}

HOST_EXPORT int airun_cache_free(void* h, int slot) {
    CacheCore* c = static_cast<CacheCore*>(h);
    if (!c->live(slot)) return c->fail(HC_MISUSE, "the request is freed twice or was never added");
    Req& r = c->reqs[slot];
    for (size_t g = 0; g < c->groups.size(); ++g) {
        for (int p : r.blocks[g])
            if (p >= 0) {
                const int rc = c->groups[g].pool.give_back(p);
                if (rc != HC_OK) return c->fail(rc, c->groups[g].pool.error);
            }
        const size_t n = std::min<size_t>(r.blocks[g].size(), c->max_blocks);
        std::fill(c->row((int)g, slot), c->row((int)g, slot) + n, -1);
        r.blocks[g].clear();
    }
    r.live = false;
    c->free_slots.push_back(slot);
    return HC_OK;
}

HOST_EXPORT long long airun_cache_num_tokens(void* h, int slot) {
    CacheCore* c = static_cast<CacheCore*>(h);
    return c->live(slot) ? c->reqs[slot].num_tokens : -1;
}
HOST_EXPORT long long airun_cache_reserved(void* h, int slot) {
    CacheCore* c = static_cast<CacheCore*>(h);
    return c->live(slot) ? c->reqs[slot].reserved : -1;
}
HOST_EXPORT int airun_cache_num_blocks(void* h, int slot, int g) {
    CacheCore* c = static_cast<CacheCore*>(h);
    return c->live(slot) ? (int)c->reqs[slot].blocks[g].size() : -1;
}
HOST_EXPORT int airun_cache_blocks(void* h, int slot, int g, int* out, int cap) {
    CacheCore* c = static_cast<CacheCore*>(h);
    if (!c->live(slot)) return -1;
    const std::vector<int>& b = c->reqs[slot].blocks[g];
    std::copy(b.begin(), b.begin() + std::min<size_t>(cap, b.size()), out);
    return (int)b.size();
}

HOST_EXPORT int airun_cache_pages_needed(void* h, int slot, long long n_new, int* out) {
    CacheCore* c = static_cast<CacheCore*>(h);
    if (!c->live(slot)) return c->fail(HC_MISUSE, "the request is not live");
    for (size_t g = 0; g < c->groups.size(); ++g) out[g] = c->need(slot, n_new, (int)g);
    return HC_OK;
}

// Takes the pages for the next n_new[i] tokens of every listed request, or none at all.
HOST_EXPORT int airun_cache_reserve_many(void* h, int count, const int* slots, const long long* n_new) {
    CacheCore* c = static_cast<CacheCore*>(h);
    for (int i = 0; i < count; ++i)
        if (!c->live(slots[i]) || n_new[i] < 0) return c->fail(HC_MISUSE, "the request is not live");
    for (size_t g = 0; g < c->groups.size(); ++g) {
        long long total = 0;
        for (int i = 0; i < count; ++i) total += c->need(slots[i], n_new[i], (int)g);
        if (total > c->groups[g].pool.num_free())
            return c->fail(HC_OUT_OF_PAGES, std::to_string(total) + " pages needed in group " + std::to_string(g) + ", " +
                                                std::to_string(c->groups[g].pool.num_free()) + " free");
    }
    for (int i = 0; i < count; ++i) {
        const int rc = c->take_for(slots[i], n_new[i]);
        if (rc != HC_OK) return rc;
    }
    return HC_OK;
}

HOST_EXPORT int airun_cache_commit_many(void* h, int count, const int* slots, const long long* n_new) {
    CacheCore* c = static_cast<CacheCore*>(h);
    for (int i = 0; i < count; ++i) {
        if (!c->live(slots[i]) || n_new[i] < 0) return c->fail(HC_MISUSE, "the request is not live");
        const int rc = c->commit(slots[i], n_new[i]);
        if (rc != HC_OK) return rc;
    }
    return HC_OK;
}

// child: a new slot holding the parent's tokens.  copies: up to n_groups triples (group, src, dst).
HOST_EXPORT int airun_cache_fork(void* h, int parent, int* child_slot, int* copies, int* n_copies) {
    CacheCore* c = static_cast<CacheCore*>(h);
    *n_copies = 0;
    if (!c->live(parent)) return c->fail(HC_MISUSE, "the request is not live");
    if (c->free_slots.empty()) return c->fail(HC_MISUSE, "all " + std::to_string(c->max_requests) + " request slots are in use");
    Req& p = c->reqs[parent];
    const long long full = p.num_tokens / c->page_size, part = p.num_tokens % c->page_size;
    for (size_t g = 0; g < c->groups.size(); ++g)
        if (part && p.blocks[g][full] >= 0 && c->groups[g].pool.num_free() < 1)
            return c->fail(HC_OUT_OF_PAGES, "the fork needs a page in group " + std::to_string(g) + ", none is free");
    const int s = airun_cache_add(h);
    Req& k = c->reqs[s];
    Req& par = c->reqs[parent];
    k.num_tokens = k.reserved = par.num_tokens;
    for (size_t g = 0; g < c->groups.size(); ++g) {
        std::vector<int>& blocks = k.blocks[g];
        blocks.assign(par.blocks[g].begin(), par.blocks[g].begin() + full);
        for (int pg : blocks)
            if (pg >= 0) c->groups[g].pool.share(pg);
        if (part) {
            const int src = par.blocks[g][full];
            if (src >= 0) {
                int fresh = -1;
                c->groups[g].pool.take(1, &fresh);
                copies[3 * *n_copies] = (int)g; copies[3 * *n_copies + 1] = src; copies[3 * *n_copies + 2] = fresh;
                ++*n_copies;
                blocks.push_back(fresh);
            } else {
                blocks.push_back(-1);
            }
        }
        for (size_t b = 0; b < blocks.size(); ++b) c->set_cell((int)g, s, b, blocks[b]);
    }
    *child_slot = s;
    return HC_OK;
}

HOST_EXPORT int airun_cache_truncate(void* h, int slot, long long n_tokens, int* copies, int* n_copies) {
    CacheCore* c = static_cast<CacheCore*>(h);
    *n_copies = 0;
    if (!c->live(slot)) return c->fail(HC_MISUSE, "the request is not live");
    Req& r = c->reqs[slot];
    if (n_tokens < 0 || n_tokens > r.num_tokens)
        return c->fail(HC_MISUSE, "the request holds " + std::to_string(r.num_tokens) + " tokens and cannot be cut to " + std::to_string(n_tokens));
    if (n_tokens == r.num_tokens && r.reserved == r.num_tokens) return HC_OK;
    if (c->has_state && n_tokens < r.num_tokens)
        return c->fail(HC_MISUSE, "a request with fixed-size state cannot be moved back, only restarted");
    const long long full = n_tokens / c->page_size, part = n_tokens % c->page_size;
    for (size_t g = 0; g < c->groups.size(); ++g) {
        const std::vector<int>& blocks = r.blocks[g];
        const int w = c->groups[g].window;
        if (w > 0 && n_tokens > 0) {
            const long long first_needed = std::max(0LL, n_tokens - w + 1) / c->page_size;
            if (first_needed < (long long)blocks.size() && blocks[first_needed] < 0)
                return c->fail(HC_MISUSE, "the window's pages before token " + std::to_string(n_tokens) + " were given back");
        }
        if (part && blocks[full] >= 0 && c->groups[g].pool.holders[blocks[full]] > 1 && c->groups[g].pool.num_free() < 1)
            return c->fail(HC_OUT_OF_PAGES, "cutting inside a shared page needs a page in group " + std::to_string(g));
    }
    const size_t keep = (size_t)(full + (part ? 1 : 0));
    for (size_t g = 0; g < c->groups.size(); ++g) {
        std::vector<int>& blocks = r.blocks[g];
        for (size_t b = keep; b < blocks.size(); ++b) {
            if (blocks[b] >= 0) c->groups[g].pool.give_back(blocks[b]);
            c->set_cell((int)g, slot, b, -1);
        }
        if (blocks.size() > keep) blocks.resize(keep);
        if (part && blocks[full] >= 0 && c->groups[g].pool.holders[blocks[full]] > 1) {
            int fresh = -1;
            c->groups[g].pool.take(1, &fresh);
            copies[3 * *n_copies] = (int)g; copies[3 * *n_copies + 1] = blocks[full]; copies[3 * *n_copies + 2] = fresh;
            ++*n_copies;
            c->groups[g].pool.give_back(blocks[full]);
            blocks[full] = fresh;
            c->set_cell((int)g, slot, (size_t)full, fresh);
        }
    }
    r.num_tokens = r.reserved = n_tokens;
    return HC_OK;
}

// No page lost, none held twice, none both free and held; the page a request writes next has no
// other holder; the block-table mirror equals the lists; no request slot lost or held twice.
HOST_EXPORT int airun_cache_check(void* h) {
    CacheCore* c = static_cast<CacheCore*>(h);
    for (size_t g = 0; g < c->groups.size(); ++g) {
        PagePool& pool = c->groups[g].pool;
        std::vector<int> seen(pool.num_pages, 0), is_free(pool.num_pages, 0);
        for (int s = 0; s < c->max_requests; ++s) {
            if (!c->reqs[s].live) continue;
            const std::vector<int>& blocks = c->reqs[s].blocks[g];
            for (size_t b = 0; b < blocks.size(); ++b) {
                const int p = blocks[b];
                if (p >= pool.num_pages) return c->fail(HC_MISUSE, "group " + std::to_string(g) + ": a block names a page outside the pool");
                if (p >= 0) ++seen[p];
                if ((long long)b < c->max_blocks && c->row((int)g, s)[b] != p)
                    return c->fail(HC_MISUSE, "group " + std::to_string(g) + ": the block-table mirror of slot " + std::to_string(s) + " differs at block " + std::to_string(b));
            }
            for (size_t b = (size_t)(c->reqs[s].num_tokens / c->page_size); b < blocks.size(); ++b)
                if (blocks[b] >= 0 && pool.holders[blocks[b]] != 1)
                    return c->fail(HC_MISUSE, "group " + std::to_string(g) + ": slot " + std::to_string(s) + " would write page " +
                                                  std::to_string(blocks[b]) + ", which " + std::to_string(pool.holders[blocks[b]]) + " tables hold");
        }
        for (int p : pool.free_list) {
            if (is_free[p]) return c->fail(HC_MISUSE, "group " + std::to_string(g) + ": page " + std::to_string(p) + " is on the free list twice");
            is_free[p] = 1;
            if (seen[p]) return c->fail(HC_MISUSE, "group " + std::to_string(g) + ": page " + std::to_string(p) + " is both free and held");
        }
        int held = 0;
        for (int p = 0; p < pool.num_pages; ++p) {
            if (seen[p]) {
                ++held;
                if (pool.holders[p] != seen[p])
                    return c->fail(HC_MISUSE, "group " + std::to_string(g) + ": page " + std::to_string(p) + " is in " + std::to_string(seen[p]) +
                                                  " tables but has " + std::to_string(pool.holders[p]) + " holders");
            }
        }
        if (held + pool.num_free() != pool.num_pages)
            return c->fail(HC_MISUSE, "group " + std::to_string(g) + ": " + std::to_string(pool.num_pages - held - pool.num_free()) + " pages are lost");
    }
    std::vector<int> slot_seen(c->max_requests, 0);
    int live = 0;
    for (int s = 0; s < c->max_requests; ++s) if (c->reqs[s].live) { ++live; slot_seen[s] = 1; }
    for (int s : c->free_slots) {
        if (s < 0 || s >= c->max_requests || slot_seen[s]) return c->fail(HC_MISUSE, "a request slot is held twice");
        slot_seen[s] = 1;
    }
    if (live + (int)c->free_slots.size() != c->max_requests) return c->fail(HC_MISUSE, "a request slot is lost");
    return HC_OK;
}

// Lays the batch of one step into the staging buffer `base` (int32 words).  offs: word offsets of
// token_ids, positions, req_of_token, want_rows, cu_tokens, context_lens, state_slots, then one
// block-table area [R_max][bt_cols] per group.  tokens: the entries' tokens one after the other;
// want: the wanted places of every entry (relative to its own tokens), want_counts of them each.
// pad_to > 0: rows up to pad_to belong to request -1 at position -1 and cu_tokens is filled to
// R_max; pad_want: wanted rows up to pad_want name row 0.  out: {tokens, wanted rows, longest
// context, longest portion, then per group the shared prefix}.  The shared prefix of a group, also
// written to the word at offs[7 + groups + g], is the number of tokens at the start of every
// request of the batch that lie in the very same pages (requests forked from one): whole pages only,
// 0 unless every request brings a single token, there are two or more, and the group has no window.
HOST_EXPORT int airun_cache_build_batch(void* h, int count, const int* slots, const int* qlens, const int32_t* tokens,
                                        const int* want_counts, const int* want, int32_t* base, const long long* offs,
                                        int R_max, int bt_cols, int pad_to, int pad_want, long long* out) {
    CacheCore* c = static_cast<CacheCore*>(h);
    if (count < 0 || count > R_max) return c->fail(HC_MISUSE, "more requests than the batch has rows for");
    int32_t* tok = base + offs[0];
    int32_t* pos = base + offs[1];
    int32_t* rot = base + offs[2];
    int32_t* wr = base + offs[3];
    int32_t* cu = base + offs[4];
    int32_t* cl = base + offs[5];
    int32_t* sl = base + offs[6];
    long long t = 0, n_want = 0, max_ctx = 0, max_q = 0;
    const int32_t* src = tokens;
    const int* w = want;
    for (int r = 0; r < count; ++r) {
        const int s = slots[r];
        if (!c->live(s) || qlens[r] <= 0) return c->fail(HC_MISUSE, "the request is not live or brings no tokens");
        const long long start = c->reqs[s].num_tokens, n = qlens[r];
        std::memcpy(tok + t, src, (size_t)n * sizeof(int32_t));
        src += n;
        for (long long i = 0; i < n; ++i) { pos[t + i] = (int32_t)(start + i); rot[t + i] = r; }
        for (int i = 0; i < want_counts[r]; ++i) {
            if (w[i] < 0 || w[i] >= n) return c->fail(HC_MISUSE, "a wanted place lies outside the request's tokens");
            wr[n_want++] = (int32_t)(t + w[i]);
        }
        w += want_counts[r];
        cu[r] = (int32_t)t;
        cl[r] = (int32_t)(start + n);
        sl[r] = s;
        max_ctx = std::max(max_ctx, start + n);
        max_q = std::max(max_q, n);
        t += n;
    }
    cu[count] = (int32_t)t;
    const long long need_blocks = std::min<long long>(std::min<long long>(c->blocks_for(max_ctx), c->max_blocks), bt_cols);
    for (size_t g = 0; g < c->groups.size(); ++g) {
        int32_t* bt = base + offs[7 + g];
        for (int r = 0; r < count; ++r)
            std::memcpy(bt + (size_t)r * bt_cols, c->row((int)g, slots[r]), (size_t)need_blocks * sizeof(int32_t));
    }
    for (size_t g = 0; g < c->groups.size(); ++g) {
        long long shared = 0;
        if (count >= 2 && max_q == 1 && c->groups[g].window == 0) {
            long long blocks = c->max_blocks;
            for (int r = 0; r < count; ++r) blocks = std::min(blocks, c->reqs[slots[r]].num_tokens / c->page_size);
            const int32_t* first = c->row((int)g, slots[0]);
            for (int r = 1; r < count && blocks > 0; ++r) {
                const int32_t* other = c->row((int)g, slots[r]);
                long long b = 0;
                while (b < blocks && other[b] == first[b] && first[b] >= 0) ++b;
                blocks = b;
            }
            shared = blocks * c->page_size;
        }
        base[offs[7 + c->groups.size() + g]] = (int32_t)shared;
        out[4 + g] = shared;
    }
    const long long real = t;
    if (pad_to > 0) {
        for (int r = count; r < R_max; ++r) cu[r + 1] = (int32_t)real;
        for (; t < pad_to; ++t) { tok[t] = 0; pos[t] = -1; rot[t] = -1; }
    }
    for (long long i = n_want; i < pad_want; ++i) wr[i] = 0;
    out[0] = real; out[1] = n_want; out[2] = max_ctx; out[3] = max_q;
    return HC_OK;
}
