// The engine's host-side bookkeeping in C++ (no CUDA): the page pools and block tables of the
// cache groups with the request slots, the scheduler's decisions of one step, and the assembly
// of a step's batch arrays.  C interface for ctypes; the Python classes CacheManager, Scheduler
// and ModelRunner are thin layers over it that own the device tensors and the request records.
//
// Counterparts in the reference: BlockManager (spymaster2h/spyinfer
// src/engine/block_manager.cpp:5-42: ids 0..N-1, allocate pops the free list's end, free pushes
// back), the per-sequence block vectors (src/engine/sequence.hpp:29) and Scheduler::schedule
// (src/engine/scheduler.cpp:17-122).  What differs is stated where it does.
//
// Every function returns 0 on success or one of the codes below after storing a message that
// spy_engine_core_last_error() returns; nothing throws across the interface.
#include <algorithm>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

namespace {

enum { OK = 0, OUT_OF_PAGES = 1, BAD_VALUE = 2, BROKEN = 3, NO_SLOT = 4, UNKNOWN_REQUEST = 5 };

thread_local char g_error[1024] = "";

int fail(int code, const char* fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return code;
}

// A pool of page ids with a last-in-first-out free list: the page given back last is handed out next.
struct PagePool {
    std::vector<int> free_list;
    std::vector<uint8_t> is_free;

    explicit PagePool(int n) : is_free((size_t)n, 1)
    {
        free_list.reserve((size_t)n);
        for (int p = n - 1; p >= 0; --p) free_list.push_back(p);   // page 0 is handed out first
    }
    int size() const { return (int)is_free.size(); }
    int num_free() const { return (int)free_list.size(); }
    int allocate()
    {
        const int p = free_list.back();
        free_list.pop_back();
        is_free[(size_t)p] = 0;
        return p;
    }
    int release(int p)
    {
        if (p < 0 || p >= size()) return fail(BAD_VALUE, "page %d is not of this pool (0..%d)", p, size() - 1);
        if (is_free[(size_t)p]) return fail(BAD_VALUE, "page %d is freed twice", p);
        is_free[(size_t)p] = 1;
        free_list.push_back(p);
        return OK;
    }
};

struct Group {
    int window;                    // -1: every key is kept
    PagePool pool;
    std::vector<int32_t> tables;   // [max_num_seqs][width], row = state slot, -1 = no page
    Group(int window_, int num_pages, int max_num_seqs, int width) : window(window_), pool(num_pages), tables((size_t)max_num_seqs * width, -1) {}
};

struct Request {
    int slot;
    int length;     // tokens stored (committed)
    int reserved;   // tokens that have pages
};

struct Cache {
    int page_size, num_pages, max_num_seqs, max_model_len, width;
    std::vector<Group> groups;
    std::vector<int> free_slots;
    std::unordered_map<int64_t, Request> requests;

    int pages_for(int length) const { return (length + page_size - 1) / page_size; }
    int min_free_pages() const
    {
        int m = num_pages;
        for (const Group& g : groups) m = std::min(m, g.pool.num_free());
        return m;
    }
    Request* find(int64_t rid)
    {
        auto it = requests.find(rid);
        return it == requests.end() ? nullptr : &it->second;
    }
    int pages_needed(const Request& r, int new_length) const { return std::max(0, pages_for(new_length) - pages_for(r.reserved)); }
    bool can_reserve(const Request& r, int new_length) const
    {
        if (new_length > max_model_len) return false;
        const int need = pages_needed(r, new_length);
        for (const Group& g : groups)
            if (g.pool.num_free() < need) return false;
        return true;
    }
    // All or nothing: no page is taken when one group cannot give what is needed.
    int reserve(int64_t rid, Request& r, int new_length)
    {
        if (new_length > max_model_len) return fail(BAD_VALUE, "request %lld: %d tokens exceed max_model_len %d", (long long)rid, new_length, max_model_len);
        if (new_length <= r.reserved) return OK;
        const int need = pages_needed(r, new_length);
        for (const Group& g : groups)
            if (g.pool.num_free() < need) return fail(OUT_OF_PAGES, "Out of memory: No free blocks available.");
        const int first = pages_for(r.reserved), last = pages_for(new_length);
        for (Group& g : groups) {
            int32_t* row = g.tables.data() + (size_t)r.slot * width;
            for (int lp = first; lp < last; ++lp) row[lp] = g.pool.allocate();
        }
        r.reserved = new_length;
        return OK;
    }
    int add(int64_t rid, int* slot_out)
    {
        if (requests.count(rid)) return fail(BAD_VALUE, "request %lld is already live", (long long)rid);
        if (free_slots.empty()) return fail(NO_SLOT, "all %d request slots are taken", max_num_seqs);
        const int slot = free_slots.back();
        free_slots.pop_back();
        requests[rid] = Request{slot, 0, 0};
        if (slot_out) *slot_out = slot;
        return OK;
    }
    int release_request(int64_t rid)
    {
        auto it = requests.find(rid);
        if (it == requests.end()) return fail(UNKNOWN_REQUEST, "request %lld is not live", (long long)rid);
        const int slot = it->second.slot;
        for (Group& g : groups) {
            int32_t* row = g.tables.data() + (size_t)slot * width;
            for (int lp = 0; lp < width; ++lp)
                if (row[lp] >= 0) {
                    if (int rc = g.pool.release(row[lp])) return rc;
                    row[lp] = -1;
                }
        }
        free_slots.push_back(slot);
        requests.erase(it);
        return OK;
    }
};

}  // namespace

extern "C" {

const char* spy_engine_core_last_error() { return g_error; }

// ---- a page pool on its own ---------------------------------------------------------------------
void* spy_pool_create(int num_pages)
{
    if (num_pages <= 0) {
        fail(BAD_VALUE, "a page pool needs at least one page, found %d", num_pages);
        return nullptr;
    }
    return new PagePool(num_pages);
}
void spy_pool_destroy(void* h) { delete static_cast<PagePool*>(h); }
int spy_pool_num_free(void* h) { return static_cast<PagePool*>(h)->num_free(); }
int spy_pool_is_free(void* h, int page)
{
    PagePool* p = static_cast<PagePool*>(h);
    return page >= 0 && page < p->size() && p->is_free[(size_t)page] ? 1 : 0;
}
int spy_pool_allocate(void* h, int* page)
{
    PagePool* p = static_cast<PagePool*>(h);
    if (p->num_free() == 0) return fail(OUT_OF_PAGES, "Out of memory: No free blocks available.");
    *page = p->allocate();
    return OK;
}
int spy_pool_free(void* h, int page) { return static_cast<PagePool*>(h)->release(page); }

// ---- the cache's bookkeeping --------------------------------------------------------------------
// windows[g]: the window of group g in tokens, or -1.  group_pages[g]: the pages of group g's pool
// (null: num_pages for every group); a windowed group, whose requests give pages back as the window
// passes them, can do with fewer than a group that keeps every key.  num_pages is the size of the
// largest pool.
void* spy_cache_create(int num_groups, const int* windows, const int* group_pages, int page_size, int num_pages, int max_num_seqs, int max_model_len)
{
    for (int g = 0; group_pages != nullptr && g < num_groups; ++g)
        if (group_pages[g] <= 0 || group_pages[g] > num_pages) {
            fail(BAD_VALUE, "group %d: %d pages, expected 1..%d", g, group_pages[g], num_pages);
            return nullptr;
        }
    if (num_groups < 0 || page_size <= 0 || num_pages <= 0 || max_num_seqs <= 0 || max_model_len <= 0) {
        fail(BAD_VALUE, "page_size, num_pages, max_num_seqs and max_model_len must be positive");
        return nullptr;
    }
    Cache* c = new Cache();
    c->page_size = page_size;
    c->num_pages = num_pages;
    c->max_num_seqs = max_num_seqs;
    c->max_model_len = max_model_len;
    c->width = (max_model_len + page_size - 1) / page_size;
    for (int g = 0; g < num_groups; ++g) c->groups.emplace_back(windows[g], group_pages ? group_pages[g] : num_pages, max_num_seqs, c->width);
    for (int s = max_num_seqs - 1; s >= 0; --s) c->free_slots.push_back(s);   // slot 0 is handed out first
    return c;
}

void spy_cache_destroy(void* h) { delete static_cast<Cache*>(h); }

int spy_cache_width(void* h) { return static_cast<Cache*>(h)->width; }
int spy_cache_num_free_pages(void* h, int group)
{
    Cache* c = static_cast<Cache*>(h);
    return c->groups.empty() ? c->num_pages : c->groups[(size_t)group].pool.num_free();
}
int spy_cache_min_free_pages(void* h) { return static_cast<Cache*>(h)->min_free_pages(); }
int spy_cache_num_free_slots(void* h) { return (int)static_cast<Cache*>(h)->free_slots.size(); }
int spy_cache_num_live(void* h) { return (int)static_cast<Cache*>(h)->requests.size(); }
int spy_cache_live(void* h, int64_t* out)
{
    int n = 0;
    for (const auto& kv : static_cast<Cache*>(h)->requests) out[n++] = kv.first;
    return n;
}
int32_t* spy_cache_tables(void* h, int group) { return static_cast<Cache*>(h)->groups[(size_t)group].tables.data(); }

int spy_cache_has_request(void* h, int64_t rid) { return static_cast<Cache*>(h)->requests.count(rid) ? 1 : 0; }

int spy_cache_add_request(void* h, int64_t rid, int* slot_out) { return static_cast<Cache*>(h)->add(rid, slot_out); }

// slot, length and reserved length of a live request
int spy_cache_request(void* h, int64_t rid, int* slot, int* length, int* reserved)
{
    Request* r = static_cast<Cache*>(h)->find(rid);
    if (!r) return fail(UNKNOWN_REQUEST, "request %lld is not live", (long long)rid);
    if (slot) *slot = r->slot;
    if (length) *length = r->length;
    if (reserved) *reserved = r->reserved;
    return OK;
}

int spy_cache_pages_needed(void* h, int64_t rid, int new_length, int* pages)
{
    Cache* c = static_cast<Cache*>(h);
    Request* r = c->find(rid);
    if (!r) return fail(UNKNOWN_REQUEST, "request %lld is not live", (long long)rid);
    *pages = c->pages_needed(*r, new_length);
    return OK;
}

int spy_cache_can_reserve(void* h, int64_t rid, int new_length, int* yes)
{
    Cache* c = static_cast<Cache*>(h);
    Request* r = c->find(rid);
    if (!r) return fail(UNKNOWN_REQUEST, "request %lld is not live", (long long)rid);
    *yes = c->can_reserve(*r, new_length) ? 1 : 0;
    return OK;
}

// Gives the request the pages its positions [reserved, new_length) will be stored in, in every group.
int spy_cache_reserve(void* h, int64_t rid, int new_length)
{
    Cache* c = static_cast<Cache*>(h);
    Request* r = c->find(rid);
    if (!r) return fail(UNKNOWN_REQUEST, "request %lld is not live", (long long)rid);
    return c->reserve(rid, *r, new_length);
}

// The step that stored positions up to new_length has been issued: the length advances and
// windowed groups give back the pages that no later query can see.
int spy_cache_commit(void* h, int64_t rid, int new_length)
{
    Cache* c = static_cast<Cache*>(h);
    Request* r = c->find(rid);
    if (!r) return fail(UNKNOWN_REQUEST, "request %lld is not live", (long long)rid);
    if (new_length > r->reserved) return fail(BAD_VALUE, "request %lld: commit of %d tokens, only %d have pages", (long long)rid, new_length, r->reserved);
    if (new_length < r->length) return fail(BAD_VALUE, "request %lld: length cannot shrink from %d to %d", (long long)rid, r->length, new_length);
    r->length = new_length;
    for (Group& g : c->groups) {
        if (g.window < 0) continue;
        const int first_needed = std::max(0, new_length - g.window + 1) / c->page_size;   // lowest page a query at new_length or later still sees
        int32_t* row = g.tables.data() + (size_t)r->slot * c->width;
        for (int lp = 0; lp < first_needed && lp < c->width; ++lp)
            if (row[lp] >= 0) {
                if (int rc = g.pool.release(row[lp])) return rc;
                row[lp] = -1;
            }
    }
    return OK;
}

int spy_cache_free_request(void* h, int64_t rid) { return static_cast<Cache*>(h)->release_request(rid); }

int spy_cache_commit(void* h, int64_t rid, int new_length);

// A step has been issued: every request of it advances by the tokens it brought.
int spy_cache_advance(void* h, int n, const int64_t* rids, const int32_t* counts)
{
    Cache* c = static_cast<Cache*>(h);
    for (int i = 0; i < n; ++i) {
        Request* r = c->find(rids[i]);
        if (!r) return fail(UNKNOWN_REQUEST, "request %lld is not live", (long long)rids[i]);
        if (int rc = spy_cache_commit(h, rids[i], r->length + counts[i])) return rc;
    }
    return OK;
}

// Rows of group `group`'s block table for n requests, `width` entries each, into out (rows out_stride apart).
int spy_cache_gather(void* h, int group, int n, const int64_t* rids, int width, int32_t* out, int out_stride)
{
    Cache* c = static_cast<Cache*>(h);
    if (group < 0 || group >= (int)c->groups.size() || width < 0 || width > c->width) return fail(BAD_VALUE, "gather: group %d or width %d is out of range", group, width);
    const Group& g = c->groups[(size_t)group];
    for (int i = 0; i < n; ++i) {
        Request* r = c->find(rids[i]);
        if (!r) return fail(UNKNOWN_REQUEST, "request %lld is not live", (long long)rids[i]);
        std::memcpy(out + (size_t)i * out_stride, g.tables.data() + (size_t)r->slot * c->width, (size_t)width * sizeof(int32_t));
    }
    return OK;
}

// No page is lost, held twice, or both free and held; slots likewise.
int spy_cache_check(void* h)
{
    Cache* c = static_cast<Cache*>(h);
    std::vector<uint8_t> live_slot((size_t)c->max_num_seqs, 0);
    for (const auto& kv : c->requests) {
        const int s = kv.second.slot;
        if (s < 0 || s >= c->max_num_seqs || live_slot[(size_t)s]) return fail(BROKEN, "state slots are lost or held twice");
        live_slot[(size_t)s] = 1;
    }
    for (int s : c->free_slots)
        if (s < 0 || s >= c->max_num_seqs || live_slot[(size_t)s]) return fail(BROKEN, "state slots are lost or held twice");
        else live_slot[(size_t)s] = 2;
    if ((int)c->requests.size() + (int)c->free_slots.size() != c->max_num_seqs) return fail(BROKEN, "state slots are lost or held twice");
    for (size_t gi = 0; gi < c->groups.size(); ++gi) {
        const Group& g = c->groups[gi];
        const int pool_pages = g.pool.size();
        std::vector<uint8_t> seen((size_t)pool_pages, 0);   // 1: held, 2: free
        int held = 0;
        for (int s = 0; s < c->max_num_seqs; ++s) {
            const int32_t* row = g.tables.data() + (size_t)s * c->width;
            for (int lp = 0; lp < c->width; ++lp) {
                const int p = row[lp];
                if (p < 0) continue;
                if (live_slot[(size_t)s] != 1) return fail(BROKEN, "group %zu: slot %d has no request but still names pages", gi, s);
                if (p >= pool_pages) return fail(BROKEN, "group %zu: slot %d names page %d, which is not of the pool", gi, s, p);
                if (seen[(size_t)p]) return fail(BROKEN, "group %zu: page %d is held twice", gi, p);
                seen[(size_t)p] = 1;
                ++held;
            }
        }
        for (int p : g.pool.free_list) {
            if (p < 0 || p >= pool_pages) return fail(BROKEN, "group %zu: the free list names page %d", gi, p);
            if (seen[(size_t)p] == 2) return fail(BROKEN, "group %zu: page %d is on the free list twice", gi, p);
            if (seen[(size_t)p] == 1) return fail(BROKEN, "group %zu: page %d is both free and held", gi, p);
            seen[(size_t)p] = 2;
        }
        if (held + g.pool.num_free() != pool_pages) return fail(BROKEN, "group %zu: %d pages are lost", gi, pool_pages - held - g.pool.num_free());
    }
    return OK;
}

// ---- the batch arrays of one step ------------------------------------------------------------
// n entries: request rids[i] brings counts[i] tokens (tokens: all of them, one after the other)
// and wants the logits at want[want_start[i] .. want_start[i + 1]) (places among its tokens).
// Requests that are not live yet get a slot.  Pages for the new tokens are reserved.  Writes
//   token_ids[T], positions[T], seq_of_token[T], q_start[n + 1], ctx_len[n], state_slot[n],
//   logit_rows[R]; *tokens_out = T, *rows_out = R, *max_ctx = the longest context.
// All or nothing: every entry is checked first (each request once, token ids, wanted places,
// max_model_len, and the slots and pages that ALL entries together need against what is free), so an
// error leaves no slot taken and no page reserved.
int spy_cache_fill_batch(void* h, int n, const int64_t* rids, const int32_t* counts, const int32_t* tokens, const int32_t* want_start,
                         const int32_t* want, int vocab_size, int32_t* token_ids, int32_t* positions, int32_t* seq_of_token, int32_t* q_start,
                         int32_t* ctx_len, int32_t* state_slot, int32_t* logit_rows, int* tokens_out, int* rows_out, int* max_ctx)
{
    Cache* c = static_cast<Cache*>(h);
    int T = 0, R = 0, longest = 0;
    {   // the checks, before anything is taken
        std::unordered_set<int64_t> seen;
        long long pages = 0;
        int slots = 0, t0 = 0;
        for (int i = 0; i < n; ++i) {
            if (!seen.insert(rids[i]).second) return fail(BAD_VALUE, "entry %d: its request appears twice in one step", i);
            const int cnt = counts[i];
            if (cnt <= 0) return fail(BAD_VALUE, "entry %d: its request brings no tokens to this step", i);
            const Request* r = c->find(rids[i]);
            const Request fresh{-1, 0, 0};
            if (!r) ++slots;
            const Request& q = r ? *r : fresh;
            if (q.length + cnt > c->max_model_len)
                return fail(BAD_VALUE, "entry %d: request %lld: %d tokens exceed max_model_len %d", i, (long long)rids[i], q.length + cnt, c->max_model_len);
            pages += c->pages_needed(q, q.length + cnt);
            for (int k = 0; k < cnt; ++k) {
                const int t = tokens[t0 + k];
                if (t < 0 || t >= vocab_size) return fail(BAD_VALUE, "entry %d: token id %d is outside the vocabulary of %d", i, t, vocab_size);
            }
            for (int w = want_start[i]; w < want_start[i + 1]; ++w)
                if (want[w] < 0 || want[w] >= cnt) return fail(BAD_VALUE, "entry %d: wanted place %d is not among its %d tokens", i, want[w], cnt);
            t0 += cnt;
        }
        if (slots > (int)c->free_slots.size()) return fail(NO_SLOT, "the step brings %d new requests, %d of %d request slots are free", slots, (int)c->free_slots.size(), c->max_num_seqs);
        for (const Group& g : c->groups)
            if (g.pool.num_free() < pages) return fail(OUT_OF_PAGES, "Out of memory: No free blocks available.");
    }
    q_start[0] = 0;
    for (int i = 0; i < n; ++i) {
        const int cnt = counts[i];
        Request* r = c->find(rids[i]);
        if (!r) {
            if (int rc = c->add(rids[i], nullptr)) return rc;
            r = c->find(rids[i]);
        }
        const int start = r->length;
        if (int rc = c->reserve(rids[i], *r, start + cnt)) return rc;
        for (int k = 0; k < cnt; ++k) {
            token_ids[T + k] = tokens[T + k];
            positions[T + k] = start + k;
            seq_of_token[T + k] = i;
        }
        for (int w = want_start[i]; w < want_start[i + 1]; ++w) logit_rows[R++] = T + want[w];
        T += cnt;
        q_start[i + 1] = T;
        ctx_len[i] = start + cnt;
        state_slot[i] = r->slot;
        longest = std::max(longest, start + cnt);
    }
    *tokens_out = T;
    *rows_out = R;
    *max_ctx = longest;
    return OK;
}

// ---- the scheduler's decisions of one step ---------------------------------------------------
// Continuous batching above the step function.  The caller keeps the request records and the
// two queues; this function sees the running requests in the order of admission
// (run_ids, run_len = all tokens so far, run_done = tokens already run) and the waiting ones in
// queue order, and decides the portions of the next step:
//   1. each running request that is decoding (one token left) gets its token, oldest first; if its
//      next position needs a page and none is free, the request admitted last is preempted (what it
//      holds is given back, the caller puts it at the front of the waiting queue and recomputes it
//      from its tokens so far) until a page is free; a request is never preempted in favour of a
//      request admitted after it;
//   2. running requests still in their prompt get a portion of min(rest, chunk, budget left, what the
//      free pages hold); chunk <= 0 means no cap of its own on a portion;
//   3. waiting requests are admitted first come first served while a slot is free, fewer than
//      max_num_seqs requests are live, budget is left and pages for the first portion are free; the
//      first that does not fit stops admission (as in the reference, scheduler.cpp:20-43);
//   and when live requests exist but none can run (prompts in progress hold every page), the request
//   admitted last is preempted and the step is decided again.  A request is preempted only in favour
//   of an older one: when the ONLY running request cannot go on, no preemption would ever give it the
//   page it needs (it holds all there is to hold), so it is reported as stuck instead and the caller
//   ends it; recomputing it would come to the same place for ever.
// The reference has no budget, no portions and no preemption (scheduler.cpp:59-87).
// Out: portions (request, start, count, samples) in the order they are to be run, the preempted
// requests in the order of preemption, and how many waiting requests were admitted (they are the
// first of the queue as the caller knows it, after the preempted ones have been put at its front in
// order, each at the very front).  Pages of the portions are reserved; admitted requests hold slots.
// *stuck is the lone running request that can never go on, or -1; nothing else has been decided then,
// and the caller calls again after ending it.
int spy_sched_step(void* h, int budget, int chunk, int max_num_seqs, int n_run, const int64_t* run_ids, const int32_t* run_len, const int32_t* run_done, int n_wait,
                   const int64_t* wait_ids, const int32_t* wait_len, int64_t* out_ids, int32_t* out_start, int32_t* out_count, int32_t* out_samples,
                   int* n_out, int64_t* preempted, int* n_preempted, int* n_admitted, int64_t* stuck)
{
    Cache* c = static_cast<Cache*>(h);
    struct Seq {
        int64_t id;
        int len, done;
    };
    std::vector<Seq> running, waiting;
    for (int i = 0; i < n_run; ++i) running.push_back({run_ids[i], run_len[i], run_done[i]});
    for (int i = 0; i < n_wait; ++i) waiting.push_back({wait_ids[i], wait_len[i], 0});
    struct Portion {
        int64_t id;
        int start, count, samples;
    };
    std::vector<Portion> out;
    int np = 0, admitted = 0;
    *stuck = -1;
    const int initial_budget = budget;
    if (chunk <= 0) chunk = budget;   // no cap of its own on a portion
    auto preempt_last = [&]() -> int {
        Seq victim = running.back();
        running.pop_back();
        if (int rc = c->release_request(victim.id)) return rc;
        out.erase(std::remove_if(out.begin(), out.end(), [&](const Portion& p) { return p.id == victim.id; }), out.end());
        victim.done = 0;
        waiting.insert(waiting.begin(), victim);
        preempted[np++] = victim.id;
        return OK;
    };
    for (;;) {
        budget = initial_budget;
        out.clear();
        // 1. decoding requests, oldest first
        for (size_t i = 0; i < running.size(); ++i) {
            Seq& s = running[i];
            if (s.len - s.done != 1 || budget <= 0) continue;
            Request* r = c->find(s.id);
            if (!r) return fail(UNKNOWN_REQUEST, "running request %lld holds nothing in the cache", (long long)s.id);
            while (!c->can_reserve(*r, s.len) && running.size() - 1 > i) {
                if (int rc = preempt_last()) return rc;
            }
            if (!c->can_reserve(*r, s.len)) continue;   // it is the newest itself: it waits (or is preempted below)
            if (int rc = c->reserve(s.id, *r, s.len)) return rc;
            out.push_back({s.id, s.done, 1, 1});
            budget -= 1;
        }
        // 2. prompts of running requests, in portions
        for (Seq& s : running) {
            const int rest = s.len - s.done;
            if (rest <= 1 || budget <= 0) continue;
            Request* r = c->find(s.id);
            if (!r) return fail(UNKNOWN_REQUEST, "running request %lld holds nothing in the cache", (long long)s.id);
            const int fit = (c->pages_for(s.done) + c->min_free_pages()) * c->page_size - s.done;
            const int n = std::min(std::min(rest, chunk), std::min(budget, fit));
            if (n <= 0) continue;
            if (int rc = c->reserve(s.id, *r, s.done + n)) return rc;
            out.push_back({s.id, s.done, n, s.done + n == s.len ? 1 : 0});
            budget -= n;
        }
        // 3. admission, first come first served
        while (!waiting.empty() && budget > 0 && (int)running.size() < max_num_seqs && !c->free_slots.empty()) {
            Seq s = waiting.front();
            int n = std::min(std::min(s.len - s.done, chunk), budget);
            if (c->pages_for(n) > c->min_free_pages()) {
                const int fit = c->min_free_pages() * c->page_size;
                if (!running.empty() || fit <= 0) break;   // wait for running requests to finish and free pages
                n = std::min(n, fit);                      // nothing else is running: start with what fits
            }
            waiting.erase(waiting.begin());
            if (int rc = c->add(s.id, nullptr)) return rc;
            if (int rc = c->reserve(s.id, *c->find(s.id), n)) return rc;
            running.push_back(s);
            out.push_back({s.id, 0, n, n == s.len ? 1 : 0});
            budget -= n;
            ++admitted;
        }
        if (!out.empty() || running.empty()) break;
        if (running.size() == 1) {   // nobody is left whose pages could help it
            *stuck = running[0].id;
            break;
        }
        // live requests, yet none can run: the request admitted last gives its pages back and is recomputed later.
        // A request admitted in this very round cannot be the one (it would have got a portion).
        if (int rc = preempt_last()) return rc;
    }
    for (size_t i = 0; i < out.size(); ++i) {
        out_ids[i] = out[i].id;
        out_start[i] = out[i].start;
        out_count[i] = out[i].count;
        out_samples[i] = out[i].samples;
    }
    *n_out = (int)out.size();
    *n_preempted = np;
    *n_admitted = admitted;
    return OK;
}

}  // extern "C"
