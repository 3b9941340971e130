// The cache manager's bookkeeping on the host: pools of pages by layer group, each sequence's
// logical pages per group, state slots, and the arrays that describe one step to the kernels.
//
// Kapel keeps this in Rust (`KvCache`, crates/kapel-models/src/cache.rs:57-72,137-168,419-433,
// 481-486,751-818): one page list a sequence, a LIFO free list, `plan_counts` that takes pages and
// builds positions / lines / rows / slots. Here the same arithmetic runs per group of layers with the
// same needs, and a group with a window gives back the pages no later query can read. Plain C
// functions over an opaque handle, called through ctypes; no GPU code, so every decision is tested
// without one. The Python class `CacheManager` owns the handle and the device tables.
//
// Orders matter and are part of the contract (a replay of the same requests takes the same pages):
// a fresh pool hands out page 0 first; the page given back last is taken first; a sequence that ends
// gives its pages back last page first, group by group; slot 1 is handed out first and the slot
// freed last is taken first.
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

namespace {

struct Pool {
    int n = 0;
    std::vector<int> free_;            // taken from the back
    std::vector<uint8_t> held;

    explicit Pool(int pages) : n(pages), held((size_t)pages, 0) {
        free_.reserve((size_t)pages);
        for (int p = pages - 1; p >= 0; --p) free_.push_back(p);
    }
    int take() {                       // page, -1 none free, -2 a free page was marked held
        if (free_.empty()) return -1;
        const int p = free_.back();
        if (held[(size_t)p]) return -2;
        free_.pop_back();
        held[(size_t)p] = 1;
        return p;
    }
    int give(int p) {                  // 0, -1 not of this pool, -2 given back twice
        if (p < 0 || p >= n) return -1;
        if (!held[(size_t)p]) return -2;
        held[(size_t)p] = 0;
        free_.push_back(p);
        return 0;
    }
    int check(std::string* why) const {
        std::vector<uint8_t> on_list((size_t)n, 0);
        for (int p : free_) {
            if (p < 0 || p >= n) { *why = "a page outside the pool is on the free list"; return 1; }
            if (on_list[(size_t)p]) { *why = "a page is on the free list twice"; return 1; }
            on_list[(size_t)p] = 1;
        }
        for (int p = 0; p < n; ++p)
            if ((held[(size_t)p] != 0) == (on_list[(size_t)p] != 0)) {
                *why = "page " + std::to_string(p) + ": held and on the free list disagree";
                return 1;
            }
        return 0;
    }
};

struct Seq {
    bool live = false;
    bool fresh = true;
    int length = 0;
    std::vector<std::vector<int>> pages;   // [group][logical page] -> physical page, -1 where given back
    std::vector<int> released;             // [group] logical pages below this index were given back
};

struct Cache {
    int page_size = 16;
    int max_sequences = 0;
    std::vector<Pool> pools;
    std::vector<int> windows;              // -1: the group keeps every key
    std::vector<Seq> seqs;                 // by slot; slot 0 belongs to padding rows
    std::vector<int> free_slots;           // taken from the back
    long long released_pages = 0;

    int groups() const { return (int)pools.size(); }
    int pages_for(long long length) const { return (int)((length + page_size - 1) / page_size); }
    Seq* live(int slot) {
        if (slot < 1 || slot > max_sequences || !seqs[(size_t)slot].live) return nullptr;
        return &seqs[(size_t)slot];
    }
};

Cache* as_cache(void* h) { return static_cast<Cache*>(h); }

}  // namespace

extern "C" {

// ---------------------------------------------------------------------------------- a pool alone
void* kp_create(int pages) { return pages < 0 ? nullptr : new Pool(pages); }
void kp_destroy(void* h) { delete static_cast<Pool*>(h); }
int kp_take(void* h) { return static_cast<Pool*>(h)->take(); }
int kp_give(void* h, int page) { return static_cast<Pool*>(h)->give(page); }
int kp_free(void* h) { return (int)static_cast<Pool*>(h)->free_.size(); }
int kp_is_held(void* h, int page) {
    Pool* p = static_cast<Pool*>(h);
    return page >= 0 && page < p->n && p->held[(size_t)page] ? 1 : 0;
}
int kp_check(void* h, char* msg, int cap) {
    std::string why;
    const int r = static_cast<Pool*>(h)->check(&why);
    if (r && msg && cap > 0) std::snprintf(msg, (size_t)cap, "%s", why.c_str());
    return r;
}

// ---------------------------------------------------------------------------------- the manager
void* kc_create(int n_groups, int page_size, const int* pages, const int* windows, int max_sequences) {
    if (n_groups < 0 || page_size <= 0 || max_sequences < 0) return nullptr;
    for (int g = 0; g < n_groups; ++g)
        if (pages[g] < 0) return nullptr;
    Cache* c = new Cache();
    c->page_size = page_size;
    c->max_sequences = max_sequences;
    for (int g = 0; g < n_groups; ++g) {
        c->pools.emplace_back(pages[g]);
        c->windows.push_back(windows[g]);
    }
    c->seqs.resize((size_t)max_sequences + 1);
    for (int s = max_sequences; s >= 1; --s) c->free_slots.push_back(s);
    return c;
}

void kc_destroy(void* h) { delete as_cache(h); }

// A slot for a new sequence (1 ..), or -1 when none is free.
int kc_add(void* h) {
    Cache* c = as_cache(h);
    if (c->free_slots.empty()) return -1;
    const int slot = c->free_slots.back();
    c->free_slots.pop_back();
    Seq& s = c->seqs[(size_t)slot];
    s = Seq();
    s.live = true;
    s.pages.assign((size_t)c->groups(), std::vector<int>());
    s.released.assign((size_t)c->groups(), 0);
    return slot;
}

// Everything the sequence holds goes back, last page first, group by group. -1: no such sequence;
// -2: a page could not be given back (the bookkeeping is broken).
int kc_remove(void* h, int slot) {
    Cache* c = as_cache(h);
    Seq* s = c->live(slot);
    if (!s) return -1;
    int bad = 0;
    for (int g = 0; g < c->groups(); ++g) {
        const std::vector<int>& pages = s->pages[(size_t)g];
        for (size_t i = pages.size(); i-- > 0;)
            if (pages[i] >= 0 && c->pools[(size_t)g].give(pages[i]) != 0) bad = 1;
    }
    *s = Seq();
    c->free_slots.push_back(slot);
    return bad ? -2 : 0;
}

int kc_length(void* h, int slot) {
    Seq* s = as_cache(h)->live(slot);
    return s ? s->length : -1;
}

int kc_free_slots(void* h) { return (int)as_cache(h)->free_slots.size(); }
long long kc_released_pages(void* h) { return as_cache(h)->released_pages; }

void kc_free_pages(void* h, int* out) {
    Cache* c = as_cache(h);
    for (int g = 0; g < c->groups(); ++g) out[g] = (int)c->pools[(size_t)g].free_.size();
}

int kc_held_pages(void* h, int slot, int* out) {
    Cache* c = as_cache(h);
    Seq* s = c->live(slot);
    if (!s) return -1;
    for (int g = 0; g < c->groups(); ++g) {
        int n = 0;
        for (int p : s->pages[(size_t)g]) n += p >= 0 ? 1 : 0;
        out[g] = n;
    }
    return 0;
}

// A sequence's logical pages in one group (-1 where given back): how many there are; up to `cap`
// of them are copied out.
int kc_pages_of(void* h, int slot, int group, int* out, int cap) {
    Cache* c = as_cache(h);
    Seq* s = c->live(slot);
    if (!s || group < 0 || group >= c->groups()) return -1;
    const std::vector<int>& pages = s->pages[(size_t)group];
    for (int i = 0; i < (int)pages.size() && i < cap; ++i) out[i] = pages[(size_t)i];
    return (int)pages.size();
}

// New pages each group must take for `count` more tokens of the sequence in `slot` (slot 0: a
// sequence not yet in the cache, which counts from zero): ceil((length + count) / page) minus the
// logical pages it has (held or passed).
int kc_pages_needed(void* h, int slot, int count, int* out) {
    Cache* c = as_cache(h);
    Seq* s = slot == 0 ? nullptr : c->live(slot);
    if (slot != 0 && !s) return -1;
    const long long length = s ? s->length : 0;
    for (int g = 0; g < c->groups(); ++g)
        out[g] = c->pages_for(length + count) - (s ? (int)s->pages[(size_t)g].size() : 0);
    return 0;
}

// What a step of `n` entries (slot, count) needs. info: [0] 0 fits / 1 a group lacks pages /
// 2 an entry is wrong, [1] rows, [2] the widest block-table row, [3] pages the step takes in all,
// and when a group lacks pages [4] the group, [5] pages needed, [6] pages free.
int kc_plan_prepare(void* h, int n, const int* slots, const int* counts, long long* info) {
    Cache* c = as_cache(h);
    std::vector<long long> need((size_t)c->groups(), 0);
    long long rows = 0, widest = 0, total = 0;
    std::memset(info, 0, 7 * sizeof(long long));
    std::vector<uint8_t> seen((size_t)c->max_sequences + 1, 0);
    for (int e = 0; e < n; ++e) {
        Seq* s = c->live(slots[e]);
        if (!s || counts[e] <= 0 || seen[(size_t)slots[e]]) { info[0] = 2; return 2; }
        seen[(size_t)slots[e]] = 1;
        rows += counts[e];
        const int want = c->pages_for((long long)s->length + counts[e]);
        widest = std::max<long long>(widest, want);
        for (int g = 0; g < c->groups(); ++g) {
            const long long more = want - (long long)s->pages[(size_t)g].size();
            need[(size_t)g] += more;
            total += std::max<long long>(0, more);
        }
    }
    info[1] = rows; info[2] = widest; info[3] = total;
    for (int g = 0; g < c->groups(); ++g)
        if (need[(size_t)g] > (long long)c->pools[(size_t)g].free_.size()) {
            info[0] = 1; info[4] = g; info[5] = need[(size_t)g]; info[6] = (long long)c->pools[(size_t)g].free_.size();
            return 1;
        }
    return 0;
}

// Takes the step's pages and writes its arrays (after a `kc_plan_prepare` that returned 0, with
// nothing in between). Rows: positions, row_entry, row_count [rows]; entries: q_start, q_len,
// kv_len, slot_out [n], fresh [n] bytes; per group lines[g] [rows] and tables[g] [n, width], which
// the caller has filled with -1. `taken` receives (group, slot, logical page, physical page) for
// every page taken, in order; returns how many, or -1 if a pool ran dry or `taken_cap` was too small
// (then what was taken has been given back).
int kc_plan_fill(void* h, int n, const int* slots, const int* counts, int* positions, int* row_entry, int* row_count,
                 int* q_start, int* q_len, int* kv_len, int* slot_out, uint8_t* fresh, int* const* lines, int* const* tables,
                 int width, int* taken, int taken_cap) {
    Cache* c = as_cache(h);
    const int ps = c->page_size;
    int n_taken = 0;
    long long r = 0;
    bool failed = false;
    for (int e = 0; e < n && !failed; ++e) {
        Seq* s = c->live(slots[e]);
        if (!s) { failed = true; break; }
        const int start = s->length, count = counts[e], end = start + count;
        q_start[e] = (int)r; q_len[e] = count; kv_len[e] = end;
        slot_out[e] = slots[e]; fresh[e] = s->fresh ? 1 : 0;
        for (int i = 0; i < count; ++i) {
            positions[r + i] = start + i;
            row_entry[r + i] = e;
            row_count[r + i] = start + i + 1;
        }
        const int want = c->pages_for(end);
        for (int g = 0; g < c->groups() && !failed; ++g) {
            std::vector<int>& pages = s->pages[(size_t)g];
            while ((int)pages.size() < want) {
                const int page = n_taken < taken_cap ? c->pools[(size_t)g].take() : -1;
                if (page < 0) { failed = true; break; }
                int* t = taken + 4 * (size_t)n_taken++;
                t[0] = g; t[1] = slots[e]; t[2] = (int)pages.size(); t[3] = page;
                pages.push_back(page);
            }
            if (failed) break;
            if ((int)pages.size() > width) { failed = true; break; }
            int* row = tables[g] + (size_t)e * (size_t)width;
            std::copy(pages.begin(), pages.end(), row);
            int* ln = lines[g] + r;
            for (int i = 0; i < count; ++i) {
                const int pos = start + i;
                ln[i] = pages[(size_t)(pos / ps)] * ps + pos % ps;
            }
        }
        r += count;
    }
    if (failed) {
        for (int i = n_taken; i-- > 0;) {
            const int* t = taken + 4 * (size_t)i;
            Seq* s = c->live(t[1]);
            if (s && (int)s->pages[(size_t)t[0]].size() == t[2] + 1 && s->pages[(size_t)t[0]].back() == t[3]) {
                s->pages[(size_t)t[0]].pop_back();
                c->pools[(size_t)t[0]].give(t[3]);
            }
        }
        return -1;
    }
    return n_taken;
}

// The step's kernels are enqueued: lengths advance, and a group with a window gives back the pages
// that lie wholly below what the next query reads (it has seen at least length + 1 positions and
// reads from length + 1 - window on). Returns the pages given back, or -1 for a wrong entry.
long long kc_commit(void* h, int n, const int* slots, const int* counts) {
    Cache* c = as_cache(h);
    long long given = 0;
    for (int e = 0; e < n; ++e) {
        Seq* s = c->live(slots[e]);
        if (!s || counts[e] <= 0) return -1;
        s->length += counts[e];
        s->fresh = false;
        for (int g = 0; g < c->groups(); ++g) {
            const int window = c->windows[(size_t)g];
            if (window < 0) continue;
            const long long first_needed = (long long)s->length + 1 - window;
            if (first_needed <= 0) continue;
            std::vector<int>& pages = s->pages[(size_t)g];
            const int upto = (int)std::min<long long>(first_needed / c->page_size, (long long)pages.size());
            for (int p = s->released[(size_t)g]; p < upto; ++p)
                if (pages[(size_t)p] >= 0) {
                    c->pools[(size_t)g].give(pages[(size_t)p]);
                    pages[(size_t)p] = -1;
                    ++given;
                }
            s->released[(size_t)g] = std::max(s->released[(size_t)g], upto);
        }
    }
    c->released_pages += given;
    return given;
}

// The step did not run: the pages it took go back, newest first. A page goes back only if it is
// still the last logical page of its sequence.
int kc_abort(void* h, int n_taken, const int* taken) {
    Cache* c = as_cache(h);
    int given = 0;
    for (int i = n_taken; i-- > 0;) {
        const int* t = taken + 4 * (size_t)i;
        if (t[0] < 0 || t[0] >= c->groups()) continue;
        Seq* s = c->live(t[1]);
        if (!s) continue;
        std::vector<int>& pages = s->pages[(size_t)t[0]];
        if ((int)pages.size() == t[2] + 1 && pages.back() == t[3]) {
            pages.pop_back();
            c->pools[(size_t)t[0]].give(t[3]);
            ++given;
        }
    }
    return given;
}

// No page lost, none held twice, no slot lost: 0, or 1 with the reason in `msg`.
int kc_check(void* h, char* msg, int cap) {
    Cache* c = as_cache(h);
    std::string why;
    auto fail = [&](const std::string& s) {
        if (msg && cap > 0) std::snprintf(msg, (size_t)cap, "%s", s.c_str());
        return 1;
    };
    for (int g = 0; g < c->groups(); ++g) {
        const Pool& pool = c->pools[(size_t)g];
        if (pool.check(&why)) return fail("group " + std::to_string(g) + ": " + why);
        std::vector<int> owner((size_t)pool.n, 0);
        long long owned = 0;
        for (int slot = 1; slot <= c->max_sequences; ++slot) {
            const Seq& s = c->seqs[(size_t)slot];
            if (!s.live) continue;
            for (int p : s.pages[(size_t)g]) {
                if (p < 0) continue;
                if (p >= pool.n) return fail("group " + std::to_string(g) + ": page " + std::to_string(p) + " is not of the pool");
                if (owner[(size_t)p]) return fail("group " + std::to_string(g) + ": page " + std::to_string(p) + " held by slots " +
                                                  std::to_string(owner[(size_t)p]) + " and " + std::to_string(slot));
                if (!pool.held[(size_t)p]) return fail("group " + std::to_string(g) + ": page " + std::to_string(p) + " of slot " +
                                                       std::to_string(slot) + " is on the free list");
                owner[(size_t)p] = slot;
                ++owned;
            }
        }
        const long long held = (long long)pool.n - (long long)pool.free_.size();
        if (owned != held) return fail("group " + std::to_string(g) + ": " + std::to_string(held) + " pages held, " +
                                       std::to_string(owned) + " owned: pages lost");
    }
    std::vector<uint8_t> free_slot((size_t)c->max_sequences + 1, 0);
    for (int s : c->free_slots) {
        if (s < 1 || s > c->max_sequences || free_slot[(size_t)s]) return fail("a slot is free twice or is not a slot");
        free_slot[(size_t)s] = 1;
    }
    int live = 0;
    for (int slot = 1; slot <= c->max_sequences; ++slot) {
        if (c->seqs[(size_t)slot].live) {
            if (free_slot[(size_t)slot]) return fail("slot " + std::to_string(slot) + " is free while held");
            ++live;
        }
    }
    if (live + (int)c->free_slots.size() != c->max_sequences) return fail("a slot was lost");
    return 0;
}

}  // extern "C"
