// Host-side bookkeeping of the paged cache in C++: page pools, block tables, state slots and the optional prefix cache,
// with the policy of cache/manager.py (which states it and remains the plain twin that the tests compare this with).
// No device memory is touched here.  After the reference's BlockManager (engine/block_manager.cpp): pages are handed out
// least-recently-freed first (:35-69), a request's pages are given back last-logical-page first (:145-153), a page that is
// given back keeps what it was registered as until it is taken for other contents (:52-69), and the prefix cache chains
// the keys of full pages (:10-24, 71-143).
//
// What differs from the Python twin is the shape of the data, chosen for the step function that reads it every step:
// the block tables of all live requests of a group are ONE dense int32 array [state slot][table width], -1 where nothing
// is held, so a step copies whole rows to its staging buffer instead of converting lists; a request is known by its state
// slot (the Python wrapper maps request ids to slots).  Every entry point is plain C (called through ctypes) and returns
// a status; nothing throws across the boundary.
#include "runtime.hpp"

using namespace cvb_rt;

namespace {

inline Manager* M(void* h) { return static_cast<Manager*>(h); }

}  // namespace

extern "C" {

void* cvb_cm_create(int num_groups, const int* num_pages, const int* windows, int page_size, int num_slots, int width,
                    int prefix_caching) {
    if (num_groups <= 0 || page_size <= 0 || num_slots <= 0 || width <= 0) return nullptr;
    if (prefix_caching && !(num_groups == 1 && windows[0] <= 0)) return nullptr;
    for (int g = 0; g < num_groups; ++g)
        if (num_pages[g] <= 0) return nullptr;
    Manager* m = new Manager();
    m->page_size = page_size; m->width = width; m->num_slots = num_slots; m->num_groups = num_groups;
    m->prefix_caching = prefix_caching != 0;
    m->window.assign(windows, windows + num_groups);
    m->pools.resize(num_groups);
    m->tables.resize(num_groups); m->table_len.resize(num_groups); m->first_held.resize(num_groups);
    for (int g = 0; g < num_groups; ++g) {
        m->pools[g].init(num_pages[g], page_size, m->prefix_caching);
        m->tables[g].assign(static_cast<size_t>(num_slots) * width, -1);
        m->table_len[g].assign(num_slots, 0);
        m->first_held[g].assign(num_slots, 0);
    }
    m->held.assign(num_slots, 0); m->computed.assign(num_slots, 0); m->registered.assign(num_slots, 0);
    for (int s = 0; s < num_slots; ++s) m->free_slots.push(s);
    return m;
}

void cvb_cm_destroy(void* h) { delete M(h); }

// Arrays that the wrapper reads in place (they never move): a group's dense block tables and their lengths, and the
// per-slot counters.
int* cvb_cm_tables(void* h, int g) { return M(h)->tables[g].data(); }
int* cvb_cm_table_len(void* h, int g) { return M(h)->table_len[g].data(); }
int* cvb_cm_computed(void* h) { return M(h)->computed.data(); }
int* cvb_cm_registered(void* h) { return M(h)->registered.data(); }
int cvb_cm_num_free(void* h, int g) { return M(h)->pools[g].free_count; }
int cvb_cm_num_free_slots(void* h) { return static_cast<int>(M(h)->free_slots.size()); }
int cvb_cm_refs(void* h, int g, int page) {
    Manager* m = M(h);
    return page >= 0 && page < m->pools[g].n ? m->pools[g].refs[page] : -1;
}
long long cvb_cm_prefix_hits(void* h) { return M(h)->prefix_hits; }

// Whether a request with these tokens could be admitted and covered up to `upto_len` now.  Registered pages that somebody
// holds cost nothing; registered pages on the free list are counted as taken from it.
int cvb_cm_can_admit(void* h, const int* tokens, int n_tokens, int upto_len) {
    Manager* m = M(h);
    if (m->free_slots.empty()) return 0;
    std::vector<int> pages;
    m->prefix_pages(tokens, n_tokens, &pages);
    int shared = 0;
    for (int p : pages) shared += m->pools[0].refs[p] > 0 ? 1 : 0;
    const int need = m->pages_for(upto_len);
    for (int g = 0; g < m->num_groups; ++g)
        if ((g == 0 ? need - shared : need) > m->pools[g].free_count) return 0;
    return 1;
}

// A new request: returns its state slot.  With the prefix cache and the request's tokens, the pages of its longest
// registered prefix are shared with it and count as computed.
int cvb_cm_admit(void* h, const int* tokens, int n_tokens) {
    Manager* m = M(h);
    if (m->free_slots.empty()) return kErrNoSlot;
    std::vector<int> pages;
    m->prefix_pages(tokens, n_tokens, &pages);
    if (static_cast<int>(pages.size()) > m->width) return kErrWidth;
    const int slot = m->free_slots.top();
    m->free_slots.pop();
    m->held[slot] = 1;
    for (int g = 0; g < m->num_groups; ++g) { m->table_len[g][slot] = 0; m->first_held[g][slot] = 0; }
    int* tab = m->row(0, slot);
    for (size_t i = 0; i < pages.size(); ++i) {
        m->pools[0].share(pages[i]);
        tab[i] = pages[i];
    }
    m->table_len[0][slot] = static_cast<int>(pages.size());
    m->registered[slot] = m->prefix_caching ? static_cast<int>(pages.size()) : 0;
    m->computed[slot] = m->registered[slot] * m->page_size;
    m->prefix_hits += m->registered[slot];
    m->fresh.push_back(slot);
    return slot;
}

// Register the request's full pages whose keys are in the cache and whose tokens are all known.
int cvb_cm_commit(void* h, int slot, const int* tokens, int n_tokens) {
    Manager* m = M(h);
    if (!m->prefix_caching) return kOk;
    if (!m->live(slot)) return kErrMisuse;
    Pool& pool = m->pools[0];
    const int* tab = m->row(0, slot);
    const int upto = m->computed[slot] < n_tokens ? m->computed[slot] : n_tokens;
    const int full = upto / m->page_size;
    int i = m->registered[slot];
    while (i < full) {
        const int* chunk = tokens + static_cast<size_t>(i) * m->page_size;
        bool known = true;
        for (int k = 0; k < m->page_size; ++k) known = known && chunk[k] >= 0;
        if (!known) break;                                 // a token that is not known on the host yet
        const bool has_prefix = i > 0 && pool.has_key[tab[i - 1]];
        pool.register_page(tab[i], has_prefix, has_prefix ? pool.key[tab[i - 1]] : 0, chunk);
        ++i;
    }
    m->registered[slot] = i;
    return kOk;
}

int cvb_cm_take_fresh_slots(void* h, int* out, int max_out) {
    Manager* m = M(h);
    int n = 0;
    for (int s : m->fresh)
        if (n < max_out) out[n++] = s;
    m->fresh.clear();
    return n;
}

int cvb_cm_pages_missing(void* h, int slot, int upto_len, int* out) {
    Manager* m = M(h);
    if (!m->live(slot)) return kErrMisuse;
    for (int g = 0; g < m->num_groups; ++g) out[g] = m->missing(g, slot, upto_len);
    return kOk;
}

int cvb_cm_covered(void* h, int slot, int upto_len) {
    Manager* m = M(h);
    if (!m->live(slot)) return kErrMisuse;
    const int need = m->pages_for(upto_len);
    for (int g = 0; g < m->num_groups; ++g)
        if (m->table_len[g][slot] < need) return 0;
    return 1;
}

int cvb_cm_can_reserve(void* h, int slot, int upto_len) {
    Manager* m = M(h);
    if (!m->live(slot)) return kErrMisuse;
    for (int g = 0; g < m->num_groups; ++g)
        if (m->missing(g, slot, upto_len) > m->pools[g].free_count) return 0;
    return 1;
}

// Cover positions below `upto_len` with pages, in every group; all or nothing.  Returns how many tokens the request's
// tables cover now, or an error.
int cvb_cm_reserve(void* h, int slot, int upto_len) {
    Manager* m = M(h);
    if (!m->live(slot)) return kErrMisuse;
    const int target = m->pages_for(upto_len);
    for (int g = 0; g < m->num_groups; ++g)
        if (m->missing(g, slot, upto_len) > m->pools[g].free_count) return kErrOutOfPages;
    if (target > m->width) return kErrWidth;
    int covered = 0x7fffffff;
    for (int g = 0; g < m->num_groups; ++g) {
        int* tab = m->row(g, slot);
        int& len = m->table_len[g][slot];
        const int first = m->first_needed(g, m->computed[slot]);
        while (len < target) {
            tab[len] = len >= first ? m->pools[g].take() : -1;
            ++len;
        }
        if (len < covered) covered = len;
    }
    return covered * m->page_size;
}

// The request's first `computed` tokens are in the cache; windowed groups give back the pages that no later token can
// read.
int cvb_cm_advance(void* h, int slot, int computed) {
    Manager* m = M(h);
    if (!m->live(slot) || computed < m->computed[slot]) return kErrMisuse;
    m->computed[slot] = computed;
    for (int g = 0; g < m->num_groups; ++g) {
        if (m->window[g] <= 0) continue;
        int* tab = m->row(g, slot);
        const int len = m->table_len[g][slot];
        int upto = m->first_needed(g, computed);
        if (upto > len) upto = len;
        for (int i = m->first_held[g][slot]; i < upto; ++i)
            if (tab[i] >= 0) {
                m->pools[g].give_back(tab[i]);
                tab[i] = -1;
            }
        if (upto > m->first_held[g][slot]) m->first_held[g][slot] = upto;
    }
    return kOk;
}

// advance() for several requests in one call; returns the index of the first request that was refused, or -1.
int cvb_cm_advance_many(void* h, const int* slots, const int* computed, int n) {
    for (int i = 0; i < n; ++i)
        if (cvb_cm_advance(h, slots[i], computed[i]) != kOk) return i;
    return -1;
}

int cvb_cm_release(void* h, int slot) {
    Manager* m = M(h);
    if (!m->live(slot)) return kErrMisuse;
    for (int g = 0; g < m->num_groups; ++g) {
        int* tab = m->row(g, slot);
        for (int i = m->table_len[g][slot] - 1; i >= 0; --i) {   // last logical page first: prefix pages survive longest
            if (tab[i] >= 0) m->pools[g].give_back(tab[i]);
            tab[i] = -1;
        }
        m->table_len[g][slot] = 0;
        m->first_held[g][slot] = 0;
    }
    m->held[slot] = 0;
    m->computed[slot] = 0;
    m->registered[slot] = 0;
    m->free_slots.push(slot);
    for (size_t i = 0; i < m->fresh.size(); ++i)
        if (m->fresh[i] == slot) { m->fresh.erase(m->fresh.begin() + i); break; }
    return kOk;
}

// Every page is either free exactly once or held, by as many requests as its reference count says and by each at most
// once (more than one holder only with the prefix cache); no state slot is lost.  0 if so; else the message tells.
int cvb_cm_check(void* h) {
    Manager* m = M(h);
    m->message.clear();
    auto fail = [&](const std::string& s) { m->message = s; return -1; };
    for (int g = 0; g < m->num_groups; ++g) {
        Pool& pool = m->pools[g];
        std::vector<int> on_list(pool.n, 0), holders(pool.n, 0);
        int count = 0, last = -1;
        for (int p = pool.head; p >= 0; p = pool.next[p]) {
            if (++count > pool.n) return fail("group " + std::to_string(g) + ": the free list has a cycle");
            if (on_list[p]++) return fail("group " + std::to_string(g) + ": a page is in the free list twice");
            if (pool.prev[p] != last) return fail("group " + std::to_string(g) + ": the free list's links disagree");
            last = p;
        }
        if (count != pool.free_count || last != pool.tail) return fail("group " + std::to_string(g) + ": the free list's count or tail is off");
        for (int s = 0; s < m->num_slots; ++s) {
            const int* tab = m->row(g, s);
            if (!m->held[s]) {
                for (int i = 0; i < m->width; ++i)
                    if (tab[i] != -1) return fail("a slot that nobody holds has a page in its table");
                continue;
            }
            std::vector<int> mine;
            for (int i = 0; i < m->width; ++i) {
                if (i >= m->table_len[g][s] && tab[i] != -1) return fail("a table has a page beyond its length");
                if (tab[i] >= 0) {
                    for (int q : mine)
                        if (q == tab[i]) return fail("group " + std::to_string(g) + ": a request holds a page twice");
                    mine.push_back(tab[i]);
                    ++holders[tab[i]];
                }
            }
        }
        for (int p = 0; p < pool.n; ++p) {
            if (holders[p] != pool.refs[p])
                return fail("group " + std::to_string(g) + ": page " + std::to_string(p) + " is held by " + std::to_string(holders[p]) +
                            " requests but counts " + std::to_string(pool.refs[p]));
            if ((holders[p] == 0) != (on_list[p] == 1))
                return fail("group " + std::to_string(g) + ": page " + std::to_string(p) + " is free and held, or neither");
            if (holders[p] > 1 && !m->prefix_caching) return fail("group " + std::to_string(g) + ": a page is held by several requests");
        }
        for (auto& kv : pool.by_key)
            if (!pool.has_key[kv.second] || pool.key[kv.second] != kv.first)
                return fail("group " + std::to_string(g) + ": key of a page and the key table disagree");
    }
    int held = 0;
    for (int s = 0; s < m->num_slots; ++s) held += m->held[s] ? 1 : 0;
    if (held + static_cast<int>(m->free_slots.size()) != m->num_slots) return fail("a state slot is lost");
    return 0;
}

const char* cvb_cm_message(void* h) { return M(h)->message.c_str(); }

}  // extern "C"
