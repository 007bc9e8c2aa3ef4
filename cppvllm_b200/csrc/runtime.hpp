// The cache manager's data and policy (shared by cache_runtime.cpp, which exports it, and scheduler_runtime.cpp, whose
// scheduler calls it directly).  See cache_runtime.cpp for what it is after.
#pragma once
#include <cstdint>
#include <cstring>
#include <queue>
#include <string>
#include <unordered_map>
#include <vector>

namespace cvb_rt {

constexpr int kOk = 0;
constexpr int kErrMisuse = -1;      // unknown or double admission, double free, shrinking length
constexpr int kErrOutOfPages = -2;  // a reservation needs more pages than a group has free
constexpr int kErrWidth = -3;       // a table would grow beyond the width of the dense array
constexpr int kErrNoSlot = -4;      // no free state slot

inline uint64_t mix64(uint64_t x) {  // splitmix64 finaliser
    x += 0x9e3779b97f4a7c15ULL;
    x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ULL;
    x = (x ^ (x >> 27)) * 0x94d049bb133111ebULL;
    return x ^ (x >> 31);
}

// Pages of one group.  The free list is a doubly linked list threaded through the page numbers (a registered page that
// lies on it can be taken out of its middle when a new request shares it).
struct Pool {
    int n = 0, page_size = 0;
    bool keyed = false;                       // prefix cache on: pages can be registered
    std::vector<int> refs, prev, next;
    std::vector<char> on_free;
    int head = -1, tail = -1, free_count = 0;
    std::vector<char> has_key;
    std::vector<uint64_t> key;
    std::vector<int> tokens;                  // [n][page_size], contents of registered pages
    std::unordered_map<uint64_t, int> by_key;

    void init(int num_pages, int ps, bool with_keys) {
        n = num_pages; page_size = ps; keyed = with_keys;
        refs.assign(n, 0); prev.assign(n, -1); next.assign(n, -1); on_free.assign(n, 0);
        has_key.assign(n, 0); key.assign(n, 0);
        if (keyed) tokens.assign(static_cast<size_t>(n) * ps, 0);
        head = tail = -1; free_count = 0;
        for (int p = 0; p < n; ++p) push_tail(p);
    }
    void push_tail(int p) {
        prev[p] = tail; next[p] = -1;
        if (tail >= 0) next[tail] = p; else head = p;
        tail = p; on_free[p] = 1; ++free_count;
    }
    void unlink(int p) {
        if (prev[p] >= 0) next[prev[p]] = next[p]; else head = next[p];
        if (next[p] >= 0) prev[next[p]] = prev[p]; else tail = prev[p];
        prev[p] = next[p] = -1; on_free[p] = 0; --free_count;
    }
    // a page for new contents: the least recently freed one; what it was registered as is forgotten
    int take() {
        if (head < 0) return -1;
        const int p = head;
        unlink(p);
        if (has_key[p]) {
            auto it = by_key.find(key[p]);
            if (it != by_key.end() && it->second == p) by_key.erase(it);
            has_key[p] = 0;
        }
        refs[p] = 1;
        return p;
    }
    bool give_back(int p) {
        if (p < 0 || p >= n || refs[p] <= 0) return false;
        if (--refs[p] == 0) push_tail(p);     // to the tail; it keeps its key until taken again
        return true;
    }
    void share(int p) {                       // one more holder of a registered page
        if (refs[p] == 0) unlink(p);
        ++refs[p];
    }
    uint64_t chain_key(bool has_prefix, uint64_t prefix, const int* toks) const {
        uint64_t h = mix64(has_prefix ? prefix ^ 0x5851f42d4c957f2dULL : 0x2545f4914f6cdd1dULL);
        for (int i = 0; i < page_size; ++i) h = mix64(h ^ static_cast<uint64_t>(static_cast<uint32_t>(toks[i])));
        return h;
    }
    // the page registered for these tokens after that prefix, or -1; the key either way
    int find(bool has_prefix, uint64_t prefix, const int* toks, uint64_t* key_out) const {
        const uint64_t k = chain_key(has_prefix, prefix, toks);
        *key_out = k;
        auto it = by_key.find(k);
        if (it == by_key.end()) return -1;
        const int p = it->second;
        if (std::memcmp(&tokens[static_cast<size_t>(p) * page_size], toks, sizeof(int) * page_size) != 0) return -1;
        return p;
    }
    // record what a held page contains; the first page registered under a key keeps it
    uint64_t register_page(int p, bool has_prefix, uint64_t prefix, const int* toks) {
        if (!has_key[p]) {
            const uint64_t k = chain_key(has_prefix, prefix, toks);
            key[p] = k; has_key[p] = 1;
            std::memcpy(&tokens[static_cast<size_t>(p) * page_size], toks, sizeof(int) * page_size);
            by_key.emplace(k, p);             // keeps an earlier page of the same key
        }
        return key[p];
    }
};

struct Manager {
    int page_size = 0, width = 0, num_slots = 0, num_groups = 0;
    bool prefix_caching = false;
    long long prefix_hits = 0;
    std::vector<int> window;
    std::vector<Pool> pools;
    std::vector<std::vector<int>> tables;     // per group [num_slots][width], -1 where nothing is held
    std::vector<std::vector<int>> table_len;  // per group [num_slots]
    std::vector<std::vector<int>> first_held; // per group [num_slots]: first logical page still held (windowed groups)
    std::vector<char> held;                   // per slot
    std::vector<int> computed, registered;    // per slot
    std::priority_queue<int, std::vector<int>, std::greater<int>> free_slots;   // lowest number first
    std::vector<int> fresh;
    std::string message;                      // of the last failed self-check

    int pages_for(int length) const { return (length + page_size - 1) / page_size; }
    int first_needed(int g, int comp) const {
        const int w = window[g];
        if (w <= 0) return 0;
        const int lo = comp - w + 1;           // the next token sits at `comp` and reads positions >= comp - w + 1
        return (lo > 0 ? lo : 0) / page_size;
    }
    int* row(int g, int slot) { return &tables[g][static_cast<size_t>(slot) * width]; }
    bool live(int slot) const { return slot >= 0 && slot < num_slots && held[slot]; }
    // pages to take in group g so that positions first_needed .. upto_len - 1 are covered
    int missing(int g, int slot, int upto_len) const {
        const int have = table_len[g][slot];
        const int fn = first_needed(g, computed[slot]);
        const int first = have > fn ? have : fn;
        const int need = pages_for(upto_len) - first;
        return need > 0 ? need : 0;
    }
    // [(page, key)] of the longest registered chain that matches the prefix of the tokens
    int prefix_pages(const int* toks, int n, std::vector<int>* pages) const {
        pages->clear();
        if (!prefix_caching || toks == nullptr) return 0;
        const Pool& pool = pools[0];
        bool has = false;
        uint64_t key = 0;
        for (int i = 0; i < (n - 1) / page_size; ++i) {     // at least one token is always computed
            const int* chunk = toks + static_cast<size_t>(i) * page_size;
            bool known = true;
            for (int k = 0; k < page_size; ++k) known = known && chunk[k] >= 0;
            if (!known) break;
            uint64_t k2;
            const int p = pool.find(has, key, chunk, &k2);
            if (p < 0) break;
            pages->push_back(p);
            has = true; key = k2;
        }
        return static_cast<int>(pages->size());
    }
};

inline int manager_computed(void* h, int slot) { return static_cast<Manager*>(h)->computed[slot]; }

}  // namespace cvb_rt

// The manager's entry points (cache_runtime.cpp); the scheduler calls them as any other user does.
extern "C" {
int cvb_cm_can_admit(void* h, const int* tokens, int n_tokens, int upto_len);
int cvb_cm_admit(void* h, const int* tokens, int n_tokens);
int cvb_cm_commit(void* h, int slot, const int* tokens, int n_tokens);
int cvb_cm_covered(void* h, int slot, int upto_len);
int cvb_cm_can_reserve(void* h, int slot, int upto_len);
int cvb_cm_reserve(void* h, int slot, int upto_len);
int cvb_cm_advance(void* h, int slot, int computed);
int cvb_cm_release(void* h, int slot);
}
