// Host side of the paged cache: page pools, block tables, state slots, and the
// per-step index arrays.  Plain C ABI, used from Python through ctypes.
//
// What it keeps from the reference: pages are handed out first-in first-out and
// freed pages go to the tail (mstar/engine/kv_store.py:25-67); a request's ordered
// page list is its block table (mstar/engine/cache_manager.py:272-317); pages are
// grown before the forward pass and the length advances only after it
// (cache_manager.py:278-285, 811-838); everything a request holds returns to the
// pool when it is removed (kv_store.py:606-614).
// What it adds: several groups of layers, each with a pool, a page size and an
// optional window of its own; a position counter per request that is kept apart from
// the number of cached tokens (the reference's position_id_start beside seq_len,
// kv_store.py:112-116, advanced on its own by set_custom_pos_advance,
// cache_manager.py:777-808); pages that a window has passed are given back while
// the request is still running; reservation of a whole batch is all-or-nothing
// (the reference leaves earlier requests of a failed batch extended,
// kv_store.py:463-482); a pool of fixed-size state slots, one per live request.
#include <cstdint>
#include <cstring>
#include <deque>
#include <mutex>
#include <unordered_map>
#include <vector>

#define MSTAR_API extern "C" __attribute__((visibility("default")))

namespace {

constexpr int kOk = 0;
constexpr int kNoSlot = -1;
constexpr int kDuplicate = -2;
constexpr int kUnknown = -3;
constexpr int kNoPages = -4;
constexpr int kBadArg = -5;
constexpr int kTooLong = -6;

struct Group {
    int page_size = 0;
    int num_pages = 0;
    int window = 0;  // 0: every key is kept
    std::deque<int> free_pages;
    std::vector<int64_t> owner;  // request id holding the page, or -1
};

struct Request {
    int slot = -1;
    int64_t len = 0;                       // committed tokens (keys in the cache)
    int64_t pos = 0;                       // position id of the next token
    std::vector<std::vector<int>> table;   // [group][logical page] -> page id or -1
};

struct Manager {
    std::vector<Group> groups;
    std::deque<int> free_slots;
    std::vector<int64_t> slot_owner;
    std::unordered_map<int64_t, Request> requests;
    int64_t max_positions = 0;  // 0: no limit; else no token gets a position id >= this
    std::mutex mu;
};

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// First logical page that a request of length `len` (about to append) still needs.
inline int64_t first_needed_page(const Group& g, int64_t len) {
    if (g.window <= 0) return 0;
    const int64_t first_key = len - g.window + 1;  // oldest key the next token sees
    return first_key <= 0 ? 0 : first_key / g.page_size;
}

// Pages that must be newly allocated in group gi so that the request can hold
// len + n_new tokens.
inline int64_t new_pages_needed(const Group& g, const Request& r, int gi, int64_t n_new) {
    const int64_t want = ceil_div(r.len + n_new, g.page_size);
    const int64_t have = (int64_t)r.table[gi].size();
    return want > have ? want - have : 0;
}

void release_passed(Manager& m, int64_t rid, Request& r) {
    for (size_t gi = 0; gi < m.groups.size(); ++gi) {
        Group& g = m.groups[gi];
        if (g.window <= 0) continue;
        const int64_t first = first_needed_page(g, r.len);
        auto& tab = r.table[gi];
        for (int64_t p = 0; p < first && p < (int64_t)tab.size(); ++p) {
            if (tab[p] >= 0) {
                g.owner[tab[p]] = -1;
                g.free_pages.push_back(tab[p]);
                tab[p] = -1;
            }
        }
    }
    (void)rid;
}

}  // namespace

MSTAR_API void* cm_create(int n_groups, const int* page_sizes, const int* num_pages,
                          const int* windows, int num_slots) {
    if (n_groups < 0 || num_slots < 0) return nullptr;
    auto* m = new Manager();
    m->groups.resize(n_groups);
    for (int i = 0; i < n_groups; ++i) {
        if (page_sizes[i] <= 0 || num_pages[i] < 0 || windows[i] < 0) {
            delete m;
            return nullptr;
        }
        Group& g = m->groups[i];
        g.page_size = page_sizes[i];
        g.num_pages = num_pages[i];
        g.window = windows[i];
        g.owner.assign(g.num_pages, -1);
        for (int p = 0; p < g.num_pages; ++p) g.free_pages.push_back(p);
    }
    m->slot_owner.assign(num_slots, -1);
    for (int s = 0; s < num_slots; ++s) m->free_slots.push_back(s);
    return m;
}

MSTAR_API void cm_destroy(void* h) { delete static_cast<Manager*>(h); }

// The number of positions the model was built for (the reference derives max_seq_len
// from max_position_embeddings, mstar/model/orpheus/orpheus_model.py:88-95): a
// reservation that would give a token a position id at or beyond it is refused with
// kTooLong.  0 lifts the limit.
MSTAR_API int cm_set_max_positions(void* h, int64_t max_positions) {
    auto& m = *static_cast<Manager*>(h);
    std::lock_guard<std::mutex> lock(m.mu);
    if (max_positions < 0) return kBadArg;
    m.max_positions = max_positions;
    return kOk;
}

MSTAR_API int cm_add_request(void* h, int64_t rid) {
    auto& m = *static_cast<Manager*>(h);
    std::lock_guard<std::mutex> lock(m.mu);
    if (m.requests.count(rid)) return kDuplicate;
    if (m.free_slots.empty()) return kNoSlot;
    Request r;
    r.slot = m.free_slots.front();
    m.free_slots.pop_front();
    m.slot_owner[r.slot] = rid;
    r.table.resize(m.groups.size());
    const int slot = r.slot;
    m.requests.emplace(rid, std::move(r));
    return slot;
}

MSTAR_API int cm_free_request(void* h, int64_t rid) {
    auto& m = *static_cast<Manager*>(h);
    std::lock_guard<std::mutex> lock(m.mu);
    auto it = m.requests.find(rid);
    if (it == m.requests.end()) return kUnknown;
    Request& r = it->second;
    for (size_t gi = 0; gi < m.groups.size(); ++gi) {
        Group& g = m.groups[gi];
        for (int p : r.table[gi]) {
            if (p >= 0) {
                g.owner[p] = -1;
                g.free_pages.push_back(p);
            }
        }
    }
    m.slot_owner[r.slot] = -1;
    m.free_slots.push_back(r.slot);
    m.requests.erase(it);
    return kOk;
}

// New pages each group would have to hand out for this batch; returns kOk, or
// kUnknown / kBadArg.  needed[g] is filled for every group.
MSTAR_API int cm_pages_needed(void* h, int n, const int64_t* rids, const int* n_new,
                              int64_t* needed) {
    auto& m = *static_cast<Manager*>(h);
    std::lock_guard<std::mutex> lock(m.mu);
    for (size_t gi = 0; gi < m.groups.size(); ++gi) needed[gi] = 0;
    for (int i = 0; i < n; ++i) {
        if (n_new[i] < 0) return kBadArg;
        auto it = m.requests.find(rids[i]);
        if (it == m.requests.end()) return kUnknown;
        for (size_t gi = 0; gi < m.groups.size(); ++gi)
            needed[gi] += new_pages_needed(m.groups[gi], it->second, (int)gi, n_new[i]);
    }
    return kOk;
}

// Make room for n_new[i] more tokens of every request of the batch, in every
// group, or change nothing.  On kNoPages, short_by[g] says how many pages group g
// lacks.  A request may appear only once in a batch.
MSTAR_API int cm_reserve(void* h, int n, const int64_t* rids, const int* n_new,
                         int64_t* short_by) {
    auto& m = *static_cast<Manager*>(h);
    std::lock_guard<std::mutex> lock(m.mu);
    const size_t ng = m.groups.size();
    std::vector<int64_t> need(ng, 0);
    std::vector<Request*> reqs(n);
    for (int i = 0; i < n; ++i) {
        if (n_new[i] < 0) return kBadArg;
        auto it = m.requests.find(rids[i]);
        if (it == m.requests.end()) return kUnknown;
        for (int j = 0; j < i; ++j)
            if (rids[j] == rids[i]) return kBadArg;
        if (m.max_positions > 0 && it->second.pos + n_new[i] > m.max_positions) {
            if (short_by) short_by[0] = i;  // which entry of the batch is too long
            return kTooLong;
        }
        reqs[i] = &it->second;
        for (size_t gi = 0; gi < ng; ++gi)
            need[gi] += new_pages_needed(m.groups[gi], it->second, (int)gi, n_new[i]);
    }
    bool ok = true;
    for (size_t gi = 0; gi < ng; ++gi) {
        const int64_t lack = need[gi] - (int64_t)m.groups[gi].free_pages.size();
        if (short_by) short_by[gi] = lack > 0 ? lack : 0;
        if (lack > 0) ok = false;
    }
    if (!ok) return kNoPages;
    for (int i = 0; i < n; ++i) {
        Request& r = *reqs[i];
        for (size_t gi = 0; gi < ng; ++gi) {
            Group& g = m.groups[gi];
            int64_t k = new_pages_needed(g, r, (int)gi, n_new[i]);
            for (; k > 0; --k) {
                const int p = g.free_pages.front();
                g.free_pages.pop_front();
                g.owner[p] = rids[i];
                r.table[gi].push_back(p);
            }
        }
    }
    return kOk;
}

// The forward pass over n_new tokens is done: advance the length by n_new and the
// position counter by pos_advance (negative: by n_new as well), and give back the
// pages of windowed groups that no later token can see.
MSTAR_API int cm_commit_positions(void* h, int64_t rid, int n_new, int64_t pos_advance) {
    auto& m = *static_cast<Manager*>(h);
    std::lock_guard<std::mutex> lock(m.mu);
    auto it = m.requests.find(rid);
    if (it == m.requests.end()) return kUnknown;
    if (n_new < 0) return kBadArg;
    Request& r = it->second;
    for (size_t gi = 0; gi < m.groups.size(); ++gi) {
        const int64_t cap = (int64_t)r.table[gi].size() * m.groups[gi].page_size;
        if (r.len + n_new > cap) return kBadArg;  // commit without reserve
    }
    r.len += n_new;
    r.pos += pos_advance < 0 ? n_new : pos_advance;
    release_passed(m, rid, r);
    return kOk;
}

MSTAR_API int cm_commit(void* h, int64_t rid, int n_new) {
    return cm_commit_positions(h, rid, n_new, -1);
}

// The position id that the request's next token gets (equal to its length unless a
// commit advanced the two differently or cm_set_position moved it).
MSTAR_API int64_t cm_position(void* h, int64_t rid) {
    auto& m = *static_cast<Manager*>(h);
    std::lock_guard<std::mutex> lock(m.mu);
    auto it = m.requests.find(rid);
    return it == m.requests.end() ? (int64_t)kUnknown : it->second.pos;
}

MSTAR_API int cm_set_position(void* h, int64_t rid, int64_t pos) {
    auto& m = *static_cast<Manager*>(h);
    std::lock_guard<std::mutex> lock(m.mu);
    auto it = m.requests.find(rid);
    if (it == m.requests.end()) return kUnknown;
    if (pos < 0) return kBadArg;
    it->second.pos = pos;
    return kOk;
}

MSTAR_API int64_t cm_len(void* h, int64_t rid) {
    auto& m = *static_cast<Manager*>(h);
    std::lock_guard<std::mutex> lock(m.mu);
    auto it = m.requests.find(rid);
    return it == m.requests.end() ? (int64_t)kUnknown : it->second.len;
}

MSTAR_API int cm_slot(void* h, int64_t rid) {
    auto& m = *static_cast<Manager*>(h);
    std::lock_guard<std::mutex> lock(m.mu);
    auto it = m.requests.find(rid);
    return it == m.requests.end() ? kUnknown : it->second.slot;
}

MSTAR_API int64_t cm_free_pages(void* h, int group) {
    auto& m = *static_cast<Manager*>(h);
    std::lock_guard<std::mutex> lock(m.mu);
    if (group < 0 || group >= (int)m.groups.size()) return kBadArg;
    return (int64_t)m.groups[group].free_pages.size();
}

MSTAR_API int cm_free_slots(void* h) {
    auto& m = *static_cast<Manager*>(h);
    std::lock_guard<std::mutex> lock(m.mu);
    return (int)m.free_slots.size();
}

MSTAR_API int cm_num_requests(void* h) {
    auto& m = *static_cast<Manager*>(h);
    std::lock_guard<std::mutex> lock(m.mu);
    return (int)m.requests.size();
}

// Block table of one request in one group: logical page -> page id (-1 once a
// window has passed it).  Returns the number of logical pages, or an error.
MSTAR_API int64_t cm_block_table(void* h, int64_t rid, int group, int* out, int64_t capacity) {
    auto& m = *static_cast<Manager*>(h);
    std::lock_guard<std::mutex> lock(m.mu);
    auto it = m.requests.find(rid);
    if (it == m.requests.end()) return kUnknown;
    if (group < 0 || group >= (int)m.groups.size()) return kBadArg;
    const auto& tab = it->second.table[group];
    const int64_t n = (int64_t)tab.size();
    for (int64_t i = 0; i < n && i < capacity; ++i) out[i] = tab[i];
    return n;
}

// Width (logical pages) of each group's block table for this batch.
MSTAR_API int cm_batch_widths(void* h, int n, const int64_t* rids, int* widths) {
    auto& m = *static_cast<Manager*>(h);
    std::lock_guard<std::mutex> lock(m.mu);
    for (size_t gi = 0; gi < m.groups.size(); ++gi) widths[gi] = 0;
    for (int i = 0; i < n; ++i) {
        auto it = m.requests.find(rids[i]);
        if (it == m.requests.end()) return kUnknown;
        for (size_t gi = 0; gi < m.groups.size(); ++gi) {
            const int w = (int)it->second.table[gi].size();
            if (w > widths[gi]) widths[gi] = w;
        }
    }
    return kOk;
}

// Per-step index arrays for a reserved batch, written into caller memory (int32):
//   token_req[T]  entry of the batch each token belongs to
//   positions[T]  position id of each token (position counter + offset in portion)
//   cache_pos[T]  index of the token's key in the request's key sequence
//                 (committed length + offset in portion)
//   qo_indptr[n+1], kv_len[n] (length after this step), slots[n]
//   tables[g]     [n, widths[g]] block tables, -1 where no page is held
MSTAR_API int cm_fill_batch(void* h, int n, const int64_t* rids, const int* n_new,
                            int* token_req, int* positions, int* cache_pos, int* qo_indptr,
                            int* kv_len, int* slots, int** tables, const int* widths) {
    auto& m = *static_cast<Manager*>(h);
    std::lock_guard<std::mutex> lock(m.mu);
    int t = 0;
    qo_indptr[0] = 0;
    for (int i = 0; i < n; ++i) {
        auto it = m.requests.find(rids[i]);
        if (it == m.requests.end()) return kUnknown;
        const Request& r = it->second;
        for (int k = 0; k < n_new[i]; ++k, ++t) {
            token_req[t] = i;
            positions[t] = (int)(r.pos + k);
            cache_pos[t] = (int)(r.len + k);
        }
        qo_indptr[i + 1] = t;
        kv_len[i] = (int)(r.len + n_new[i]);
        slots[i] = r.slot;
        for (size_t gi = 0; gi < m.groups.size(); ++gi) {
            const auto& tab = r.table[gi];
            const int64_t need = ceil_div(r.len + n_new[i], m.groups[gi].page_size);
            if ((int64_t)tab.size() < need) return kBadArg;  // not reserved
            if ((int)tab.size() > widths[gi]) return kBadArg;  // row too narrow for the table
            int* row = tables[gi] + (size_t)i * widths[gi];
            for (int w = 0; w < widths[gi]; ++w) row[w] = w < (int)tab.size() ? tab[w] : -1;
        }
    }
    return kOk;
}

// Invariants: every page is free exactly once or held exactly once by the request
// recorded as its owner; the same for slots.  Returns 0 or the number of faults.
MSTAR_API int cm_check(void* h) {
    auto& m = *static_cast<Manager*>(h);
    std::lock_guard<std::mutex> lock(m.mu);
    int faults = 0;
    for (size_t gi = 0; gi < m.groups.size(); ++gi) {
        const Group& g = m.groups[gi];
        std::vector<int> seen(g.num_pages, 0);
        for (int p : g.free_pages) {
            if (p < 0 || p >= g.num_pages) { ++faults; continue; }
            ++seen[p];
            if (g.owner[p] != -1) ++faults;
        }
        for (const auto& kv : m.requests) {
            for (int p : kv.second.table[gi]) {
                if (p < 0) continue;
                if (p >= g.num_pages) { ++faults; continue; }
                ++seen[p];
                if (g.owner[p] != kv.first) ++faults;
            }
        }
        for (int p = 0; p < g.num_pages; ++p)
            if (seen[p] != 1) ++faults;
    }
    std::vector<int> sseen(m.slot_owner.size(), 0);
    for (int s : m.free_slots) {
        if (s < 0 || s >= (int)sseen.size()) { ++faults; continue; }
        ++sseen[s];
        if (m.slot_owner[s] != -1) ++faults;
    }
    for (const auto& kv : m.requests) {
        const int s = kv.second.slot;
        if (s < 0 || s >= (int)sseen.size()) { ++faults; continue; }
        ++sseen[s];
        if (m.slot_owner[s] != kv.first) ++faults;
    }
    for (size_t s = 0; s < sseen.size(); ++s)
        if (sseen[s] != 1) ++faults;
    return faults;
}
