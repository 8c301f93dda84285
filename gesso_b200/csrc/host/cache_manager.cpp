// The cache manager's bookkeeping, on the host.
//
// Keys and values live in pages of `page_size` positions.  Layers with the same need form a group;
// a group has a page pool of its own and every request one block table per group, so one page id
// covers the same positions in every layer of the group.  Pages go back to the pool when the request
// ends or, in a windowed group, as soon as every position on them lies behind the window of all
// queries still to come; freed pages are reused at once (last freed, first reused).  Beside the pages
// every request holds one slot: the index of its fixed-size state.
//
// This file owns no device memory and runs no kernel (the reference's paged manager owns storage and
// append and gathers on read, src/Inference/kv_manager.jl:68-95, 234-297, 370-400; here kernels read
// pages in place through the block table, so the manager only hands out indices).  Requests are named
// by 64-bit handles that the Python layer maps its request ids to.  Every function returns 0 or a
// negative code; nothing throws across the C boundary.
#include <cstdint>
#include <cstring>
#include <unordered_map>
#include <vector>

#define HOST_API extern "C" __attribute__((visibility("default")))

namespace {

enum {
    OK = 0,
    E_NOT_LIVE = -1,       // the request is not live
    E_LIVE = -2,           // the request is already live
    E_NO_SLOT = -3,        // no free state slot
    E_CONTEXT = -4,        // the positions would exceed the context length
    E_PAGES = -5,          // a group has too few free pages (see last_short)
    E_BAD_ARG = -6,
    E_COMMIT = -7,         // commit beyond what is reserved
    E_INVARIANT = -8,      // check_invariants found an inconsistency (see last_short for the kind)
    E_INDEX = -9,          // pool: index freed but not held / handed out twice
    E_EMPTY = -10,         // pool: nothing free
};

const int FREED = -1;

struct Pool {
    int count = 0;
    std::vector<int> free_list;    // back() is handed out next
    std::vector<char> held;
    explicit Pool(int n = 0) : count(n), held(n, 0) {
        free_list.reserve(n);
        for (int i = n - 1; i >= 0; --i) free_list.push_back(i);     // 0 is handed out first
    }
    int free_count() const { return (int)free_list.size(); }
    int alloc() {
        if (free_list.empty()) return E_EMPTY;
        const int i = free_list.back();
        if (held[i]) return E_INDEX;
        free_list.pop_back();
        held[i] = 1;
        return i;
    }
    int release(int i) {
        if (i < 0 || i >= count || !held[i]) return E_INDEX;
        held[i] = 0;
        free_list.push_back(i);
        return OK;
    }
};

struct Request {
    int slot = 0;
    int length = 0;       // positions committed so far
    int reserved = 0;     // positions covered by pages (>= length)
    bool fresh = true;    // state slot not zeroed yet
    std::vector<int> n_pages;              // per group: entries of the block table in use
    std::vector<std::vector<int>> rows;    // per group: fixed-width block table, FREED where no page is held
};

struct Manager {
    std::vector<int> windows;              // per group: 0 = every earlier key is kept
    int page_size = 1, max_positions = 1, max_pages = 1;
    std::vector<Pool> pools;
    Pool slots;
    std::unordered_map<int64_t, Request> reqs;
    std::vector<int64_t> order;            // live requests in admission order
    int short_group = -1, short_need = 0, short_free = 0;   // details of the last E_PAGES / E_INVARIANT

    int pages_for(int positions) const { return (positions + page_size - 1) / page_size; }
    Request* find(int64_t rid) {
        auto it = reqs.find(rid);
        return it == reqs.end() ? nullptr : &it->second;
    }
    // hand out pages so that every group's table covers `want` pages (the caller has checked the pools)
    int grow(Request& r, int want) {
        for (size_t g = 0; g < pools.size(); ++g) {
            while (r.n_pages[g] < want) {
                const int page = pools[g].alloc();
                if (page < 0) return page;
                r.rows[g][r.n_pages[g]++] = page;
            }
        }
        return OK;
    }
};

}  // namespace

// ---- index pool on its own (pages of a group, state slots) --------------------------------------------
HOST_API void* gesso_pool_new(int count) { return count < 0 ? nullptr : new Pool(count); }
HOST_API void gesso_pool_delete(void* p) { delete static_cast<Pool*>(p); }
HOST_API int gesso_pool_alloc(void* p) { return static_cast<Pool*>(p)->alloc(); }
HOST_API int gesso_pool_free(void* p, int i) { return static_cast<Pool*>(p)->release(i); }
HOST_API int gesso_pool_free_count(void* p) { return static_cast<Pool*>(p)->free_count(); }
HOST_API int gesso_pool_is_held(void* p, int i) {
    Pool* q = static_cast<Pool*>(p);
    return i >= 0 && i < q->count && q->held[i];
}

// ---- the manager -------------------------------------------------------------------------------------
HOST_API void* gesso_cm_new(int n_groups, const int* windows, int page_size, const int* num_pages, int num_slots,
                            int max_positions) {
    if (n_groups < 0 || page_size < 1 || max_positions < 1 || num_slots < 0) return nullptr;
    Manager* m = new Manager();
    m->page_size = page_size;
    m->max_positions = max_positions;
    m->max_pages = (max_positions + page_size - 1) / page_size;
    for (int g = 0; g < n_groups; ++g) {
        if (windows[g] < 0 || num_pages[g] < 0) { delete m; return nullptr; }
        m->windows.push_back(windows[g]);
        m->pools.emplace_back(num_pages[g]);
    }
    m->slots = Pool(num_slots);
    return m;
}
HOST_API void gesso_cm_delete(void* cm) { delete static_cast<Manager*>(cm); }

HOST_API int gesso_cm_admit(void* cm, int64_t rid) {
    Manager* m = static_cast<Manager*>(cm);
    if (m->find(rid)) return E_LIVE;
    const int slot = m->slots.alloc();
    if (slot == E_EMPTY) return E_NO_SLOT;
    if (slot < 0) return slot;
    Request r;
    r.slot = slot;
    r.n_pages.assign(m->pools.size(), 0);
    r.rows.assign(m->pools.size(), std::vector<int>(m->max_pages, FREED));
    m->reqs.emplace(rid, std::move(r));
    m->order.push_back(rid);
    return slot;
}

HOST_API int gesso_cm_release(void* cm, int64_t rid) {
    Manager* m = static_cast<Manager*>(cm);
    Request* r = m->find(rid);
    if (!r) return E_NOT_LIVE;
    for (size_t g = 0; g < m->pools.size(); ++g)
        for (int i = r->n_pages[g] - 1; i >= 0; --i)
            if (r->rows[g][i] != FREED) {
                const int e = m->pools[g].release(r->rows[g][i]);
                if (e < 0) return e;
            }
    const int e = m->slots.release(r->slot);
    m->reqs.erase(rid);
    for (size_t i = 0; i < m->order.size(); ++i)
        if (m->order[i] == rid) { m->order.erase(m->order.begin() + i); break; }
    return e;
}

// info[0..3] = length, reserved, slot, fresh
HOST_API int gesso_cm_info(void* cm, int64_t rid, int* info) {
    Request* r = static_cast<Manager*>(cm)->find(rid);
    if (!r) return E_NOT_LIVE;
    info[0] = r->length;
    info[1] = r->reserved;
    info[2] = r->slot;
    info[3] = r->fresh ? 1 : 0;
    return OK;
}

// 1 exactly once per admission: the caller must zero the slot's state now
HOST_API int gesso_cm_take_fresh(void* cm, int64_t rid) {
    Request* r = static_cast<Manager*>(cm)->find(rid);
    if (!r) return E_NOT_LIVE;
    const int was = r->fresh ? 1 : 0;
    r->fresh = false;
    return was;
}

// pages each group still has to hand out so that n_new more positions fit
HOST_API int gesso_cm_pages_needed(void* cm, int64_t rid, int n_new, int* out) {
    Manager* m = static_cast<Manager*>(cm);
    Request* r = m->find(rid);
    if (!r) return E_NOT_LIVE;
    const int want = m->pages_for(r->length + n_new);
    for (size_t g = 0; g < m->pools.size(); ++g) out[g] = want > r->n_pages[g] ? want - r->n_pages[g] : 0;
    return OK;
}

// the pages for positions length .. length + n_new - 1, in all groups or in none
HOST_API int gesso_cm_reserve(void* cm, int64_t rid, int n_new) {
    Manager* m = static_cast<Manager*>(cm);
    Request* r = m->find(rid);
    if (!r) return E_NOT_LIVE;
    if (n_new < 0) return E_BAD_ARG;
    if (r->length + n_new > m->max_positions) return E_CONTEXT;
    const int want = m->pages_for(r->length + n_new);
    for (size_t g = 0; g < m->pools.size(); ++g) {
        const int need = want > r->n_pages[g] ? want - r->n_pages[g] : 0;
        if (need > m->pools[g].free_count()) {
            m->short_group = (int)g;
            m->short_need = need;
            m->short_free = m->pools[g].free_count();
            return E_PAGES;
        }
    }
    const int e = m->grow(*r, want);
    if (e < 0) return e;
    if (r->length + n_new > r->reserved) r->reserved = r->length + n_new;
    return OK;
}

// n_new positions were written; windowed groups give back what no query will read
HOST_API int gesso_cm_commit(void* cm, int64_t rid, int n_new) {
    Manager* m = static_cast<Manager*>(cm);
    Request* r = m->find(rid);
    if (!r) return E_NOT_LIVE;
    if (n_new < 0 || r->length + n_new > r->reserved) return E_COMMIT;
    r->length += n_new;
    for (size_t g = 0; g < m->pools.size(); ++g) {
        if (m->windows[g] == 0) continue;
        // the next query sits at position >= length and reads keys >= length - window + 1
        const int first_needed = r->length - m->windows[g] + 1;
        int dead = (first_needed > 0 ? first_needed : 0) / m->page_size;
        if (dead > r->n_pages[g]) dead = r->n_pages[g];
        for (int i = 0; i < dead; ++i)
            if (r->rows[g][i] != FREED) {
                const int e = m->pools[g].release(r->rows[g][i]);
                if (e < 0) return e;
                r->rows[g][i] = FREED;
            }
    }
    return OK;
}

HOST_API int gesso_cm_commit_many(void* cm, const int64_t* rids, int n, int n_new) {
    for (int i = 0; i < n; ++i) {
        const int e = gesso_cm_commit(cm, rids[i], n_new);
        if (e < 0) return e;
    }
    return OK;
}

// A whole step at once: the pages for n_new[i] more positions of request i, for all requests or for none.
// starts[i] = the request's length now, slots[i] = its state slot; fresh_slots receives the slots whose
// state must be zeroed before the step; info[0] = their count (or the index of the offending request),
// info[1] = the longest sequence after the step.
HOST_API int gesso_cm_reserve_step(void* cm, const int64_t* rids, const int* n_new, int n, int* starts, int* slots,
                                   int* fresh_slots, int* info) {
    Manager* m = static_cast<Manager*>(cm);
    if (n <= 0) return E_BAD_ARG;
    const int G = (int)m->pools.size();
    std::vector<Request*> reqs(n);
    std::vector<int> need(G, 0);
    for (int i = 0; i < n; ++i) {
        Request* r = m->find(rids[i]);
        if (!r) { info[0] = i; return E_NOT_LIVE; }
        for (int j = 0; j < i; ++j)
            if (reqs[j] == r) { info[0] = i; return E_BAD_ARG; }     // a request twice in one step
        if (n_new[i] < 0) { info[0] = i; return E_BAD_ARG; }
        if (r->length + n_new[i] > m->max_positions) { info[0] = i; return E_CONTEXT; }
        const int wantp = m->pages_for(r->length + n_new[i]);
        for (int g = 0; g < G; ++g)
            if (wantp > r->n_pages[g]) need[g] += wantp - r->n_pages[g];
        reqs[i] = r;
    }
    for (int g = 0; g < G; ++g)
        if (need[g] > m->pools[g].free_count()) {
            m->short_group = g;
            m->short_need = need[g];
            m->short_free = m->pools[g].free_count();
            return E_PAGES;
        }
    int n_fresh = 0, max_kv = 0;
    for (int i = 0; i < n; ++i) {
        Request& r = *reqs[i];
        const int e = m->grow(r, m->pages_for(r.length + n_new[i]));
        if (e < 0) return e;
        if (r.length + n_new[i] > r.reserved) r.reserved = r.length + n_new[i];
        if (r.fresh) {
            r.fresh = false;
            fresh_slots[n_fresh++] = r.slot;
        }
        starts[i] = r.length;
        slots[i] = r.slot;
        if (r.length + n_new[i] > max_kv) max_kv = r.length + n_new[i];
    }
    info[0] = n_fresh;
    info[1] = max_kv;
    return OK;
}

// n_new[i] positions of request i were written
HOST_API int gesso_cm_commit_step(void* cm, const int64_t* rids, const int* n_new, int n) {
    for (int i = 0; i < n; ++i) {
        const int e = gesso_cm_commit(cm, rids[i], n_new[i]);
        if (e < 0) return e;
    }
    return OK;
}

// the block table of a request in a group: a pointer to max_pages ints that stays valid (and up to date)
// until the request is released; *n_used entries are in use
HOST_API const int* gesso_cm_row(void* cm, int64_t rid, int group, int* n_used) {
    Manager* m = static_cast<Manager*>(cm);
    Request* r = m->find(rid);
    if (!r || group < 0 || group >= (int)m->pools.size()) return nullptr;
    if (n_used) *n_used = r->n_pages[group];
    return r->rows[group].data();
}

// out[0..G) pages in use, out[G..2G) pages free, out[2G] slots in use, out[2G+1] slots free, out[2G+2] live requests
HOST_API void gesso_cm_counts(void* cm, int* out) {
    Manager* m = static_cast<Manager*>(cm);
    const int G = (int)m->pools.size();
    for (int g = 0; g < G; ++g) {
        out[g] = m->pools[g].count - m->pools[g].free_count();
        out[G + g] = m->pools[g].free_count();
    }
    out[2 * G] = m->slots.count - m->slots.free_count();
    out[2 * G + 1] = m->slots.free_count();
    out[2 * G + 2] = (int)m->order.size();
}

HOST_API int gesso_cm_live(void* cm, int64_t* out, int cap) {
    Manager* m = static_cast<Manager*>(cm);
    const int n = (int)m->order.size();
    for (int i = 0; i < n && i < cap; ++i) out[i] = m->order[i];
    return n;
}

// details of the last E_PAGES (group, need, free) or E_INVARIANT (group, kind, page)
HOST_API void gesso_cm_last_short(void* cm, int* out) {
    Manager* m = static_cast<Manager*>(cm);
    out[0] = m->short_group;
    out[1] = m->short_need;
    out[2] = m->short_free;
}

// No page lost, none held twice, the pools' counts equal what the tables hold.
// kinds (last_short[1]): 1 a page is held twice, 2 a table names a page its pool does not hold, 3 the pool
// holds more pages than the tables name, 4 the free list is inconsistent, 5 a page was lost, 6 slots.
HOST_API int gesso_cm_check(void* cm) {
    Manager* m = static_cast<Manager*>(cm);
    auto fail = [&](int g, int kind, int page) { m->short_group = g; m->short_need = kind; m->short_free = page; return (int)E_INVARIANT; };
    for (size_t g = 0; g < m->pools.size(); ++g) {
        Pool& p = m->pools[g];
        std::vector<char> seen(p.count, 0);
        int n_seen = 0;
        for (auto& kv : m->reqs) {
            const Request& r = kv.second;
            for (int i = 0; i < r.n_pages[g]; ++i) {
                const int page = r.rows[g][i];
                if (page == FREED) continue;
                if (page < 0 || page >= p.count || !p.held[page]) return fail((int)g, 2, page);
                if (seen[page]) return fail((int)g, 1, page);
                seen[page] = 1;
                ++n_seen;
            }
        }
        if (n_seen != p.count - p.free_count()) return fail((int)g, 3, n_seen);
        std::vector<char> in_free(p.count, 0);
        for (int page : p.free_list) {
            if (page < 0 || page >= p.count || in_free[page] || seen[page] || p.held[page]) return fail((int)g, 4, page);
            in_free[page] = 1;
        }
        int held = 0;
        for (char h : p.held) held += h;
        if (held + p.free_count() != p.count) return fail((int)g, 5, held);
    }
    std::vector<char> slot_seen(m->slots.count, 0);
    for (auto& kv : m->reqs) {
        const int s = kv.second.slot;
        if (s < 0 || s >= m->slots.count || slot_seen[s] || !m->slots.held[s]) return fail(-1, 6, s);
        slot_seen[s] = 1;
    }
    if ((int)m->reqs.size() != m->slots.count - m->slots.free_count()) return fail(-1, 6, (int)m->reqs.size());
    return OK;
}
