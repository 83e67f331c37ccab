// Host bookkeeping of the paged cache, in C++: page pools with a FIFO free list,
// request slots, and a block table per request and cache group, with the rules of
// growth and give-back.  No device memory is touched here; the Python classes of
// kipp_b200/cache are thin wrappers that map request ids to 64-bit integers and
// error codes to exceptions.
//
// Reference counterparts: the block pool (src/kipp_kv_pool.c:89-99 all blocks free in
// id order, :202-213 take the head of the free list, :258-269 and :306-321 a
// released block goes to the tail) and the mapping of a session's logical blocks
// (src/kipp.c:3616-3635 grow or leave untouched, :3755-3768 truncate, :3776-3791
// release).  Prefix sharing (the reference's content index and reference counts) is
// not built: a page has one owner at most.
#include <cstdint>
#include <deque>
#include <unordered_map>
#include <utility>
#include <vector>

namespace {
constexpr int OK = 0;
constexpr int ERR_OUT_OF_PAGES = -1;
constexpr int ERR_OUT_OF_SLOTS = -2;
constexpr int ERR_ARGUMENT = -3;        // unknown or duplicate request, shrinking, outside a range
constexpr int ERR_BEHIND_WINDOW = -4;   // a page the window has given back was asked for
constexpr int ERR_CHECK = -5;           // an invariant does not hold
constexpr int ERR_FREED_TWICE = -6;
constexpr int ERR_NOT_OWNER = -7;
constexpr int ERR_WINDOW_REFUSES = -8;  // truncate into pages a window group no longer holds
constexpr int UNMAPPED = -1;
constexpr int64_t NO_OWNER = INT64_MIN;

struct Pool {
    int n_pages;
    std::deque<int> free_list;
    std::vector<int64_t> owner;
    explicit Pool(int n) : n_pages(n), owner((size_t)n, NO_OWNER) {
        for (int i = 0; i < n; ++i) free_list.push_back(i);
    }
    int alloc(int64_t who) {
        if (free_list.empty()) return ERR_OUT_OF_PAGES;
        const int page = free_list.front();
        free_list.pop_front();
        owner[(size_t)page] = who;
        return page;
    }
    int release(int page, int64_t who) {
        if (page < 0 || page >= n_pages) return ERR_ARGUMENT;
        if (owner[(size_t)page] == NO_OWNER) return ERR_FREED_TWICE;
        if (owner[(size_t)page] != who) return ERR_NOT_OWNER;
        owner[(size_t)page] = NO_OWNER;
        free_list.push_back(page);
        return OK;
    }
    // every page is either free exactly once or owned
    int check() const {
        std::vector<char> is_free((size_t)n_pages, 0);
        for (int p : free_list) {
            if (p < 0 || p >= n_pages || is_free[(size_t)p]) return ERR_CHECK;
            is_free[(size_t)p] = 1;
        }
        for (int p = 0; p < n_pages; ++p)
            if ((owner[(size_t)p] == NO_OWNER) != (is_free[(size_t)p] != 0)) return ERR_CHECK;
        return OK;
    }
};

struct Slots {
    int max_requests;
    std::vector<int> free_stack;                     // the lowest slot is handed out first
    std::unordered_map<int, int64_t> owner;
    explicit Slots(int n) : max_requests(n) {
        for (int i = n - 1; i >= 0; --i) free_stack.push_back(i);
    }
    int alloc(int64_t who) {
        if (free_stack.empty()) return ERR_OUT_OF_SLOTS;
        const int slot = free_stack.back();
        free_stack.pop_back();
        owner[slot] = who;
        return slot;
    }
    int release(int slot, int64_t who) {
        auto it = owner.find(slot);
        if (it == owner.end() || it->second != who) return ERR_NOT_OWNER;
        owner.erase(it);
        free_stack.push_back(slot);
        return OK;
    }
    int check() const {
        std::vector<char> seen((size_t)max_requests, 0);
        for (int s : free_stack) {
            if (s < 0 || s >= max_requests || seen[(size_t)s]) return ERR_CHECK;
            seen[(size_t)s] = 1;
        }
        for (const auto& kv : owner) {
            if (kv.first < 0 || kv.first >= max_requests || seen[(size_t)kv.first]) return ERR_CHECK;
            seen[(size_t)kv.first] = 1;
        }
        for (char c : seen)
            if (!c) return ERR_CHECK;
        return OK;
    }
};

struct Request {
    int slot = 0;
    int length = 0;
    std::vector<std::vector<int>> tables;            // per group: logical page -> physical page or UNMAPPED
    std::vector<int> first_live;                     // per group: first logical page that may still be mapped
};

struct Group {
    Pool pool;
    int window;                                      // -1: every key is kept
    Group(int pages, int w) : pool(pages), window(w) {}
};

struct Manager {
    int page_size;
    std::vector<Group> groups;
    Slots slots;
    std::unordered_map<int64_t, Request> requests;
    Manager(int ps, int max_requests) : page_size(ps), slots(max_requests) {}

    Request* find(int64_t rid) {
        auto it = requests.find(rid);
        return it == requests.end() ? nullptr : &it->second;
    }
    static void set_page(std::vector<int>& table, int logical, int page) {
        if ((int)table.size() <= logical) table.resize((size_t)logical + 1, UNMAPPED);
        table[(size_t)logical] = page;
    }
    static void trim(std::vector<int>& table) {
        while (!table.empty() && table.back() == UNMAPPED) table.pop_back();
    }
    // logical pages that hold positions [first, end)
    std::pair<int, int> pages_for(int first, int end) const {
        if (end <= first) return {0, 0};
        return {first / page_size, (end - 1) / page_size + 1};
    }
    int first_needed_position(const Group& g, int length) const {
        if (g.window < 0) return 0;
        const int p = length - g.window + 1;
        return p > 0 ? p : 0;
    }
};
}  // namespace

// ------------------------------------------------------------------ stand-alone pool and slots
extern "C" void* kipp_pool_create(int n_pages) { return n_pages > 0 ? new Pool(n_pages) : nullptr; }
extern "C" void kipp_pool_destroy(void* h) { delete static_cast<Pool*>(h); }
extern "C" int kipp_pool_alloc(void* h, int64_t owner) { return static_cast<Pool*>(h)->alloc(owner); }
extern "C" int kipp_pool_free(void* h, int page, int64_t owner) { return static_cast<Pool*>(h)->release(page, owner); }
extern "C" int kipp_pool_free_pages(void* h) { return (int)static_cast<Pool*>(h)->free_list.size(); }
extern "C" int64_t kipp_pool_owner(void* h, int page) {
    Pool* p = static_cast<Pool*>(h);
    return (page < 0 || page >= p->n_pages) ? NO_OWNER : p->owner[(size_t)page];
}
extern "C" int kipp_pool_check(void* h) { return static_cast<Pool*>(h)->check(); }

extern "C" void* kipp_slots_create(int n) { return n > 0 ? new Slots(n) : nullptr; }
extern "C" void kipp_slots_destroy(void* h) { delete static_cast<Slots*>(h); }
extern "C" int kipp_slots_alloc(void* h, int64_t owner) { return static_cast<Slots*>(h)->alloc(owner); }
extern "C" int kipp_slots_free(void* h, int slot, int64_t owner) { return static_cast<Slots*>(h)->release(slot, owner); }
extern "C" int kipp_slots_free_count(void* h) { return (int)static_cast<Slots*>(h)->free_stack.size(); }
extern "C" int kipp_slots_check(void* h) { return static_cast<Slots*>(h)->check(); }

// ------------------------------------------------------------------ the manager
// windows[g] < 0: group g keeps every key.
extern "C" void* kipp_cm_create(int n_groups, const int* n_pages, const int* windows, int page_size,
                                int max_requests) {
    if (n_groups < 0 || page_size <= 0 || max_requests <= 0) return nullptr;
    for (int g = 0; g < n_groups; ++g)
        if (n_pages[g] <= 0) return nullptr;
    Manager* m = new Manager(page_size, max_requests);
    m->groups.reserve((size_t)n_groups);
    for (int g = 0; g < n_groups; ++g) m->groups.emplace_back(n_pages[g], windows[g]);
    return m;
}
extern "C" void kipp_cm_destroy(void* h) { delete static_cast<Manager*>(h); }

// The pool and the slots of a manager, for the stand-alone calls above (not to be destroyed).
extern "C" void* kipp_cm_pool(void* h, int group) { return &static_cast<Manager*>(h)->groups[(size_t)group].pool; }
extern "C" void* kipp_cm_slots(void* h) { return &static_cast<Manager*>(h)->slots; }

// A slot for the request; it holds no pages yet.  Returns the slot.
extern "C" int kipp_cm_admit(void* h, int64_t rid) {
    Manager* m = static_cast<Manager*>(h);
    if (m->find(rid)) return ERR_ARGUMENT;
    const int slot = m->slots.alloc(rid);
    if (slot < 0) return slot;
    Request r;
    r.slot = slot;
    r.tables.resize(m->groups.size());
    r.first_live.assign(m->groups.size(), 0);
    m->requests.emplace(rid, std::move(r));
    return slot;
}

// The request ended: all its pages and its slot go back.
extern "C" int kipp_cm_release(void* h, int64_t rid) {
    Manager* m = static_cast<Manager*>(h);
    auto it = m->requests.find(rid);
    if (it == m->requests.end()) return ERR_ARGUMENT;
    for (size_t g = 0; g < m->groups.size(); ++g)
        for (int page : it->second.tables[g])
            if (page != UNMAPPED) {
                const int rc = m->groups[g].pool.release(page, rid);
                if (rc) return rc;
            }
    const int rc = m->slots.release(it->second.slot, rid);
    m->requests.erase(it);
    return rc;
}

extern "C" int kipp_cm_slot(void* h, int64_t rid) {
    Request* r = static_cast<Manager*>(h)->find(rid);
    return r ? r->slot : ERR_ARGUMENT;
}
extern "C" int kipp_cm_length(void* h, int64_t rid) {
    Request* r = static_cast<Manager*>(h)->find(rid);
    return r ? r->length : ERR_ARGUMENT;
}

// Pages per group that a reserve up to new_length would take.
extern "C" int kipp_cm_missing_pages(void* h, int64_t rid, int new_length, int* out) {
    Manager* m = static_cast<Manager*>(h);
    Request* r = m->find(rid);
    if (!r) return ERR_ARGUMENT;
    for (size_t g = 0; g < m->groups.size(); ++g) {
        const auto range = m->pages_for(r->length, new_length);
        int missing = 0;
        for (int lp = range.first; lp < range.second; ++lp)
            if (lp >= (int)r->tables[g].size() || r->tables[g][(size_t)lp] == UNMAPPED) ++missing;
        out[g] = missing;
    }
    return OK;
}

// Map pages so that every (rid, new_length) can be written: either every request of
// the call gets its pages or none does, and then nothing has changed.
extern "C" int kipp_cm_reserve(void* h, int n, const int64_t* rids, const int* new_lengths) {
    Manager* m = static_cast<Manager*>(h);
    struct Taken { int group; int64_t rid; int logical; int page; };
    std::vector<Taken> taken;
    int rc = OK;
    for (int i = 0; i < n && rc == OK; ++i) {
        Request* r = m->find(rids[i]);
        if (!r || new_lengths[i] < r->length) { rc = ERR_ARGUMENT; break; }
        for (size_t g = 0; g < m->groups.size() && rc == OK; ++g) {
            std::vector<int>& table = r->tables[g];
            const auto range = m->pages_for(r->length, new_lengths[i]);
            for (int lp = range.first; lp < range.second; ++lp) {
                if (lp < (int)table.size() && table[(size_t)lp] != UNMAPPED) continue;
                if (lp < r->first_live[g]) { rc = ERR_BEHIND_WINDOW; break; }
                const int page = m->groups[g].pool.alloc(rids[i]);
                if (page < 0) { rc = page; break; }
                Manager::set_page(table, lp, page);
                taken.push_back({(int)g, rids[i], lp, page});
            }
        }
    }
    if (rc != OK) {
        for (auto it = taken.rbegin(); it != taken.rend(); ++it) {
            m->groups[(size_t)it->group].pool.release(it->page, it->rid);
            m->find(it->rid)->tables[(size_t)it->group][(size_t)it->logical] = UNMAPPED;
        }
        for (int i = 0; i < n; ++i)                  // drop the trailing holes the call made
            if (Request* r = m->find(rids[i]))
                for (auto& table : r->tables) Manager::trim(table);
    }
    return rc;
}

// The step wrote positions up to new_length: window groups give back the pages no
// later token can see.
extern "C" int kipp_cm_advance(void* h, int64_t rid, int new_length) {
    Manager* m = static_cast<Manager*>(h);
    Request* r = m->find(rid);
    if (!r || new_length < r->length) return ERR_ARGUMENT;
    r->length = new_length;
    for (size_t g = 0; g < m->groups.size(); ++g) {
        Group& grp = m->groups[g];
        if (grp.window < 0) continue;
        std::vector<int>& table = r->tables[g];
        int keep_from = m->first_needed_position(grp, new_length) / m->page_size;
        if (keep_from > (int)table.size()) keep_from = (int)table.size();
        for (int lp = r->first_live[g]; lp < keep_from; ++lp)
            if (table[(size_t)lp] != UNMAPPED) {
                const int rc = grp.pool.release(table[(size_t)lp], rid);
                if (rc) return rc;
                table[(size_t)lp] = UNMAPPED;
            }
        if (keep_from > r->first_live[g]) r->first_live[g] = keep_from;
    }
    return OK;
}

// Forget the positions from new_length on.  A window group can only be cut back to
// where the pages it still holds cover what the next token may see; else nothing
// changes and *refusing_group names the group.
extern "C" int kipp_cm_truncate(void* h, int64_t rid, int new_length, int* refusing_group) {
    Manager* m = static_cast<Manager*>(h);
    Request* r = m->find(rid);
    if (!r || new_length < 0 || new_length > r->length) return ERR_ARGUMENT;
    for (size_t g = 0; g < m->groups.size(); ++g) {
        const Group& grp = m->groups[g];
        if (grp.window < 0 || new_length == 0) continue;
        if (m->first_needed_position(grp, new_length) / m->page_size < r->first_live[g]) {
            if (refusing_group) *refusing_group = (int)g;
            return ERR_WINDOW_REFUSES;
        }
    }
    const int keep = (new_length + m->page_size - 1) / m->page_size;     // pages with positions below new_length
    for (size_t g = 0; g < m->groups.size(); ++g) {
        std::vector<int>& table = r->tables[g];
        for (int lp = keep; lp < (int)table.size(); ++lp)
            if (table[(size_t)lp] != UNMAPPED) {
                const int rc = m->groups[g].pool.release(table[(size_t)lp], rid);
                if (rc) return rc;
            }
        if ((int)table.size() > keep) table.resize((size_t)keep);
        if (new_length == 0) r->first_live[g] = 0;
        else if (r->first_live[g] > keep) r->first_live[g] = keep;
    }
    r->length = new_length;
    return OK;
}

extern "C" int kipp_cm_table_len(void* h, int64_t rid, int group) {
    Request* r = static_cast<Manager*>(h)->find(rid);
    return r ? (int)r->tables[(size_t)group].size() : ERR_ARGUMENT;
}
// The request's table of a group into out[0 .. cap); returns its length.
extern "C" int kipp_cm_table(void* h, int64_t rid, int group, int* out, int cap) {
    Request* r = static_cast<Manager*>(h)->find(rid);
    if (!r) return ERR_ARGUMENT;
    const std::vector<int>& table = r->tables[(size_t)group];
    for (int i = 0; i < (int)table.size() && i < cap; ++i) out[i] = table[(size_t)i];
    return (int)table.size();
}
// int32 [n, width] of physical pages, UNMAPPED where none; a table longer than width is an error.
extern "C" int kipp_cm_rows(void* h, int group, int n, const int64_t* rids, int width, int* out) {
    Manager* m = static_cast<Manager*>(h);
    for (int i = 0; i < n; ++i) {
        Request* r = m->find(rids[i]);
        if (!r) return ERR_ARGUMENT;
        const std::vector<int>& table = r->tables[(size_t)group];
        if ((int)table.size() > width) return ERR_ARGUMENT;
        int* row = out + (size_t)i * width;
        int j = 0;
        for (; j < (int)table.size(); ++j) row[j] = table[(size_t)j];
        for (; j < width; ++j) row[j] = UNMAPPED;
    }
    return OK;
}
extern "C" int kipp_cm_pages_held(void* h, int64_t rid, int* out) {
    Manager* m = static_cast<Manager*>(h);
    Request* r = m->find(rid);
    if (!r) return ERR_ARGUMENT;
    for (size_t g = 0; g < m->groups.size(); ++g) {
        int held = 0;
        for (int page : r->tables[g]) held += page != UNMAPPED;
        out[g] = held;
    }
    return OK;
}

// No page lost, held twice or free and held; tables, pools and slots agree.
extern "C" int kipp_cm_check(void* h) {
    Manager* m = static_cast<Manager*>(h);
    for (size_t g = 0; g < m->groups.size(); ++g) {
        const Pool& pool = m->groups[g].pool;
        if (pool.check()) return ERR_CHECK;
        std::vector<char> seen((size_t)pool.n_pages, 0);
        int held = 0;
        for (const auto& kv : m->requests)
            for (int page : kv.second.tables[g]) {
                if (page == UNMAPPED) continue;
                if (page < 0 || page >= pool.n_pages || seen[(size_t)page]) return ERR_CHECK;   // held twice
                seen[(size_t)page] = 1;
                if (pool.owner[(size_t)page] != kv.first) return ERR_CHECK;                     // table and pool disagree
                ++held;
            }
        if (held != pool.n_pages - (int)pool.free_list.size()) return ERR_CHECK;                // pages are lost
    }
    if (m->slots.check()) return ERR_CHECK;
    for (const auto& kv : m->requests) {
        auto it = m->slots.owner.find(kv.second.slot);
        if (it == m->slots.owner.end() || it->second != kv.first) return ERR_CHECK;
    }
    return OK;
}
