// The host side of a step, free of CUDA and of Python: the cache's bookkeeping (which slots are held, which
// pages every slot holds in every group of layers, how long every sequence is), the checks a step must pass
// before anything is launched, and the packing of a step's rows into the one int32 buffer that goes to the
// device in a single copy.  Python drives it through a C ABI (ctypes); every function returns 0 (or a count)
// on success and a negative code on failure, with the message in tqh_error().
//
// Reference: src/models/turbo_generic.rs:1606-1618 keeps one growing (K, V) pair per layer for a single
// sequence and src/engine.rs:117 one `position`; tq-kv/src/candle_kv.rs:53-153 shows the interface (append /
// current_seq_len / reset) that a slot offers here per sequence.  src/engine.rs:347-349 refuses an empty prompt.
#include <algorithm>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#define TQH_API extern "C" __attribute__((visibility("default")))

namespace {

// error codes (the Python side maps them to its exception classes)
enum { TQH_OK = 0, TQH_CACHE = -1, TQH_STEP = -2, TQH_BROKEN = -3 };

// A pool of integer handles 0..n-1 (slots, or pages of one group).  Handles are given out lowest first, so
// that a handle given back is used again soon: stale contents then show up in tests rather than in use.
struct Pool {
    int n = 0;
    std::vector<int> free_desc;        // descending, so that back() is the lowest
    std::vector<char> held;

    void init(int count) {
        n = count;
        free_desc.resize(n);
        for (int i = 0; i < n; ++i) free_desc[i] = n - 1 - i;
        held.assign(n, 0);
    }
    int free_count() const { return (int)free_desc.size(); }
    bool is_held(int i) const { return i >= 0 && i < n && held[i]; }
    int take() {                        // -1: none left; -2: the handle would be held twice
        if (free_desc.empty()) return -1;
        const int i = free_desc.back();
        free_desc.pop_back();
        if (held[i]) return -2;
        held[i] = 1;
        return i;
    }
    int give_back(int i) {              // -1: no such handle; -2: freed twice or never held
        if (i < 0 || i >= n) return -1;
        if (!held[i]) return -2;
        held[i] = 0;
        auto at = std::lower_bound(free_desc.begin(), free_desc.end(), i, [](int a, int b) { return a > b; });
        free_desc.insert(at, i);
        return 0;
    }
};

// Pages of one group of layers.  A sequence's logical page i (tokens i * page_tokens ..) lives in physical
// page pages[slot][i]; a ring group holds at most ring_pages pages per sequence and reuses them modulo.
struct Group {
    std::string name;
    int page_tokens = 64;
    int ring_pages = 0;                // 0: all keys are kept
    Pool pool;
    std::vector<std::vector<int>> pages;   // by slot

    int pages_for_length(int length) const {
        int n = (length + page_tokens - 1) / page_tokens;
        if (ring_pages > 0 && n > ring_pages) n = ring_pages;
        return n;
    }
    int need(int slot, int new_length) const {
        const int n = pages_for_length(new_length) - (int)pages[slot].size();
        return n > 0 ? n : 0;
    }
};

struct Book {
    Pool slots;
    std::vector<Group> groups;
    int max_length = 0;
    std::vector<int> length;           // by slot (0 for slots that are not held)
    std::vector<int> scratch;
    char error[512] = {0};

    int fail(int code, const char* fmt, ...) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(error, sizeof(error), fmt, ap);
        va_end(ap);
        return code;
    }
};

int pad4(int n) { return (n + 3) / 4 * 4; }

}  // namespace

struct TqhBook : Book {};

TQH_API TqhBook* tqh_book_new(int max_slots, int max_length, int n_groups, const int* n_pages, const int* page_tokens,
                              const int* ring_pages, const char* const* names) {
    if (max_slots <= 0 || max_length <= 0 || n_groups < 0) return nullptr;
    TqhBook* b = new TqhBook();
    b->slots.init(max_slots);
    b->max_length = max_length;
    b->length.assign(max_slots, 0);
    b->groups.resize(n_groups);
    for (int g = 0; g < n_groups; ++g) {
        Group& grp = b->groups[g];
        grp.name = names && names[g] ? names[g] : "";
        grp.page_tokens = page_tokens[g];
        grp.ring_pages = ring_pages[g] > 0 ? ring_pages[g] : 0;
        grp.pool.init(n_pages[g]);
        grp.pages.resize(max_slots);
        if (page_tokens[g] <= 0 || n_pages[g] < 0) {
            delete b;
            return nullptr;
        }
    }
    return b;
}

TQH_API void tqh_book_delete(TqhBook* b) { delete b; }
TQH_API const char* tqh_error(const TqhBook* b) { return b->error; }

// A free slot of length 0, the lowest one; fails when all are held.
TQH_API int tqh_alloc(TqhBook* b) {
    const int s = b->slots.take();
    if (s == -1) return b->fail(TQH_CACHE, "no free slot left (all %d are held)", b->slots.n);
    if (s < 0) return b->fail(TQH_BROKEN, "a slot would be held twice");
    b->length[s] = 0;
    return s;
}

// Gives the slot and every page it holds back; a double free is refused before any page moves.
TQH_API int tqh_free(TqhBook* b, int slot) {
    const int r = b->slots.give_back(slot);
    if (r == -1) return b->fail(TQH_CACHE, "slot %d does not exist (0..%d)", slot, b->slots.n - 1);
    if (r == -2) return b->fail(TQH_CACHE, "slot %d is freed twice or was never held", slot);
    for (Group& g : b->groups) {
        for (int p : g.pages[slot])
            if (g.pool.give_back(p) != 0)
                return b->fail(TQH_BROKEN, "page %d of cache group '%s' is freed twice or was never held", p, g.name.c_str());
        g.pages[slot].clear();
    }
    b->length[slot] = 0;
    return TQH_OK;
}

// Pages for new_tokens[i] more tokens in slots[i], for all rows or for none.
TQH_API int tqh_reserve(TqhBook* b, int n, const int* slots, const int* new_tokens) {
    b->scratch.assign(b->slots.n, 0);
    for (int i = 0; i < n; ++i) {
        const int s = slots[i];
        if (!b->slots.is_held(s)) return b->fail(TQH_CACHE, "slot %d is not held", s);
        if (b->scratch[s]++) return b->fail(TQH_CACHE, "a slot is named twice in one step: %d", s);
        if (new_tokens[i] <= 0) return b->fail(TQH_CACHE, "slot %d: a step must bring at least one token", s);
        if ((long long)b->length[s] + new_tokens[i] > b->max_length)
            return b->fail(TQH_CACHE, "slot %d: %d cached + %d new tokens exceed the context limit %d", s, b->length[s],
                           new_tokens[i], b->max_length);
    }
    for (const Group& g : b->groups) {         // every group's pool is checked before a page is taken
        long long want = 0;
        for (int i = 0; i < n; ++i) want += g.need(slots[i], b->length[slots[i]] + new_tokens[i]);
        if (want > g.pool.free_count())
            return b->fail(TQH_CACHE,
                           "cache group '%s' is full: the step needs %lld more pages of %d tokens, %d of %d are free",
                           g.name.c_str(), want, g.page_tokens, g.pool.free_count(), g.pool.n);
    }
    for (Group& g : b->groups)
        for (int i = 0; i < n; ++i) {
            const int s = slots[i];
            for (int k = g.need(s, b->length[s] + new_tokens[i]); k > 0; --k) {
                const int p = g.pool.take();
                if (p < 0) return b->fail(TQH_BROKEN, "cache group '%s': a page would be held twice", g.name.c_str());
                g.pages[s].push_back(p);
            }
        }
    return TQH_OK;
}

TQH_API int tqh_commit(TqhBook* b, int n, const int* slots, const int* new_tokens) {
    for (int i = 0; i < n; ++i)
        if (b->slots.is_held(slots[i])) b->length[slots[i]] += new_tokens[i];
    return TQH_OK;
}

// Gives back the pages of `slots` beyond what their committed lengths need (pages reserved for a step that did
// not happen).
TQH_API int tqh_trim(TqhBook* b, int n, const int* slots) {
    for (int i = 0; i < n; ++i) {
        const int s = slots[i];
        if (!b->slots.is_held(s)) continue;
        for (Group& g : b->groups) {
            const int keep = g.pages_for_length(b->length[s]);
            while ((int)g.pages[s].size() > keep) {
                if (g.pool.give_back(g.pages[s].back()) != 0)
                    return b->fail(TQH_BROKEN, "cache group '%s': a page is freed twice", g.name.c_str());
                g.pages[s].pop_back();
            }
        }
    }
    return TQH_OK;
}

TQH_API int tqh_length(const TqhBook* b, int slot) { return b->slots.is_held(slot) ? b->length[slot] : -1; }
// The lengths of n slots at once (-1 for one that is not held).
TQH_API int tqh_lengths(const TqhBook* b, int n, const int* slots, int* out) {
    for (int i = 0; i < n; ++i) out[i] = b->slots.is_held(slots[i]) ? b->length[slots[i]] : -1;
    return 0;
}
TQH_API int tqh_is_held(const TqhBook* b, int slot) { return b->slots.is_held(slot) ? 1 : 0; }
TQH_API int tqh_free_slots(const TqhBook* b) { return b->slots.free_count(); }
TQH_API int tqh_free_pages(const TqhBook* b, int group) { return b->groups[group].pool.free_count(); }
TQH_API int tqh_total_pages(const TqhBook* b, int group) { return b->groups[group].pool.n; }
TQH_API int tqh_page_count(const TqhBook* b, int group, int slot) {
    return b->slots.is_held(slot) ? (int)b->groups[group].pages[slot].size() : 0;
}
// The slot's physical pages in `group`, in logical order; returns how many there are (at most `cap` are written).
TQH_API int tqh_pages(const TqhBook* b, int group, int slot, int* out, int cap) {
    if (slot < 0 || slot >= b->slots.n) return 0;
    const std::vector<int>& p = b->groups[group].pages[slot];
    for (int i = 0; i < (int)p.size() && i < cap; ++i) out[i] = p[i];
    return (int)p.size();
}

// Invariants: every slot and page is either free or held, never both or neither; a page is held by one slot
// only, and only by a slot that is held; every held sequence has the pages its length needs.
TQH_API int tqh_check(TqhBook* b) {
    auto pool_ok = [&](const Pool& p, const char* what, const char* name) {
        std::vector<char> free_mark(p.n, 0);
        for (int i : p.free_desc) {
            if (i < 0 || i >= p.n || free_mark[i]) return b->fail(TQH_BROKEN, "a %s%s is on the free list twice", what, name);
            free_mark[i] = 1;
        }
        for (int i = 0; i < p.n; ++i)
            if ((free_mark[i] != 0) == (p.held[i] != 0))
                return b->fail(TQH_BROKEN, "%s%s %d is %s", what, name, i, p.held[i] ? "both free and held" : "lost");
        return (int)TQH_OK;
    };
    int r = pool_ok(b->slots, "slot", "");
    if (r) return r;
    for (const Group& g : b->groups) {
        r = pool_ok(g.pool, "page of cache group ", g.name.c_str());
        if (r) return r;
        std::vector<char> seen(g.pool.n, 0);
        int n_seen = 0;
        for (int s = 0; s < b->slots.n; ++s) {
            if (!g.pages[s].empty() && !b->slots.is_held(s))
                return b->fail(TQH_BROKEN, "group '%s' keeps pages for slot %d, which is not held", g.name.c_str(), s);
            for (int p : g.pages[s]) {
                if (p < 0 || p >= g.pool.n || seen[p] || !g.pool.held[p])
                    return b->fail(TQH_BROKEN, "group '%s': page %d is held twice or not marked held", g.name.c_str(), p);
                seen[p] = 1;
                ++n_seen;
            }
            if (b->slots.is_held(s) && (int)g.pages[s].size() < g.pages_for_length(b->length[s]))
                return b->fail(TQH_BROKEN, "group '%s': slot %d holds %d pages, its %d tokens need %d", g.name.c_str(), s,
                               (int)g.pages[s].size(), b->length[s], g.pages_for_length(b->length[s]));
        }
        if (n_seen != g.pool.n - g.pool.free_count())
            return b->fail(TQH_BROKEN, "group '%s': %d pages are lost", g.name.c_str(), g.pool.n - g.pool.free_count() - n_seen);
    }
    return TQH_OK;
}

// ---- a step's rows ------------------------------------------------------------------
// Rows are given flat: lens[i] tokens of row i follow one another in `tokens`, want_counts[i] places in `want`;
// sources[i] >= 0 names the row of the sampler's ids on the device that holds row i's one token (-1: none).

// The checks of a step that need no device: every row brings tokens, ids lie in the vocabulary, wanted places
// among the tokens brought, slots held; then the pages (tqh_reserve: all rows or none).
TQH_API int tqh_begin_step(TqhBook* b, int n_rows, const int* slots, const int* lens, const int* tokens,
                           const int* want_counts, const int* want, const int* sources, int vocab, int source_rows) {
    if (n_rows <= 0) return b->fail(TQH_STEP, "a step needs at least one row");
    int t0 = 0, w0 = 0;
    for (int i = 0; i < n_rows; ++i) {
        const int s = slots[i], n = lens[i];
        if (n <= 0) return b->fail(TQH_STEP, "slot %d: Empty prompt", s);
        if (sources && sources[i] >= 0) {
            if (n != 1 || sources[i] >= source_rows)
                return b->fail(TQH_STEP, "slot %d: a row fed from the sampler brings exactly one token", s);
        } else {
            for (int j = 0; j < n; ++j)
                if (tokens[t0 + j] < 0 || tokens[t0 + j] >= vocab)
                    return b->fail(TQH_STEP, "slot %d: token id %d is outside the vocabulary (0..%d)", s, tokens[t0 + j], vocab - 1);
        }
        for (int j = 0; j < want_counts[i]; ++j)
            if (want[w0 + j] < 0 || want[w0 + j] >= n)
                return b->fail(TQH_STEP, "slot %d: wanted place %d is outside the %d tokens brought", s, want[w0 + j], n);
        if (!b->slots.is_held(s)) return b->fail(TQH_STEP, "slot %d is not held", s);
        t0 += n;
        w0 += want_counts[i];
    }
    return TQH_OK;
}

// Layout of the packed buffer: tokens | tok_seq | tok_pos | cu_seqlens | slots | start_pos | new_lens | logit_rows
// | tok_src | one block table per cache group (rows of widths[g] entries); every segment starts on a 16-byte
// boundary.  Writes 9 + groups offsets and the table widths (the widest page list of the rows, at least 1);
// returns the buffer's length in int32 words.
TQH_API int tqh_step_layout(const TqhBook* b, int n_rows, const int* slots, const int* lens, const int* want_counts,
                            int* offs, int* widths) {
    int T = 0, R = 0;
    for (int i = 0; i < n_rows; ++i) { T += lens[i]; R += want_counts[i]; }
    const int G = (int)b->groups.size();
    int total = 0, k = 0;
    const int seg[9] = {T, T, T, n_rows + 1, n_rows, n_rows, n_rows, R, T};
    for (int i = 0; i < 9; ++i) { offs[k++] = total; total += pad4(std::max(seg[i], 1)); }
    for (int g = 0; g < G; ++g) {
        int w = 1;
        for (int i = 0; i < n_rows; ++i)
            if (slots[i] >= 0 && slots[i] < b->slots.n) w = std::max(w, (int)b->groups[g].pages[slots[i]].size());
        widths[g] = w;
        offs[k++] = total;
        total += pad4(n_rows * w);
    }
    return total;
}

// Fills the buffer (already sized by tqh_step_layout; the caller zeroes nothing: every word of every segment is
// written) for rows whose pages are reserved; positions follow the committed lengths.
TQH_API int tqh_pack_step(const TqhBook* b, int n_rows, const int* slots, const int* lens, const int* tokens,
                          const int* want_counts, const int* want, const int* sources, const int* offs,
                          const int* widths, int total, int32_t* buf) {
    std::memset(buf, 0, (size_t)total * sizeof(int32_t));
    int t0 = 0, w0 = 0, r = 0;
    buf[offs[3]] = 0;
    for (int i = 0; i < n_rows; ++i) {
        const int s = slots[i], n = lens[i], start = b->length[s];
        for (int j = 0; j < n; ++j) {
            buf[offs[0] + t0 + j] = tokens[t0 + j];
            buf[offs[1] + t0 + j] = i;
            buf[offs[2] + t0 + j] = start + j;
            buf[offs[8] + t0 + j] = -1;
        }
        if (sources && sources[i] >= 0) buf[offs[8] + t0] = sources[i];
        buf[offs[3] + i + 1] = t0 + n;
        buf[offs[4] + i] = s;
        buf[offs[5] + i] = start;
        buf[offs[6] + i] = start + n;
        for (int j = 0; j < want_counts[i]; ++j) buf[offs[7] + r++] = t0 + want[w0 + j];
        t0 += n;
        w0 += want_counts[i];
    }
    for (int g = 0; g < (int)b->groups.size(); ++g) {
        const int w = widths[g];
        for (int i = 0; i < n_rows; ++i) {
            const std::vector<int>& p = b->groups[g].pages[slots[i]];
            std::copy(p.begin(), p.begin() + std::min<int>((int)p.size(), w), buf + offs[9 + g] + (size_t)i * w);
        }
    }
    return TQH_OK;
}

// The same for a decode step of B rows of one token each, into a buffer whose layout is fixed (offs and widths
// of B rows with every row wanted, as tqh_step_layout gives them for full-width tables): only what changes from
// step to step is written — tokens, sources, positions, slots, lengths and the block tables.
TQH_API int tqh_pack_decode(const TqhBook* b, int B, const int* slots, const int* tokens, const int* sources,
                            const int* offs, const int* widths, int32_t* buf) {
    for (int i = 0; i < B; ++i) {
        const int s = slots[i];
        if (!b->slots.is_held(s)) return const_cast<TqhBook*>(b)->fail(TQH_STEP, "slot %d is not held", s);
        const int start = b->length[s];
        buf[offs[0] + i] = tokens[i];
        buf[offs[8] + i] = sources ? sources[i] : -1;
        buf[offs[2] + i] = start;
        buf[offs[4] + i] = s;
        buf[offs[5] + i] = start;
        buf[offs[6] + i] = start + 1;
    }
    for (int g = 0; g < (int)b->groups.size(); ++g) {
        const int w = widths[g];
        for (int i = 0; i < B; ++i) {
            const std::vector<int>& p = b->groups[g].pages[slots[i]];
            if ((int)p.size() > w)
                return const_cast<TqhBook*>(b)->fail(TQH_STEP, "slot %d holds %d pages of group '%s', the table has room for %d",
                                                     slots[i], (int)p.size(), b->groups[g].name.c_str(), w);
            std::copy(p.begin(), p.end(), buf + offs[9 + g] + (size_t)i * w);
        }
    }
    return TQH_OK;
}
