// Host-side cache manager (see manager.hpp).  Reference: combs-models/src/kv.rs.
#include "manager.hpp"

#include <algorithm>
#include <cstdio>
#include <cstring>

namespace cbkv {

static thread_local std::string g_err;
void set_error(const std::string& msg) { g_err = msg; }
void set_error_nothrow(const char* msg) noexcept {
    try { g_err = msg; } catch (...) { g_err.clear(); }  // clear() cannot throw
}
const char* last_error() { return g_err.c_str(); }

void Allocator::init(int64_t n) {
    // Reversed so page 0 is allocated first (kv.rs:424-429).
    initial_.resize((size_t)n);
    for (int64_t i = 0; i < n; i++) initial_[(size_t)i] = n - 1 - i;
    free_ = initial_;
}

bool Allocator::set_initial(const int64_t* ids, int64_t n) {
    if (n != (int64_t)initial_.size() || free_.size() != initial_.size()) return false;
    std::vector<char> seen((size_t)n, 0);
    for (int64_t i = 0; i < n; i++) {
        if (ids[i] < 0 || ids[i] >= n || seen[(size_t)ids[i]]) return false;
        seen[(size_t)ids[i]] = 1;
    }
    for (int64_t i = 0; i < n; i++) initial_[(size_t)(n - 1 - i)] = ids[i];
    free_ = initial_;
    return true;
}

int32_t arena_create(const cbkv_config* c, Arena** out) {
    if (!c || !out) { set_error("null argument"); return CBKV_ERR_ARG; }
    if (c->num_layers <= 0 || c->n_q_heads <= 0 || c->n_kv_heads <= 0 || c->head_dim <= 0 ||
        c->page_size <= 0 || c->max_seq_len <= 0 || c->num_pages < 0) {
        set_error("invalid cache geometry"); return CBKV_ERR_ARG;
    }
    if (c->n_q_heads % c->n_kv_heads != 0) { set_error("n_q_heads must be a multiple of n_kv_heads"); return CBKV_ERR_ARG; }
    if (c->head_dim % 8 != 0) { set_error("head_dim must be a multiple of 8 (16-byte rows)"); return CBKV_ERR_ARG; }
    if (c->dtype != CBKV_F16 && c->dtype != CBKV_BF16) { set_error("dtype must be CBKV_F16 or CBKV_BF16"); return CBKV_ERR_ARG; }
    if (c->max_seq_len > (int64_t)1 << 30) { set_error("max_seq_len too large"); return CBKV_ERR_ARG; }
    Arena* a = new Arena();
    a->cfg = *c;
    a->windows.assign((size_t)c->num_layers, 0);
    if (c->layer_windows) {
        for (int i = 0; i < c->num_layers; i++) {
            int64_t w = c->layer_windows[i];
            if (w != 0 && w < 2) {  // kv.rs:514-516
                set_error("sliding window must be >= 2, got " + std::to_string(w));
                delete a; return CBKV_ERR_ARG;
            }
            a->windows[(size_t)i] = w;
        }
    }
    a->cfg.layer_windows = nullptr;  // owned copy lives in `windows`
    a->num_pages = c->num_pages > 0 ? c->num_pages : (c->max_seq_len + c->page_size - 1) / c->page_size;  // kv.rs:82-84
    if (a->num_pages > (int64_t)1 << 30) { set_error("num_pages too large"); delete a; return CBKV_ERR_ARG; }
    a->alloc.init(a->num_pages);
    a->refcnt.assign((size_t)a->num_pages, 0);
    *out = a;
    return CBKV_OK;
}

int32_t seq_create(Arena* a, Seq** out) {
    if (!a || !out) { set_error("null argument"); return CBKV_ERR_ARG; }
    Seq* s = new Seq();
    s->arena = a;
    a->seqs.push_back(s);
    *out = s;
    return CBKV_OK;
}

// Drop the last table entry; the page returns to the free stack when its last
// holder lets go (one holder: exactly kv.rs:830-833).
static void table_pop_release(Seq* s) {
    int64_t page = s->table.back();
    s->table.pop_back();
    if (--s->arena->refcnt[(size_t)page] == 0) s->arena->alloc.free_page(page);
}

int32_t seq_destroy(Seq* s) {
    if (!s) return CBKV_OK;
    Arena* a = s->arena;
    if (a->step_open && std::find(a->step_seqs.begin(), a->step_seqs.end(), s) != a->step_seqs.end()) {
        a->step_open = false;  // the step's tables no longer describe live sequences
    }
    while (!s->table.empty()) table_pop_release(s);
    a->seqs.erase(std::remove(a->seqs.begin(), a->seqs.end(), s), a->seqs.end());
    delete s;
    return CBKV_OK;
}

int32_t seq_fork_prefix(Seq* parent, int64_t n_tokens, Seq** out) {
    if (!parent || !out) { set_error("null argument"); return CBKV_ERR_ARG; }
    Arena* a = parent->arena;
    if (n_tokens < 0 || n_tokens > parent->seq_len || n_tokens % a->cfg.page_size != 0) {
        set_error("fork_prefix: prefix must be whole pages within the parent"); return CBKV_ERR_ARG;
    }
    Seq* c = nullptr;
    seq_create(a, &c);
    int64_t pages = n_tokens / a->cfg.page_size;
    c->table.assign(parent->table.begin(), parent->table.begin() + pages);
    for (int64_t p : c->table) a->refcnt[(size_t)p]++;
    c->seq_len = n_tokens;
    *out = c;
    return CBKV_OK;
}

int32_t begin_step(Arena* a, Seq* const* seqs, const int64_t* new_tokens, const int64_t* pos, int32_t n) {
    if (!a || (n > 0 && (!seqs || !new_tokens)) || n < 0) { set_error("null argument"); return CBKV_ERR_ARG; }
    const int64_t P = a->cfg.page_size;
    int64_t pages_wanted = 0, tokens = 0;
    const uint64_t mark = ++a->mark_gen;  // a sequence seen in this call carries the call's mark
    // validate everything first: state is only mutated when the whole step fits
    for (int32_t b = 0; b < n; b++) {
        Seq* s = seqs[b];
        if (!s || s->arena != a) { set_error("sequence does not belong to this arena"); return CBKV_ERR_ARG; }
        if (s->mark == mark) { set_error("sequence listed twice in one step"); return CBKV_ERR_ARG; }
        s->mark = mark;
        if (new_tokens[b] < 1) { set_error("new_tokens must be >= 1"); return CBKV_ERR_ARG; }
        if (pos && pos[b] != s->seq_len) {  // kv.rs:671-674
            set_error("paged cache expects dense contiguous appends (pos == seq_len)"); return CBKV_ERR_POS;
        }
        int64_t total = s->seq_len + new_tokens[b];
        if (total > a->cfg.max_seq_len) {  // kv.rs:679-683
            set_error("paged cache capacity exceeded: " + std::to_string(total) + " > " + std::to_string(a->cfg.max_seq_len));
            return CBKV_ERR_CAPACITY;
        }
        if (s->seq_len % P != 0 && a->refcnt[(size_t)s->table[(size_t)(s->seq_len / P)]] > 1) {
            set_error("append would write into a page shared with another sequence"); return CBKV_ERR_STATE;
        }
        int64_t need = (total + P - 1) / P;
        pages_wanted += std::max<int64_t>(0, need - (int64_t)s->table.size());
        tokens += new_tokens[b];
    }
    if (pages_wanted > a->alloc.num_free()) {  // kv.rs:552-555
        set_error("page allocator exhausted (max_seq_len exceeded)"); return CBKV_ERR_EXHAUSTED;
    }
    if (tokens > (int64_t)1 << 30) { set_error("step too large"); return CBKV_ERR_ARG; }

    a->step_seqs.assign(seqs, seqs + n);
    a->step_meta.resize((size_t)n);
    a->step_tables.clear();
    a->step_is_decode = n > 0;
    int64_t tok_off = 0;
    for (int32_t b = 0; b < n; b++) {
        Seq* s = seqs[b];
        int64_t total = s->seq_len + new_tokens[b];
        int64_t need = (total + P - 1) / P;
        while ((int64_t)s->table.size() < need) {  // ensure_pages, kv.rs:549-559
            int64_t p = a->alloc.alloc();
            a->refcnt[(size_t)p] = 1;
            s->table.push_back(p);
        }
        SeqMeta& m = a->step_meta[(size_t)b];
        m.pos = (int32_t)s->seq_len;
        m.snew = (int32_t)new_tokens[b];
        m.tok_off = (int32_t)tok_off;
        m.tbl_off = (int32_t)a->step_tables.size();
        for (int64_t p : s->table) a->step_tables.push_back((int32_t)p);
        s->seq_len = total;  // kv.rs:675
        tok_off += new_tokens[b];
        if (new_tokens[b] != 1) a->step_is_decode = false;
    }
    a->step_tokens = tok_off;
    a->step_open = true;
    a->step_id++;
    return CBKV_OK;
}

int32_t popn(Seq* s, int64_t n, int64_t* popped) {
    if (!s || !popped) { set_error("null argument"); return CBKV_ERR_ARG; }
    Arena* a = s->arena;
    *popped = 0;
    n = std::min(n, s->seq_len);  // kv.rs:808
    if (n <= 0) return CBKV_OK;
    if (a->cfg.sliding_popn_refuses) {
        for (int64_t w : a->windows)
            if (w > 0 && s->seq_len > w - 1) return CBKV_OK;  // kv.rs:812-816: eviction would have happened
    }
    const int64_t P = a->cfg.page_size;
    int64_t new_len = s->seq_len - n;
    int64_t keep = (new_len + P - 1) / P;
    // A rollback may not end inside a page other sequences also hold: the next
    // append would overwrite their rows.  Refused, state untouched.
    if (new_len % P != 0 && a->refcnt[(size_t)s->table[(size_t)(keep - 1)]] > 1) return CBKV_OK;
    s->seq_len = new_len;                                  // kv.rs:828
    while ((int64_t)s->table.size() > keep) table_pop_release(s);  // kv.rs:829-833
    if (a->step_open && std::find(a->step_seqs.begin(), a->step_seqs.end(), s) != a->step_seqs.end())
        a->step_open = false;
    *popped = n;
    return CBKV_OK;
}

int32_t reset(Seq* s) {
    if (!s) { set_error("null argument"); return CBKV_ERR_ARG; }
    Arena* a = s->arena;
    if (a->seqs.size() == 1) {  // kv.rs:837-846: table cleared, allocator rebuilt
        for (int64_t p : s->table) a->refcnt[(size_t)p] = 0;
        s->table.clear();
        a->alloc.reset();
    } else {
        while (!s->table.empty()) table_pop_release(s);
    }
    s->seq_len = 0;
    a->step_open = false;
    return CBKV_OK;
}

void page_stats(const Seq* s, int64_t layers_materialized, cbkv_page_stats_t* out) {  // kv.rs:535-546
    const Arena* a = s->arena;
    out->pages_used = (int64_t)s->table.size();
    out->pages_free = a->alloc.num_free();
    out->num_pages = a->num_pages;
    out->page_size = a->cfg.page_size;
    out->seq_len = s->seq_len;
    out->layers_materialized = layers_materialized;
    out->layers_total = a->cfg.num_layers;
    out->layers_sliding = 0;  // windows are masks over pages here; no rolling stores exist
}

void build_decode_plan(const Arena& a, int64_t window, int32_t n_ctas, const DecodeSplit& split, DecodePlan* pl) {
    const int64_t P = a.cfg.page_size;
    const int Hkv = a.cfg.n_kv_heads;
    const int n = (int)a.step_meta.size();
    pl->window = window;
    pl->n_segs = n * Hkv;
    pl->segs.assign((size_t)pl->n_segs + 1, SegInfo{});
    int64_t units = 0;
    for (int b = 0; b < n; b++) {
        const SeqMeta& m = a.step_meta[(size_t)b];
        int64_t L = (int64_t)m.pos + m.snew;
        int64_t q_pos = L - 1;                                   // the single decode query
        int64_t lo_key = window > 0 ? std::max<int64_t>(0, q_pos - window + 1) : 0;  // keys in (p - w, p], kv.rs:112-115
        int64_t p_lo = lo_key / P, p_hi = q_pos / P;
        for (int h = 0; h < Hkv; h++) {
            SegInfo& sg = pl->segs[(size_t)b * Hkv + h];
            sg.unit_begin = (int32_t)units;
            sg.page_lo = (int32_t)p_lo;
            sg.q_pos = (int32_t)q_pos;
            sg.tok_off = m.tok_off;
            sg.nparts = 0;
            sg.part_base = -1;
            sg.tbl_off = m.tbl_off;
            units += p_hi - p_lo + 1;
        }
    }
    pl->segs[(size_t)pl->n_segs].unit_begin = (int32_t)units;
    pl->n_units = (int32_t)units;
    n_ctas = (int32_t)std::max<int64_t>(1, std::min<int64_t>(n_ctas, units));
    pl->n_ctas = n_ctas;

    // Levels of the tail, decided on the shortest range so that every range has the same number of items.
    const int64_t lmin = units / n_ctas;
    int levels = 1;
    {
        const int64_t tail = lmin * split.tail_pct / 100;
        if (split.min_item > 0 && tail >= split.min_item) {
            int pieces = 1;
            while (pieces + 1 < split.max_levels && (tail >> pieces) >= split.min_item) pieces++;
            levels = 1 + pieces;
        }
    }
    pl->levels = levels;
    pl->n_items = n_ctas * levels;
    pl->items.assign((size_t)pl->n_items, ItemInfo{});
    // item (level j, range c) sits at claim index j * n_ctas + c; inside a range the levels follow each other
    for (int c = 0; c < n_ctas; c++) {
        const int64_t rb = units * c / n_ctas, re = units * (c + 1) / n_ctas;
        const int64_t len = re - rb;
        int64_t rest = levels > 1 ? len * split.tail_pct / 100 : 0;
        int64_t at = rb;
        for (int j = 0; j < levels; j++) {
            int64_t take;
            if (j == 0) take = len - rest;
            else if (j == levels - 1) take = rest;
            else take = (rest + 1) / 2;
            if (j > 0) rest -= take;
            ItemInfo& it = pl->items[(size_t)j * n_ctas + c];
            it.u_begin = (int32_t)at;
            it.u_end = (int32_t)(at + take);
            at += take;
        }
    }
    // parts of every segment: sweep the items in unit order (range by range, level by level)
    std::vector<int32_t> order;
    order.reserve((size_t)pl->n_items);
    for (int c = 0; c < n_ctas; c++)
        for (int j = 0; j < levels; j++)
            if (pl->items[(size_t)j * n_ctas + c].u_end > pl->items[(size_t)j * n_ctas + c].u_begin) order.push_back(j * n_ctas + c);
    size_t io = 0;
    int parts = 0;
    for (int s = 0; s < pl->n_segs; s++) {
        SegInfo& sg = pl->segs[(size_t)s];
        const int32_t sb = sg.unit_begin, se = pl->segs[(size_t)s + 1].unit_begin;
        if (se == sb) continue;
        while (io < order.size() && pl->items[(size_t)order[io]].u_end <= sb) io++;
        int cnt = 0;
        for (size_t k = io; k < order.size() && pl->items[(size_t)order[k]].u_begin < se; k++) {
            ItemInfo& it = pl->items[(size_t)order[k]];
            if (it.u_begin >= sb) { it.first_seg = s; it.first_part = cnt; }
            cnt++;
        }
        sg.nparts = cnt;
        if (cnt > 1) { sg.part_base = parts; parts += cnt; }
    }
    pl->n_parts = parts;
    for (ItemInfo& it : pl->items)  // empty items (possible only when units < items) are never claimed usefully
        if (it.u_end <= it.u_begin) { it.first_seg = 0; it.first_part = 0; }
}

void build_chunk_plan(const Arena& a, int32_t cols_per_item, ChunkPlan* pl) {
    const int n = (int)a.step_meta.size();
    pl->cols_per_item = cols_per_item;
    pl->item_begin.assign((size_t)n + 1, 0);
    int64_t items = 0;
    for (int b = 0; b < n; b++) {
        pl->item_begin[(size_t)b] = (int32_t)items;
        int64_t cols = (int64_t)a.step_meta[(size_t)b].snew * a.n_rep();
        items += (int64_t)a.cfg.n_kv_heads * ((cols + cols_per_item - 1) / cols_per_item);
    }
    pl->item_begin[(size_t)n] = (int32_t)items;
    pl->n_items = (int32_t)items;
}

void build_chunk_tile_plan(const Arena& a, int32_t tokens_per_tile, ChunkPlan* pl) {
    const int n = (int)a.step_meta.size();
    pl->cols_per_item = tokens_per_tile;
    pl->item_begin.assign((size_t)n + 1, 0);
    int64_t items = 0;
    for (int b = 0; b < n; b++) {
        pl->item_begin[(size_t)b] = (int32_t)items;
        items += (int64_t)a.cfg.n_kv_heads * ((a.step_meta[(size_t)b].snew + tokens_per_tile - 1) / tokens_per_tile);
    }
    pl->item_begin[(size_t)n] = (int32_t)items;
    pl->n_items = (int32_t)items;
}

}  // namespace cbkv
