/*
 * kv_oracle.c — CPU restatement of CombsEngine's paged KV cache + attention.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA path is compared
 * against and the CPU baseline that gets timed next to it.  Nothing in the
 * product library links, imports or calls it.
 *
 * Every function restates one piece of the reference file
 *   engine/core/combs-models/src/kv.rs
 * and cites the lines it follows.  The arithmetic of the reference lives in
 * un-vendored crates (burn 0.21.0 / burn-ndarray 0.21.0, matrixmultiply 0.3.11);
 * what is restated here is the published algorithm of those ops: row-major
 * matmul with f32 accumulation, `mask_fill(-1e30)`, `softmax` = exp(x - max) /
 * sum, casts to and from f16.
 *
 * Pinning status:
 *   - integer / state results (allocator order, page counts, free counts,
 *     seq_len after popn / reset) are pinned by the reference's own
 *     known-answer tests (kv.rs:1075-1192, tests/kv_cache.rs) — see
 *     tests/test_oracle_reference_kats.py;
 *   - floating-point attention outputs: the reference stores no golden output
 *     vectors for this path, only cross-implementation equivalences
 *     (paged == contiguous within 1e-4, sliding == masked-global within 1e-5).
 *     The oracle satisfies those equivalences and is additionally checked
 *     against an independent float64 implementation; in the strict
 *     golden-vector sense its floating-point parity is UNPINNED.
 *
 * Build twice from this one source:
 *   default        elem = float     (the reference's NdArray<f32> test build)
 *   -DORC_F16      elem = IEEE half (the reference's `--features f16` build:
 *                  f16 storage, f32 scores/softmax/accumulation, kv.rs:210-215)
 *
 * Extensions that the reference does not have (one cache = one sequence =
 * one private arena there, kv.rs:452-454) are marked EXTENSION; each is
 * defined so that a single sequence in a fresh arena behaves exactly like a
 * reference `PagedKVCache`.
 */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#ifdef ORC_F16
typedef uint16_t elem_t;
static inline float ld(elem_t x) { _Float16 h; memcpy(&h, &x, 2); return (float)h; }
static inline elem_t st(float f) { _Float16 h = (_Float16)f; elem_t x; memcpy(&x, &h, 2); return x; }
#define ORC_ELEM_BYTES 2
#else
typedef float elem_t;
static inline float ld(elem_t x) { return x; }
static inline elem_t st(float f) { return f; }
#define ORC_ELEM_BYTES 4
#endif

#define ORC_OK 0
#define ORC_ERR_POS -1       /* kv.rs:671-674 */
#define ORC_ERR_CAPACITY -2  /* kv.rs:679-683 */
#define ORC_ERR_EXHAUSTED -3 /* kv.rs:552-555 */
#define ORC_ERR_ARG -4

#ifdef _OPENMP
#include <omp.h>
#endif

static __thread char g_err[256];
const char* orc_last_error(void) { return g_err; }
int orc_elem_bytes(void) { return ORC_ELEM_BYTES; }
/* Threads of the batch driver (the launcher may have pinned OMP_NUM_THREADS to 1). */
int orc_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ---------------------------------------------------------------- allocator
 * PageAllocator, kv.rs:417-446: a stack of page ids; `new` pushes n-1..0 so
 * that `alloc` (pop) yields 0,1,2,...; `free_page` pushes; `reset` rebuilds.  */
typedef struct {
    int64_t* free;     /* stack, top at free[n_free-1] */
    int64_t n_free;
    int64_t* initial;  /* EXTENSION: seeded initial stack order (set_free_list) */
    int64_t num_pages;
} orc_alloc;

static void alloc_init(orc_alloc* a, int64_t n) {
    a->num_pages = n;
    a->free = (int64_t*)malloc(sizeof(int64_t) * (size_t)(n > 0 ? n : 1));
    a->initial = (int64_t*)malloc(sizeof(int64_t) * (size_t)(n > 0 ? n : 1));
    for (int64_t i = 0; i < n; i++) a->initial[i] = n - 1 - i; /* (0..n).rev(), kv.rs:427 */
    memcpy(a->free, a->initial, sizeof(int64_t) * (size_t)n);
    a->n_free = n;
}
static int64_t alloc_pop(orc_alloc* a) { return a->n_free ? a->free[--a->n_free] : -1; } /* kv.rs:431-433 */
static void alloc_push(orc_alloc* a, int64_t id) { a->free[a->n_free++] = id; }          /* kv.rs:435-437 */
static void alloc_reset(orc_alloc* a) {                                                   /* kv.rs:443-445 */
    memcpy(a->free, a->initial, sizeof(int64_t) * (size_t)a->num_pages);
    a->n_free = a->num_pages;
}

/* -------------------------------------------------------------------- arena */
typedef struct orc_seq orc_seq;
typedef struct {
    int layers, n_kv, d, page_size;
    int64_t max_seq_len; /* CacheConfig::max_seq_len, per-sequence capacity */
    int64_t num_pages;   /* CacheConfig::num_pages(), kv.rs:82-84, unless overridden (EXTENSION) */
    int64_t* windows;    /* per layer, 0 = global (kv.rs:489) */
    int rolling;         /* 1: sliding layers keep a rolling store and use no pages (kv.rs:561-609);
                            0: EXTENSION, sliding layers live in pages and the window is a mask
                               (the "masked global" of kv.rs:1006-1015) */
    orc_alloc alloc;
    elem_t** k;          /* per layer [num_pages, n_kv, page_size, d], lazily zero-allocated (kv.rs:695-713) */
    elem_t** v;
    int32_t* refcnt;     /* EXTENSION: holders per page (prefix sharing) */
    int live_seqs;
    /* CacheConfig::quantize_kv (kv.rs:464-475,694-705): int8 pages for the layers without a
       window of their own, when head_dim is a multiple of 32.  kp/vp hold the packed words
       [num_pages, n_kv, page_size, d/4], ksc/vsc the group scales [.., d/32]; k/v then hold the
       de-quantised values, which is what attention reads (kv.rs:771-780). */
    int quantize;
    int32_t** kp; int32_t** vp; elem_t** ksc; elem_t** vsc;
} orc_arena;

struct orc_seq {
    orc_arena* a;
    int64_t* table;      /* logical page -> physical page, kv.rs:481 */
    int64_t n_table, cap_table;
    int64_t seq_len;
    /* rolling K/V per sliding layer: [n_kv, len, d], kv.rs:490-493 */
    elem_t** sk; elem_t** sv; int64_t* slen;
};

orc_arena* orc_arena_new(int layers, int n_kv, int d, int64_t max_seq_len, int page_size,
                         int64_t num_pages, const int64_t* windows, int rolling) {
    if (layers <= 0 || n_kv <= 0 || d <= 0 || page_size <= 0 || max_seq_len <= 0) {
        snprintf(g_err, sizeof g_err, "invalid cache geometry"); return NULL;
    }
    if (windows) for (int i = 0; i < layers; i++) if (windows[i] != 0 && windows[i] < 2) {
        snprintf(g_err, sizeof g_err, "sliding window must be >= 2, got %lld", (long long)windows[i]); /* kv.rs:515 */
        return NULL;
    }
    orc_arena* a = (orc_arena*)calloc(1, sizeof *a);
    a->layers = layers; a->n_kv = n_kv; a->d = d; a->page_size = page_size;
    a->max_seq_len = max_seq_len;
    a->num_pages = num_pages > 0 ? num_pages : (max_seq_len + page_size - 1) / page_size;
    a->windows = (int64_t*)calloc((size_t)layers, sizeof(int64_t));
    if (windows) memcpy(a->windows, windows, sizeof(int64_t) * (size_t)layers);
    a->rolling = rolling;
    alloc_init(&a->alloc, a->num_pages);
    a->k = (elem_t**)calloc((size_t)layers, sizeof(elem_t*));
    a->v = (elem_t**)calloc((size_t)layers, sizeof(elem_t*));
    a->refcnt = (int32_t*)calloc((size_t)a->num_pages, sizeof(int32_t));
    a->kp = (int32_t**)calloc((size_t)layers, sizeof(int32_t*));
    a->vp = (int32_t**)calloc((size_t)layers, sizeof(int32_t*));
    a->ksc = (elem_t**)calloc((size_t)layers, sizeof(elem_t*));
    a->vsc = (elem_t**)calloc((size_t)layers, sizeof(elem_t*));
    return a;
}

void orc_arena_set_quantize(orc_arena* a, int on) { a->quantize = on; }

void orc_arena_free(orc_arena* a) {
    if (!a) return;
    for (int i = 0; i < a->layers; i++) { free(a->k[i]); free(a->v[i]); free(a->kp[i]); free(a->vp[i]); free(a->ksc[i]); free(a->vsc[i]); }
    free(a->k); free(a->v); free(a->kp); free(a->vp); free(a->ksc); free(a->vsc); free(a->windows); free(a->refcnt);
    free(a->alloc.free); free(a->alloc.initial); free(a);
}

/* EXTENSION: seeded initial free-list.  ids[0] is handed out first. */
int orc_set_free_list(orc_arena* a, const int64_t* ids, int64_t n) {
    if (n != a->num_pages || a->alloc.n_free != a->num_pages) {
        snprintf(g_err, sizeof g_err, "set_free_list needs a full permutation on an unused arena"); return ORC_ERR_ARG;
    }
    char* seen = (char*)calloc((size_t)n, 1);
    for (int64_t i = 0; i < n; i++) {
        if (ids[i] < 0 || ids[i] >= n || seen[ids[i]]) { free(seen); snprintf(g_err, sizeof g_err, "set_free_list: not a permutation"); return ORC_ERR_ARG; }
        seen[ids[i]] = 1;
    }
    free(seen);
    for (int64_t i = 0; i < n; i++) a->alloc.initial[n - 1 - i] = ids[i];
    alloc_reset(&a->alloc);
    return ORC_OK;
}

orc_seq* orc_seq_new(orc_arena* a) {
    orc_seq* s = (orc_seq*)calloc(1, sizeof *s);
    s->a = a;
    s->sk = (elem_t**)calloc((size_t)a->layers, sizeof(elem_t*));
    s->sv = (elem_t**)calloc((size_t)a->layers, sizeof(elem_t*));
    s->slen = (int64_t*)calloc((size_t)a->layers, sizeof(int64_t));
    a->live_seqs++;
    return s;
}

static void table_push(orc_seq* s, int64_t page) {
    if (s->n_table == s->cap_table) {
        s->cap_table = s->cap_table ? s->cap_table * 2 : 16;
        s->table = (int64_t*)realloc(s->table, sizeof(int64_t) * (size_t)s->cap_table);
    }
    s->table[s->n_table++] = page;
}

/* Drop the last table entry.  A page goes back on the free stack when its last
 * holder lets go (EXTENSION; with one holder this is kv.rs:830-833). */
static void table_pop_release(orc_seq* s) {
    int64_t page = s->table[--s->n_table];
    if (--s->a->refcnt[page] == 0) alloc_push(&s->a->alloc, page);
}

static void drop_sliding(orc_seq* s) {
    for (int i = 0; i < s->a->layers; i++) {
        free(s->sk[i]); free(s->sv[i]); s->sk[i] = s->sv[i] = NULL; s->slen[i] = 0;
    }
}

void orc_seq_free(orc_seq* s) {
    if (!s) return;
    while (s->n_table) table_pop_release(s);
    drop_sliding(s);
    free(s->sk); free(s->sv); free(s->slen); free(s->table);
    s->a->live_seqs--;
    free(s);
}

/* ensure_pages, kv.rs:549-559 */
static int ensure_pages(orc_seq* s, int64_t total, int64_t* pages_needed) {
    orc_arena* a = s->a;
    int64_t need = (total + a->page_size - 1) / a->page_size;
    /* all-or-nothing: the reference panics mid-way; a C caller needs the state intact */
    if (need - s->n_table > a->alloc.n_free) {
        snprintf(g_err, sizeof g_err, "page allocator exhausted (max_seq_len exceeded)");
        return ORC_ERR_EXHAUSTED;
    }
    while (s->n_table < need) {
        int64_t p = alloc_pop(&a->alloc);
        a->refcnt[p] = 1;
        table_push(s, p);
    }
    *pages_needed = need;
    return ORC_OK;
}

/* Test hook mirroring the reference's `grow()` helper (kv.rs:1134-1137). */
int orc_grow(orc_seq* s, int64_t total) {
    int64_t n; int rc = ensure_pages(s, total, &n);
    if (rc == ORC_OK) s->seq_len = total;
    return rc;
}

/* EXTENSION: cross-sequence prefix sharing.  The child aliases the parent's
 * first n_tokens / page_size pages (whole pages only). */
orc_seq* orc_seq_fork_prefix(orc_seq* parent, int64_t n_tokens) {
    orc_arena* a = parent->a;
    if (n_tokens < 0 || n_tokens > parent->seq_len || n_tokens % a->page_size != 0) {
        snprintf(g_err, sizeof g_err, "fork_prefix: prefix must be whole pages within the parent"); return NULL;
    }
    orc_seq* c = orc_seq_new(a);
    for (int64_t i = 0; i < n_tokens / a->page_size; i++) {
        a->refcnt[parent->table[i]]++;
        table_push(c, parent->table[i]);
    }
    c->seq_len = n_tokens;
    return c;
}

/* ---------------------------------------------------------------- attention */

/* attend(), manual branch, kv.rs:201-269, on one sequence.
 * q [n_q, seq, d]; k, v [n_kv, total, d] (already gathered); out [n_q, seq, d].
 * Steps kept as the reference performs them: upcast to f32 (kv.rs:213-215),
 * repeat_kv (kv.rs:219-220), scores = q k^T * scale (kv.rs:243), mask
 * (kv.rs:244-264), softmax over keys, P V (kv.rs:268), cast back. */
static void attend(const elem_t* q, const elem_t* k, const elem_t* v, elem_t* out,
                   int n_q, int n_kv, int64_t seq, int64_t total, int d,
                   int64_t pos, double scale, int64_t window) {
    int n_rep = n_q / n_kv;
    size_t kv_elems = (size_t)n_kv * (size_t)total * (size_t)d;
    float* kf = (float*)malloc(sizeof(float) * kv_elems);
    float* vf = (float*)malloc(sizeof(float) * kv_elems);
    for (size_t i = 0; i < kv_elems; i++) { kf[i] = ld(k[i]); vf[i] = ld(v[i]); }
    /* repeat_kv (kv.rs:177-187): q head h reads kv head h / n_rep; the expand is
       materialised like the reference does */
    float* kr = (float*)malloc(sizeof(float) * (size_t)n_q * (size_t)total * (size_t)d);
    float* vr = (float*)malloc(sizeof(float) * (size_t)n_q * (size_t)total * (size_t)d);
    for (int h = 0; h < n_q; h++) {
        memcpy(kr + (size_t)h * total * d, kf + (size_t)(h / n_rep) * total * d, sizeof(float) * (size_t)total * d);
        memcpy(vr + (size_t)h * total * d, vf + (size_t)(h / n_rep) * total * d, sizeof(float) * (size_t)total * d);
    }
    free(kf); free(vf);
    const float fscale = (float)scale;
    const int masked = (seq > 1) || (window > 0); /* kv.rs:244 */
#pragma omp parallel for schedule(dynamic) if (n_q * seq * total > 65536)
    for (int h = 0; h < n_q; h++) {
        float* qf = (float*)malloc(sizeof(float) * (size_t)d);
        float* sc = (float*)malloc(sizeof(float) * (size_t)total);
        float* acc = (float*)malloc(sizeof(float) * (size_t)d);
        for (int64_t r = 0; r < seq; r++) {
            const elem_t* qrow = q + ((size_t)h * seq + r) * d;
            for (int j = 0; j < d; j++) qf[j] = ld(qrow[j]);
            int64_t q_pos = pos + r;
            for (int64_t t = 0; t < total; t++) {
                const float* krow = kr + ((size_t)h * total + t) * d;
                float s = 0.f;
                for (int j = 0; j < d; j++) s += qf[j] * krow[j];
                s *= fscale;
                if (masked) {
                    int forbidden = t > q_pos;                                   /* kv.rs:251 */
                    if (window > 0 && t + window - 1 < q_pos) forbidden = 1;     /* kv.rs:252-257 */
                    if (forbidden) s = -1e30f;                                   /* kv.rs:261 */
                }
                sc[t] = s;
            }
            float mx = sc[0];
            for (int64_t t = 1; t < total; t++) mx = sc[t] > mx ? sc[t] : mx;
            float sum = 0.f;
            for (int64_t t = 0; t < total; t++) { sc[t] = expf(sc[t] - mx); sum += sc[t]; }
            float inv = 1.f / sum;
            for (int j = 0; j < d; j++) acc[j] = 0.f;
            for (int64_t t = 0; t < total; t++) {
                float p = sc[t] * inv;
                const float* vrow = vr + ((size_t)h * total + t) * d;
                for (int j = 0; j < d; j++) acc[j] += p * vrow[j];
            }
            elem_t* orow = out + ((size_t)h * seq + r) * d;
            for (int j = 0; j < d; j++) orow[j] = st(acc[j]);
        }
        free(qf); free(sc); free(acc);
    }
    free(kr); free(vr);
}

/* ------------------------------------------------------------ int8 KV pages
 * kv_quantize, kv.rs:284-313, for `rows` rows of d values (d % 32 == 0): per 32-value group
 * scale = max(absmax / 127, 1e-8) in f32, q = clamp(round(x / scale), -127, 127), four values
 * per word p = (q0+128) + (q1+128)*2^8 + (q2+128)*2^16 + q3*2^24; the scale is returned in the
 * element type (kv.rs:312). */
#define ORC_QGROUP 32
void orc_kv_quantize(const elem_t* x, int64_t rows, int d, int32_t* packed, elem_t* scales) {
    const int groups = d / ORC_QGROUP;
    for (int64_t r = 0; r < rows; r++)
        for (int g = 0; g < groups; g++) {
            const elem_t* src = x + r * d + g * ORC_QGROUP;
            float absmax = 0.f;
            for (int j = 0; j < ORC_QGROUP; j++) { float v = fabsf(ld(src[j])); absmax = v > absmax ? v : absmax; }
            float scale = absmax / 127.0f;
            if (scale < 1e-8f) scale = 1e-8f;
            int32_t q[ORC_QGROUP];
            for (int j = 0; j < ORC_QGROUP; j++) {
                float v = roundf(ld(src[j]) / scale);
                v = v < -127.f ? -127.f : (v > 127.f ? 127.f : v);
                q[j] = (int32_t)v;
            }
            for (int w = 0; w < ORC_QGROUP / 4; w++)
                packed[r * (d / 4) + g * (ORC_QGROUP / 4) + w] =
                    (q[4 * w] + 128) + (q[4 * w + 1] + 128) * 256 + (q[4 * w + 2] + 128) * 65536 + q[4 * w + 3] * 16777216;
            scales[r * groups + g] = st(scale);
        }
}

/* kv_dequantize, kv.rs:319-358: floor-division unpacking of the four lanes, then q * scale in
 * the element type. */
void orc_kv_dequantize(const int32_t* packed, const elem_t* scales, int64_t rows, int d, elem_t* out) {
    const int groups = d / ORC_QGROUP;
    for (int64_t r = 0; r < rows; r++)
        for (int w = 0; w < d / 4; w++) {
            int32_t p = packed[r * (d / 4) + w];
            int32_t t = p / 16777216;                 /* truncating division, kv.rs:326 */
            int32_t r3 = p - t * 16777216;
            int32_t q3 = r3 < 0 ? t - 1 : t;          /* kv.rs:328-329 */
            int32_t rem = r3 < 0 ? r3 + 16777216 : r3;
            int32_t l2 = rem / 65536; rem -= l2 * 65536;
            int32_t l1 = rem / 256;
            int32_t l0 = rem - l1 * 256;
            int32_t q[4] = {l0 - 128, l1 - 128, l2 - 128, q3};
            float sc = ld(scales[r * groups + (4 * w) / ORC_QGROUP]);
            for (int i = 0; i < 4; i++) out[r * d + 4 * w + i] = st(ld(st((float)q[i])) * sc);
        }
}

static int layer_is_quantized(const orc_arena* a, int layer) {
    return a->quantize && a->d % ORC_QGROUP == 0 && a->windows[layer] == 0; /* kv.rs:690-694 */
}

/* Packed words and scales of a quantised layer appear with the layer's arenas (kv.rs:699-705). */
static void ensure_quant_arrays(orc_arena* a, int layer) {
    if (!layer_is_quantized(a, layer) || a->kp[layer]) return;
    size_t n = (size_t)a->num_pages * a->n_kv * a->page_size;
    a->kp[layer] = (int32_t*)calloc(n * (size_t)(a->d / 4), sizeof(int32_t));
    a->vp[layer] = (int32_t*)calloc(n * (size_t)(a->d / 4), sizeof(int32_t));
    a->ksc[layer] = (elem_t*)calloc(n * (size_t)(a->d / ORC_QGROUP), sizeof(elem_t));
    a->vsc[layer] = (elem_t*)calloc(n * (size_t)(a->d / ORC_QGROUP), sizeof(elem_t));
}

/* One run of new rows of one head into a page: plain copy, or quantise + keep the packed form
 * and store what de-quantisation gives back (kv.rs:740-780). */
static void store_rows(orc_arena* a, int layer, int is_v, size_t dst_row, const elem_t* src, int64_t run) {
    const int d = a->d;
    elem_t* dst = (is_v ? a->v[layer] : a->k[layer]) + dst_row * d;
    if (!layer_is_quantized(a, layer)) { memcpy(dst, src, sizeof(elem_t) * (size_t)run * d); return; }
    int32_t** pk = is_v ? a->vp : a->kp;
    elem_t** sc = is_v ? a->vsc : a->ksc;
    orc_kv_quantize(src, run, d, pk[layer] + dst_row * (d / 4), sc[layer] + dst_row * (d / ORC_QGROUP));
    orc_kv_dequantize(pk[layer] + dst_row * (d / 4), sc[layer] + dst_row * (d / ORC_QGROUP), run, d, dst);
}

void orc_export_page_quant(const orc_arena* a, int layer, int64_t page, int32_t* kp, elem_t* ks, int32_t* vp, elem_t* vs) {
    size_t rows = (size_t)a->n_kv * a->page_size, d4 = (size_t)a->d / 4, dg = (size_t)a->d / ORC_QGROUP;
    if (a->kp[layer]) { memcpy(kp, a->kp[layer] + page * rows * d4, 4 * rows * d4); memcpy(ks, a->ksc[layer] + page * rows * dg, sizeof(elem_t) * rows * dg); }
    else { memset(kp, 0, 4 * rows * d4); memset(ks, 0, sizeof(elem_t) * rows * dg); }
    if (a->vp[layer]) { memcpy(vp, a->vp[layer] + page * rows * d4, 4 * rows * d4); memcpy(vs, a->vsc[layer] + page * rows * dg, sizeof(elem_t) * rows * dg); }
    else { memset(vp, 0, 4 * rows * d4); memset(vs, 0, sizeof(elem_t) * rows * dg); }
}

/* gather_window, kv.rs:624-636: select pages, swap to head-major, trim to total */
static elem_t* gather_window(const orc_seq* s, const elem_t* arena, int64_t pages, int64_t total) {
    const orc_arena* a = s->a;
    int P = a->page_size, d = a->d, H = a->n_kv;
    elem_t* w = (elem_t*)malloc(sizeof(elem_t) * (size_t)H * (size_t)total * (size_t)d);
    for (int64_t lp = 0; lp < pages; lp++) {
        int64_t phys = s->table[lp];
        for (int h = 0; h < H; h++)
            for (int slot = 0; slot < P; slot++) {
                int64_t t = lp * P + slot;
                if (t >= total) break;
                memcpy(w + ((size_t)h * total + t) * d,
                       arena + (((size_t)phys * H + h) * P + slot) * d, sizeof(elem_t) * (size_t)d);
            }
    }
    return w;
}

/* sliding_attention, kv.rs:570-609 (rolling store; only when a->rolling) */
static void sliding_attention(orc_seq* s, int layer, const elem_t* q, const elem_t* k, const elem_t* v,
                              elem_t* out, int n_q, int64_t seq, int64_t pos, double scale, int64_t w) {
    orc_arena* a = s->a;
    int H = a->n_kv, d = a->d;
    int64_t old = s->slen[layer], full = old + seq;
    elem_t* kf = (elem_t*)malloc(sizeof(elem_t) * (size_t)H * full * d);
    elem_t* vf = (elem_t*)malloc(sizeof(elem_t) * (size_t)H * full * d);
    for (int h = 0; h < H; h++) { /* cat along the sequence axis, kv.rs:582-588 */
        if (old) {
            memcpy(kf + (size_t)h * full * d, s->sk[layer] + (size_t)h * old * d, sizeof(elem_t) * (size_t)old * d);
            memcpy(vf + (size_t)h * full * d, s->sv[layer] + (size_t)h * old * d, sizeof(elem_t) * (size_t)old * d);
        }
        memcpy(kf + ((size_t)h * full + old) * d, k + (size_t)h * seq * d, sizeof(elem_t) * (size_t)seq * d);
        memcpy(vf + ((size_t)h * full + old) * d, v + (size_t)h * seq * d, sizeof(elem_t) * (size_t)seq * d);
    }
    int64_t kv_offset = pos + seq - full;                                   /* kv.rs:590 */
    attend(q, kf, vf, out, n_q, H, seq, full, d, pos - kv_offset, scale, w); /* kv.rs:591-598 */
    int64_t keep = full < w - 1 ? full : w - 1;                              /* kv.rs:603 */
    free(s->sk[layer]); free(s->sv[layer]);
    s->sk[layer] = (elem_t*)malloc(sizeof(elem_t) * (size_t)H * (keep ? keep : 1) * d);
    s->sv[layer] = (elem_t*)malloc(sizeof(elem_t) * (size_t)H * (keep ? keep : 1) * d);
    for (int h = 0; h < H; h++) {
        memcpy(s->sk[layer] + (size_t)h * keep * d, kf + ((size_t)h * full + (full - keep)) * d, sizeof(elem_t) * (size_t)keep * d);
        memcpy(s->sv[layer] + (size_t)h * keep * d, vf + ((size_t)h * full + (full - keep)) * d, sizeof(elem_t) * (size_t)keep * d);
    }
    s->slen[layer] = keep;
    free(kf); free(vf);
}

/* Layer-0 bookkeeping of attention_opts (kv.rs:665-683) split out so that a batch
 * of sequences can be advanced in sequence-index order before any layer runs
 * (EXTENSION: allocation order across sequences = call order). */
int orc_begin(orc_seq* s, int64_t pos, int64_t seq) {
    orc_arena* a = s->a;
    int64_t total = pos + seq;
    if (pos != s->seq_len) {
        snprintf(g_err, sizeof g_err, "paged cache expects dense contiguous appends (pos == seq_len)"); return ORC_ERR_POS;
    }
    if (total > a->max_seq_len) {
        snprintf(g_err, sizeof g_err, "paged cache capacity exceeded: %lld > %lld", (long long)total, (long long)a->max_seq_len);
        return ORC_ERR_CAPACITY;
    }
    /* pages are needed unless every layer is a rolling sliding layer */
    int any_paged = 0;
    for (int i = 0; i < a->layers; i++) if (!(a->rolling && a->windows[i] > 0)) any_paged = 1;
    if (any_paged) {
        int64_t n; int rc = ensure_pages(s, total, &n);
        if (rc != ORC_OK) return rc;
    }
    s->seq_len = total;
    return ORC_OK;
}

/* PagedKVCache::attention_opts for one layer after orc_begin, kv.rs:685-791.
 * q [n_q, seq, d]; k, v [n_kv, seq, d]; out [n_q, seq, d]. */
int orc_layer(orc_seq* s, int layer, const elem_t* q, const elem_t* k, const elem_t* v, elem_t* out,
              int n_q, int64_t seq, int64_t pos, double scale, int64_t window) {
    orc_arena* a = s->a;
    int H = a->n_kv, d = a->d, P = a->page_size;
    int64_t total = pos + seq;
    if (layer < 0 || layer >= a->layers || n_q % H != 0) { snprintf(g_err, sizeof g_err, "bad layer or head count"); return ORC_ERR_ARG; }
    if (total != s->seq_len) { snprintf(g_err, sizeof g_err, "layer call does not match the step begun"); return ORC_ERR_POS; } /* kv.rs:677 */
    /* the cache's own per-layer window wins over the argument, kv.rs:688-693 */
    int64_t lw = a->windows[layer];
    if (lw > 0 && a->rolling) { sliding_attention(s, layer, q, k, v, out, n_q, seq, pos, scale, lw); return ORC_OK; }
    if (lw > 0) window = lw;
    if (!a->k[layer]) { /* lazy zeroed arenas, kv.rs:695-713 */
        size_t n = (size_t)a->num_pages * H * P * d;
        a->k[layer] = (elem_t*)calloc(n, sizeof(elem_t));
        a->v[layer] = (elem_t*)calloc(n, sizeof(elem_t));
    }
    ensure_quant_arrays(a, layer);
    int64_t pages = (total + P - 1) / P;
    /* append loop, kv.rs:723-734 */
    int64_t written = 0;
    while (written < seq) {
        int64_t global = pos + written;
        int64_t slot = global % P;
        int64_t run = (P - slot) < (seq - written) ? (P - slot) : (seq - written);
        int64_t phys = s->table[global / P];
        for (int h = 0; h < H; h++) {
            store_rows(a, layer, 0, ((size_t)phys * H + h) * P + slot, k + ((size_t)h * seq + written) * d, run);
            store_rows(a, layer, 1, ((size_t)phys * H + h) * P + slot, v + ((size_t)h * seq + written) * d, run);
        }
        written += run;
    }
    elem_t* kw = gather_window(s, a->k[layer], pages, total); /* kv.rs:735-736 */
    elem_t* vw = gather_window(s, a->v[layer], pages, total);
    attend(q, kw, vw, out, n_q, H, seq, total, d, pos, scale, window); /* kv.rs:790 */
    free(kw); free(vw);
    return ORC_OK;
}

/* EXTENSION (benchmark set-up only): the append loop of kv.rs:723-734 without the
 * attention that follows it, to fill long contexts cheaply.  k, v [n_kv, seq, d]. */
int orc_append_only(orc_seq* s, int layer, const elem_t* k, const elem_t* v, int64_t seq, int64_t pos) {
    orc_arena* a = s->a;
    int H = a->n_kv, d = a->d, P = a->page_size;
    if (pos + seq != s->seq_len) { snprintf(g_err, sizeof g_err, "layer call does not match the step begun"); return ORC_ERR_POS; }
    if (!a->k[layer]) {
        size_t n = (size_t)a->num_pages * H * P * d;
        a->k[layer] = (elem_t*)calloc(n, sizeof(elem_t));
        a->v[layer] = (elem_t*)calloc(n, sizeof(elem_t));
    }
    ensure_quant_arrays(a, layer);
    int64_t written = 0;
    while (written < seq) {
        int64_t global = pos + written, slot = global % P;
        int64_t run = (P - slot) < (seq - written) ? (P - slot) : (seq - written);
        int64_t phys = s->table[global / P];
        for (int h = 0; h < H; h++) {
            store_rows(a, layer, 0, ((size_t)phys * H + h) * P + slot, k + ((size_t)h * seq + written) * d, run);
            store_rows(a, layer, 1, ((size_t)phys * H + h) * P + slot, v + ((size_t)h * seq + written) * d, run);
        }
        written += run;
    }
    return ORC_OK;
}

/* The reference call: layer 0 advances the sequence (kv.rs:670-678). */
int orc_attention(orc_seq* s, int layer, const elem_t* q, const elem_t* k, const elem_t* v, elem_t* out,
                  int n_q, int64_t seq, int64_t pos, double scale, int64_t window) {
    if (layer == 0) { int rc = orc_begin(s, pos, seq); if (rc != ORC_OK) return rc; }
    return orc_layer(s, layer, q, k, v, out, n_q, seq, pos, scale, window);
}

/* popn, kv.rs:807-835 */
int64_t orc_popn(orc_seq* s, int64_t n) {
    orc_arena* a = s->a;
    if (n > s->seq_len) n = s->seq_len;
    if (n <= 0) return 0;
    if (a->rolling) {
        for (int i = 0; i < a->layers; i++)
            if (a->windows[i] > 0 && s->seq_len > a->windows[i] - 1) return 0; /* kv.rs:812-816 */
        for (int i = 0; i < a->layers; i++) if (s->sk[i]) { /* tail truncation, kv.rs:817-827 */
            int64_t len = s->slen[i], keep = len > n ? len - n : 0;
            int H = a->n_kv, d = a->d;
            if (keep > 0) {
                elem_t* nk = (elem_t*)malloc(sizeof(elem_t) * (size_t)H * keep * d);
                elem_t* nv = (elem_t*)malloc(sizeof(elem_t) * (size_t)H * keep * d);
                for (int h = 0; h < H; h++) {
                    memcpy(nk + (size_t)h * keep * d, s->sk[i] + (size_t)h * len * d, sizeof(elem_t) * (size_t)keep * d);
                    memcpy(nv + (size_t)h * keep * d, s->sv[i] + (size_t)h * len * d, sizeof(elem_t) * (size_t)keep * d);
                }
                free(s->sk[i]); free(s->sv[i]); s->sk[i] = nk; s->sv[i] = nv; s->slen[i] = keep;
            } else { free(s->sk[i]); free(s->sv[i]); s->sk[i] = s->sv[i] = NULL; s->slen[i] = 0; }
        }
    }
    int64_t new_len = s->seq_len - n;
    int64_t keep = (new_len + a->page_size - 1) / a->page_size;
    /* EXTENSION: a rollback may not end inside a page that other sequences also
       hold (the next append would overwrite their rows); refused like the
       sliding case, state untouched. */
    if (new_len % a->page_size != 0 && keep >= 1 && keep <= s->n_table && a->refcnt[s->table[keep - 1]] > 1) return 0;
    s->seq_len = new_len;
    while (s->n_table > keep) table_pop_release(s); /* kv.rs:829-833 */
    return n;
}

/* reset, kv.rs:837-846.  With other live sequences in the arena (EXTENSION) only
 * this sequence's pages are released, in table.pop() order. */
void orc_reset(orc_seq* s) {
    orc_arena* a = s->a;
    if (a->live_seqs == 1) {
        for (int64_t i = 0; i < s->n_table; i++) a->refcnt[s->table[i]] = 0;
        s->n_table = 0;
        alloc_reset(&a->alloc);
    } else {
        while (s->n_table) table_pop_release(s);
    }
    s->seq_len = 0;
    drop_sliding(s);
}

int64_t orc_seq_len(const orc_seq* s) { return s->seq_len; }                 /* kv.rs:793-795 */
int64_t orc_pages_used(const orc_seq* s) { return s->n_table; }              /* kv.rs:848-850 */
int64_t orc_num_free_pages(const orc_arena* a) { return a->alloc.n_free; }   /* kv.rs:529-532 */

/* page_stats_inner, kv.rs:535-546: 8 counters in declaration order */
void orc_page_stats(const orc_seq* s, int64_t out[8]) {
    const orc_arena* a = s->a;
    int mat = 0, sl = 0;
    for (int i = 0; i < a->layers; i++) { if (a->k[i]) mat++; if (s->sk[i]) sl++; }
    out[0] = s->n_table; out[1] = a->alloc.n_free; out[2] = a->num_pages; out[3] = a->page_size;
    out[4] = s->seq_len; out[5] = mat; out[6] = a->layers; out[7] = sl;
}

int64_t orc_export_block_table(const orc_seq* s, int64_t* out, int64_t cap) {
    for (int64_t i = 0; i < s->n_table && i < cap; i++) out[i] = s->table[i];
    return s->n_table;
}
/* free stack bottom-to-top (the last entry is handed out next) */
int64_t orc_export_free_list(const orc_arena* a, int64_t* out, int64_t cap) {
    for (int64_t i = 0; i < a->alloc.n_free && i < cap; i++) out[i] = a->alloc.free[i];
    return a->alloc.n_free;
}
/* one page of one layer as [n_kv, page_size, d]; zeros if the layer never materialised */
void orc_export_page(const orc_arena* a, int layer, int64_t page, elem_t* k_out, elem_t* v_out) {
    size_t n = (size_t)a->n_kv * a->page_size * a->d;
    if (!a->k[layer]) { memset(k_out, 0, n * sizeof(elem_t)); memset(v_out, 0, n * sizeof(elem_t)); return; }
    memcpy(k_out, a->k[layer] + (size_t)page * n, n * sizeof(elem_t));
    memcpy(v_out, a->v[layer] + (size_t)page * n, n * sizeof(elem_t));
}
int32_t orc_page_refcount(const orc_arena* a, int64_t page) { return a->refcnt[page]; }

/* ------------------------------------------------------ ContiguousKVCache
 * kv.rs:360-415: cat per step + attend; the reference's own cross-check. */
typedef struct { int layers, n_kv, d; elem_t** k; elem_t** v; int64_t* len; int64_t seq_len; } orc_contig;

orc_contig* orc_contig_new(int layers, int n_kv, int d) {
    orc_contig* c = (orc_contig*)calloc(1, sizeof *c);
    c->layers = layers; c->n_kv = n_kv; c->d = d;
    c->k = (elem_t**)calloc((size_t)layers, sizeof(elem_t*));
    c->v = (elem_t**)calloc((size_t)layers, sizeof(elem_t*));
    c->len = (int64_t*)calloc((size_t)layers, sizeof(int64_t));
    return c;
}
void orc_contig_reset(orc_contig* c) { /* kv.rs:409-414 */
    for (int i = 0; i < c->layers; i++) { free(c->k[i]); free(c->v[i]); c->k[i] = c->v[i] = NULL; c->len[i] = 0; }
    c->seq_len = 0;
}
void orc_contig_free(orc_contig* c) { if (!c) return; orc_contig_reset(c); free(c->k); free(c->v); free(c->len); free(c); }
int64_t orc_contig_seq_len(const orc_contig* c) { return c->seq_len; }

int orc_contig_attention(orc_contig* c, int layer, const elem_t* q, const elem_t* k, const elem_t* v, elem_t* out,
                         int n_q, int64_t seq, int64_t pos, double scale, int64_t window) {
    int H = c->n_kv, d = c->d;
    int64_t old = c->len[layer], full = old + seq;
    elem_t* kf = (elem_t*)malloc(sizeof(elem_t) * (size_t)H * full * d);
    elem_t* vf = (elem_t*)malloc(sizeof(elem_t) * (size_t)H * full * d);
    for (int h = 0; h < H; h++) {
        if (old) {
            memcpy(kf + (size_t)h * full * d, c->k[layer] + (size_t)h * old * d, sizeof(elem_t) * (size_t)old * d);
            memcpy(vf + (size_t)h * full * d, c->v[layer] + (size_t)h * old * d, sizeof(elem_t) * (size_t)old * d);
        }
        memcpy(kf + ((size_t)h * full + old) * d, k + (size_t)h * seq * d, sizeof(elem_t) * (size_t)seq * d);
        memcpy(vf + ((size_t)h * full + old) * d, v + (size_t)h * seq * d, sizeof(elem_t) * (size_t)seq * d);
    }
    free(c->k[layer]); free(c->v[layer]);
    c->k[layer] = kf; c->v[layer] = vf; c->len[layer] = full;
    c->seq_len = full; /* kv.rs:399 */
    attend(q, kf, vf, out, n_q, H, seq, full, d, pos, scale, window);
    return ORC_OK;
}

/* ------------------------------------------------------------ batch driver
 * EXTENSION used by the timed CPU baseline: one decode/prefill step of a batch
 * = the reference call made once per sequence (sequence index ascending for the
 * bookkeeping, then sequences in parallel since they are independent caches).
 * Packed layout: sequence b's block is the reference tensor [H, seq_b, d]. */
int orc_batch_begin(orc_seq** seqs, const int64_t* new_tokens, int n) {
    for (int b = 0; b < n; b++) {
        int rc = orc_begin(seqs[b], seqs[b]->seq_len, new_tokens[b]);
        if (rc != ORC_OK) return rc;
    }
    return ORC_OK;
}

int orc_batch_layer(orc_seq** seqs, const int64_t* new_tokens, int n, int layer,
                    const elem_t* q, const elem_t* k, const elem_t* v, elem_t* out,
                    int n_q, double scale, int64_t window) {
    if (n <= 0) return ORC_OK;
    orc_arena* a = seqs[0]->a;
    int64_t* off = (int64_t*)malloc(sizeof(int64_t) * (size_t)(n + 1));
    off[0] = 0;
    for (int b = 0; b < n; b++) off[b + 1] = off[b] + new_tokens[b];
    /* materialise arenas before going parallel */
    if (!a->k[layer] && !(a->rolling && a->windows[layer] > 0)) {
        size_t cnt = (size_t)a->num_pages * a->n_kv * a->page_size * a->d;
        a->k[layer] = (elem_t*)calloc(cnt, sizeof(elem_t));
        a->v[layer] = (elem_t*)calloc(cnt, sizeof(elem_t));
    }
    ensure_quant_arrays(a, layer);
    int rc_all = ORC_OK;
#pragma omp parallel for schedule(dynamic)
    for (int b = 0; b < n; b++) {
        int64_t sq = new_tokens[b];
        int rc = orc_layer(seqs[b], layer, q + (size_t)off[b] * n_q * a->d, k + (size_t)off[b] * a->n_kv * a->d,
                           v + (size_t)off[b] * a->n_kv * a->d, out + (size_t)off[b] * n_q * a->d,
                           n_q, sq, seqs[b]->seq_len - sq, scale, window);
        if (rc != ORC_OK) rc_all = rc;
    }
    free(off);
    return rc_all;
}
