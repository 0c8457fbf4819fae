/*
 * combs_kv.h — C ABI of the B200 paged KV cache + attention library (libcombskv.so).
 *
 * Drop-in boundary for one path of CombsEngine: the `KVCache` operator surface of
 * engine/core/combs-models/src/kv.rs (trait at kv.rs:92-151, `PagedKVCache` at
 * kv.rs:477-855).  A Rust `impl KVCache<B>` binds these symbols one-to-one; each
 * declaration cites the reference item it replaces.
 *
 * Conventions (those of the reference's own C ABI, combs-ffi/src/lib.rs:41-71):
 *   - opaque handles, plain pointers and sizes, no C++ or torch types;
 *   - every call returns int32_t: 0 = ok, negative = error; nothing aborts: no C++
 *     exception leaves the library (each entry point catches them, as the reference's FFI
 *     wraps every entry point in catch_unwind, combs-ffi/src/lib.rs:143,173-183), and a
 *     null handle is an error, not a crash; on error the cache state is untouched
 *     (all-or-nothing, kv.rs:805-806);
 *   - cbkv_last_error() is thread-local, borrowed, valid until the next call on
 *     the same thread; it carries the reference's panic texts verbatim;
 *   - handles are not thread-safe (the trait is Send, not Sync): one owner
 *     thread at a time per arena;
 *   - device work is enqueued on the caller's cudaStream_t (passed as void*);
 *     nothing synchronises except the cbkv_export_* and *_host calls.
 *
 * Tensor layouts are the reference's: Q [1, n_q, seq, d], K/V [1, n_kv, seq, d]
 * (kv.rs:89-91).  A batch of sequences is the concatenation of per-sequence
 * blocks in the order given to cbkv_begin_step: sequence b contributes one
 * contiguous block [n_heads, seq_b, d].
 */
#ifndef COMBS_KV_H
#define COMBS_KV_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct cbkv_arena cbkv_arena; /* arenas + free-list shared by its sequences */
typedef struct cbkv_seq cbkv_seq;     /* one sequence == one reference PagedKVCache  */

enum {
    CBKV_OK = 0,
    CBKV_ERR_POS = -1,       /* "paged cache expects dense contiguous appends"  kv.rs:671-674 */
    CBKV_ERR_CAPACITY = -2,  /* "paged cache capacity exceeded"                 kv.rs:679-683 */
    CBKV_ERR_EXHAUSTED = -3, /* "page allocator exhausted"                      kv.rs:552-555 */
    CBKV_ERR_ARG = -4,       /* bad argument / bad geometry (kv.rs:513-516)     */
    CBKV_ERR_CUDA = -5,      /* a CUDA runtime or driver call failed            */
    CBKV_ERR_STATE = -6,     /* call out of order (no step begun, layer mismatch) */
    CBKV_ERR_DEVICE = -7,    /* a kernel reported a problem in its status word   */
    CBKV_ERR_INTERNAL = -8   /* a C++ exception was stopped at the boundary (the reference's FFI turns a
                                panic into rc = -1 plus the message, combs-ffi/src/lib.rs:173-183) */
};

enum { CBKV_F16 = 0, CBKV_BF16 = 1 };

/* CacheConfig (kv.rs:40-85) plus the model geometry the reference reads off its
 * tensors, plus the per-layer windows of PagedKVCache::new_with_windows
 * (kv.rs:508-527). */
typedef struct {
    int32_t num_layers;
    int32_t n_q_heads;
    int32_t n_kv_heads;
    int32_t head_dim;
    int32_t page_size;            /* CacheConfig::DEFAULT_PAGE_SIZE = 16 (kv.rs:59) */
    int32_t dtype;                /* CBKV_F16 (the reference's f16 build) or CBKV_BF16 */
    int64_t max_seq_len;          /* per-sequence capacity, CacheConfig::max_seq_len */
    int64_t num_pages;            /* 0 => ceil(max_seq_len / page_size) (kv.rs:82-84);
                                     larger when several sequences share the arena */
    const int64_t* layer_windows; /* NULL or num_layers entries; 0 = global, w >= 2 = sliding */
    int32_t sliding_popn_refuses; /* 1 = popn refuses once a sliding layer would have
                                     evicted (kv.rs:812-816); 0 = windows are pure masks */
    int32_t device;               /* CUDA device ordinal */
    int32_t quantize_kv;          /* CacheConfig::quantize_kv (kv.rs:464-475,694): int8 pages with one scale
                                     per 32 values for every layer without a window of its own, when
                                     head_dim is a multiple of 32; other layers keep float pages */
} cbkv_config;

/* PageStats (kv.rs:153-175), same eight counters in the same order. */
typedef struct {
    int64_t pages_used;
    int64_t pages_free;
    int64_t num_pages;
    int64_t page_size;
    int64_t seq_len;
    int64_t layers_materialized;
    int64_t layers_total;
    int64_t layers_sliding;
} cbkv_page_stats_t;

/* Thread-local text of the last failure, or "" (combs_last_error, combs-ffi/src/lib.rs:52-58). */
const char* cbkv_last_error(void);

/* ---- construction ------------------------------------------------------- */

/* PagedKVCache::new_with_windows (kv.rs:508-527): validates geometry and windows,
 * builds the free-list (page 0 first, kv.rs:424-429).  Touches no device memory:
 * arenas appear lazily on a layer's first write (kv.rs:695-713). */
int32_t cbkv_arena_create(const cbkv_config* cfg, cbkv_arena** out);
int32_t cbkv_arena_destroy(cbkv_arena* arena);

/* Extension (no reference counterpart; the reference order 0,1,2,... is the
 * default): replace the initial free-list order; ids[0] is handed out first.
 * Only on an arena no page of which is in use. */
int32_t cbkv_set_free_list(cbkv_arena* arena, const int64_t* ids, int64_t n);

/* A new empty sequence over the arena (the per-request `create_kv_cache`,
 * traits.rs:26 / llama.rs:377-390).  Destroying it returns its pages in
 * table.pop() order (kv.rs:830-833). */
int32_t cbkv_seq_create(cbkv_arena* arena, cbkv_seq** out);
int32_t cbkv_seq_destroy(cbkv_seq* seq);

/* Extension: cross-sequence prefix sharing.  The child starts with seq_len =
 * n_tokens and aliases the parent's first n_tokens / page_size pages (whole pages
 * only); a shared page returns to the free-list when its last holder drops it. */
int32_t cbkv_seq_fork_prefix(cbkv_seq* parent, int64_t n_tokens, cbkv_seq** out);

/* ---- one forward pass ---------------------------------------------------- */

/* The layer-0 prologue of attention_opts (kv.rs:665-683) and ensure_pages
 * (kv.rs:549-559) for every sequence of the step, in the order given:
 * requires pos[b] == seq_len (pass pos = NULL to skip the check), advances
 * seq_len by new_tokens[b], allocates pages, and uploads the step's block tables
 * and work partition to the device on `stream`.  n_seqs = 0 opens an empty step:
 * the attention and append calls that follow return 0 and launch nothing. */
int32_t cbkv_begin_step(cbkv_arena* arena, cbkv_seq* const* seqs, const int64_t* new_tokens,
                        const int64_t* pos, int32_t n_seqs, void* stream);

/* The append loop (kv.rs:721-734) for the step's sequences: scatters the new K/V
 * rows into their page slots.  k, v: device, packed per sequence [n_kv, seq_b, d]. */
int32_t cbkv_append(cbkv_arena* arena, int32_t layer, const void* k, const void* v, void* stream);

/* gather_window + attend (kv.rs:735-736,790 and 201-269) without the gather:
 * attention of the step's queries over the paged prefix plus the rows just
 * appended.  window: 0 = none; the arena's own layer window wins (kv.rs:688-693).
 * q, out: device, packed per sequence [n_q, seq_b, d]. */
int32_t cbkv_paged_attention(cbkv_arena* arena, int32_t layer, const void* q, void* out,
                             double scale, int64_t window, void* stream);

/* KVCache::attention_opts (kv.rs:116-125, 655-791) for one layer of the step begun:
 * append + attention in one call (one fused launch on the decode path). */
int32_t cbkv_attention(cbkv_arena* arena, int32_t layer, const void* q, const void* k, const void* v,
                       void* out, double scale, int64_t window, void* stream);

/* The same call with HOST buffers (what a caller holding host tensors makes):
 * copies q, k, v to the device, runs cbkv_attention, copies `out` back and waits
 * for it.  Buffers from cbkv_host_alloc are pinned and copy asynchronously. */
int32_t cbkv_attention_host(cbkv_arena* arena, int32_t layer, const void* q_host, const void* k_host,
                            const void* v_host, void* out_host, double scale, int64_t window, void* stream);
/* The same call without the wait: the copies run on the library's own copy streams
 * so that layer l+1's inputs and layer l's output move while a kernel runs; `out_host`
 * is valid after cbkv_host_sync.  Needs pinned buffers to overlap; 32 calls can be in flight,
 * a 33rd waits for the oldest.  On a decode step `stream` is not made to wait for the input
 * copies (a wait between two kernels would end the overlap of consecutive layers' launches):
 * the kernel itself waits, with the usual limit, for a number that the copy stream writes
 * behind its inputs. */
int32_t cbkv_attention_host_async(cbkv_arena* arena, int32_t layer, const void* q_host, const void* k_host,
                                  const void* v_host, void* out_host, double scale, int64_t window, void* stream);
int32_t cbkv_host_sync(cbkv_arena* arena);
int32_t cbkv_host_alloc(size_t bytes, void** out);
int32_t cbkv_host_free(void* p);

/* ---- the step right before the cache: rotary embedding and QK norm, fused into the append ----
 *
 * The model rotates q and k (RotaryEmbedding::apply, combs-models/src/rope.rs:180-204) after an
 * optional per-head RMS norm (combs-models/src/llama.rs:275-281, norm.rs:11-39) and only then calls
 * the cache (llama.rs:283-289).  These entry points take the UN-rotated q and k and do all of it in
 * one launch that writes k and v into their page slots and the rotated q into a dense buffer. */
enum { CBKV_ROPE_NONE = 0, CBKV_ROPE_LINEAR = 1, CBKV_ROPE_LLAMA3 = 2, CBKV_ROPE_YARN = 3, CBKV_ROPE_LONGROPE = 4 };

/* RotaryEmbedding::new_scaled + combs_formats::RopeScaling (rope.rs:31-125,160-177). */
typedef struct cbkv_rope_config {
    int32_t head_dim;
    int32_t scaling;                /* CBKV_ROPE_* */
    double theta;
    int64_t max_position;           /* rows of the tables */
    double factor;                  /* linear, llama3, yarn, longrope */
    double low_freq_factor;         /* llama3 */
    double high_freq_factor;        /* llama3 */
    double beta_fast, beta_slow;    /* yarn */
    int64_t original_max_position;  /* llama3, yarn, longrope */
    int32_t has_attention_factor;   /* yarn, longrope: 0 = derive it as the reference does */
    double attention_factor;
    const double* short_factor;     /* longrope: head_dim/2 divisors (missing entries = 1) */
    int32_t n_short_factor;
} cbkv_rope_config;

typedef struct cbkv_rope cbkv_rope;

/* build_tables_scaled (rope.rs:129-151) on the host: cos and sin [max_position][head_dim] f32.
 * Needs no device. */
int32_t cbkv_rope_tables_host(const cbkv_rope_config* cfg, float* cos_out, float* sin_out);
/* scaled_inv_freq (rope.rs:31-125): head_dim/2 frequencies and the table multiplier. */
int32_t cbkv_rope_inv_freq_host(const cbkv_rope_config* cfg, double* inv_freq_out, double* mscale_out);
/* Tables on the arena's device in the arena's element type (rope.rs:160-177). */
int32_t cbkv_rope_create(cbkv_arena* arena, const cbkv_rope_config* cfg, cbkv_rope** out);
int32_t cbkv_rope_destroy(cbkv_rope* rope);

/* Per-head norm of q and k over head_dim before the rotation: weights are device pointers to
 * head_dim elements of the arena's type, either may be NULL; gemma != 0 scales by (1 + w)
 * (norm.rs:33-39). */
typedef struct cbkv_qk_norm {
    const void* q_weight;
    const void* k_weight;
    double eps;
    int32_t gemma;
} cbkv_qk_norm;

/* norm (optional, NULL = none) + rotate q -> q_out (may alias q), norm + rotate k -> pages,
 * v -> pages, for the step opened by cbkv_begin_step.  Positions are the step's (pos + row). */
int32_t cbkv_rope_append(cbkv_arena* arena, int32_t layer, const cbkv_rope* rope, const cbkv_qk_norm* norm,
                         const void* q, const void* k, const void* v, void* q_out, void* stream);
/* cbkv_rope_append into an internal buffer followed by cbkv_paged_attention: the whole of
 * llama.rs:275-289 for one layer. */
int32_t cbkv_attention_rope(cbkv_arena* arena, int32_t layer, const cbkv_rope* rope, const cbkv_qk_norm* norm,
                            const void* q, const void* k, const void* v, void* out, double scale, int64_t window,
                            void* stream);

/* ---- the callers that drive allocate / popn / reuse (host only, no device work) -------------
 *
 * Named rolling sessions over one arena: SessionSet with LRU eviction
 * (combs-runtime/src/engine.rs:266-314, MAX_SESSIONS = 4 at :243).  The reference gives every
 * session a private cache; here a session is a sequence of the shared arena. */
typedef struct cbkv_sessions cbkv_sessions;
int32_t cbkv_sessions_create(cbkv_arena* arena, int32_t max_sessions /* 0 = 4 */, cbkv_sessions** out);
int32_t cbkv_sessions_destroy(cbkv_sessions* set);
/* Start of a generation (engine.rs:1235-1287): takes the session `key` out of the table and rolls its
 * cache back to the longest common prefix of its history with `prompt`, capped at n_prompt - 1; when
 * nothing is shared, or the cache refuses the rollback, the old sequence is dropped and a fresh one
 * returned.  *lcp_out = tokens already cached (prefill starts there).  reuse = 0: always fresh. */
int32_t cbkv_sessions_acquire(cbkv_sessions* set, const char* key, const uint32_t* prompt, int64_t n_prompt,
                              int32_t reuse, cbkv_seq** seq_out, int64_t* lcp_out);
/* End of a generation (engine.rs:1541-1568, SessionSet::put :296-313): stores the sequence with its
 * history (which must equal what the cache holds), evicting the least recently used session beyond
 * max_sessions.  reuse = 0: the sequence is destroyed instead. */
int32_t cbkv_sessions_release(cbkv_sessions* set, const char* key, cbkv_seq* seq, const uint32_t* history,
                              int64_t n_history, int32_t reuse);
int32_t cbkv_sessions_clear(cbkv_sessions* set, int64_t* removed);          /* clear_all, engine.rs:287-291 */
int64_t cbkv_sessions_count(const cbkv_sessions* set);
int64_t cbkv_sessions_evictions(const cbkv_sessions* set);
int64_t cbkv_sessions_history_len(const cbkv_sessions* set, const char* key); /* -1: no such session */
/* Speculative verification (engine.rs:1476-1493): `argmax` holds the model's k+1 row-wise choices after
 * feeding [next, draft...]; accepts the longest matching prefix of the draft, pops the rejected tail
 * from the cache (an incomplete pop is CBKV_ERR_STATE, as in the reference) and returns the correction
 * token argmax[min(accepted, k)]. */
int32_t cbkv_spec_verify_rollback(cbkv_seq* seq, const uint32_t* draft, const uint32_t* argmax, int32_t k,
                                  int32_t* accepted_out, uint32_t* correction_out);
/* The "kv" object of GET /v1/stats (combs-cli/src/serve.rs:146-166,197-208) as JSON text, sessions
 * ordered by id.  Returns the length needed (excluding the terminator); writes at most cap bytes. */
int64_t cbkv_sessions_stats_json(const cbkv_sessions* set, char* buf, int64_t cap);

/* No counterpart in the reference.  Decode attention over pages the CALLER owns, for
 * callers that must not allocate device memory while they run (a server that gave
 * the whole GPU to its own pool at start-up, a plugin inside a host that forbids
 * late allocations): nothing is allocated or freed, the kernel's working memory is a
 * fixed ~6 MB array inside the library image.  Limits: at most 128 sequences,
 * 1024 sequence x kv-head pairs and 524288 (sequence, kv head, visible page) triples per
 * call, head_dim 64/128/256, at most 8 q heads per kv head, 16-token pages; larger problems
 * return CBKV_ERR_ARG.
 *   kv_pages      device, one layer's pages [num_pages][n_kv][2 (slots 0-7, 8-15)][2 (K,V)][8][head_dim]
 *   block_tables  device, [n_seqs][table_stride] physical page ids
 *   seq_lens_host HOST, [n_seqs]: cached tokens including the one being decoded
 *   q, out        device, [n_seqs][n_q][head_dim]
 * All calls on a device share the working memory: calls that overlap on the GPU
 * race, so keep them on one stream or order them.  The first call on a device does a
 * one-time set-up and should be made before any stream capture begins.  The kernel reports a
 * bad block-table entry or a wait that ran out in a status word inside the same array, which
 * every call clears at its start: read it with cbkv_static_status after the call. */
int32_t cbkv_decode_attention_static(const void* kv_pages, int64_t num_pages, const int32_t* block_tables,
                                     int32_t table_stride, const int32_t* seq_lens_host, int32_t n_seqs,
                                     int32_t n_q_heads, int32_t n_kv_heads, int32_t head_dim, int32_t dtype,
                                     const void* q, void* out, double scale, int64_t window, void* stream);

/* No counterpart in the reference.  Waits for `stream`, then reads and clears the status word
 * of the static entry point on the current device (same bits as cbkv_device_status); allocates
 * nothing.  A non-zero word returns CBKV_ERR_DEVICE with *status set. */
int32_t cbkv_static_status(void* stream, int32_t* status);

/* ---- rollback / reset / counters ----------------------------------------- */

/* KVCache::popn (kv.rs:807-835): *popped = tokens dropped; 0 = refused. */
int32_t cbkv_popn(cbkv_seq* seq, int64_t n, int64_t* popped);
/* KVCache::reset (kv.rs:837-846).  Alone in its arena: allocator back to its
 * initial order.  Otherwise only this sequence's pages are released. */
int32_t cbkv_reset(cbkv_seq* seq);
int64_t cbkv_seq_len(const cbkv_seq* seq);              /* kv.rs:793-795 */
int64_t cbkv_pages_used(const cbkv_seq* seq);           /* kv.rs:848-850 */
int64_t cbkv_num_free_pages(const cbkv_arena* arena);   /* kv.rs:529-532 */
int32_t cbkv_page_stats(const cbkv_seq* seq, cbkv_page_stats_t* out); /* kv.rs:535-546 */
/* kv_page_bytes (combs-runtime/src/engine.rs:475-498): bytes one page id costs
 * across K, V and all paged layers. */
int64_t cbkv_page_bytes(const cbkv_arena* arena);

/* ---- state export (parity checks, checkpoints) ---------------------------- */

/* logical -> physical page ids (kv.rs:481); returns the table length. */
int64_t cbkv_export_block_table(const cbkv_seq* seq, int64_t* out, int64_t cap);
/* free stack bottom-to-top (the last entry is handed out next, kv.rs:431-437). */
int64_t cbkv_export_free_list(const cbkv_arena* arena, int64_t* out, int64_t cap);
/* One page of one layer as the reference lays it out, [n_kv, page_size, d] for K
 * and for V (kv.rs:450-451), copied to host; zeros if the layer has not
 * materialised.  Synchronises `stream`. */
int32_t cbkv_export_page(cbkv_arena* arena, int32_t layer, int64_t page, void* k_out_host,
                         void* v_out_host, void* stream);
/* One page of a quantised layer as the reference's Arena::Quant holds it (kv.rs:464-475): packed
 * int32 words [n_kv][page_size][head_dim/4] (kv.rs:276-283) and scales [n_kv][page_size][head_dim/32]
 * in the arena's element type, for K and for V.  Host buffers; synchronises. */
int32_t cbkv_export_page_quant(cbkv_arena* arena, int32_t layer, int64_t page, int32_t* k_packed_host, void* k_scales_host,
                               int32_t* v_packed_host, void* v_scales_host, void* stream);
/* 1 if the layer stores int8 pages, 0 if float pages, negative on a bad argument. */
int32_t cbkv_layer_is_quantized(const cbkv_arena* arena, int32_t layer);
int32_t cbkv_page_refcount(const cbkv_arena* arena, int64_t page);

/* ---- diagnostics ----------------------------------------------------------- */

/* Reads and clears the status word the kernels write instead of trapping
 * (0 = clean; bits: 1 = a block-table entry outside the arena, which the kernels replace by
 * page 0 for reading and skip for writing; 2 = a bounded wait ran out; 4 = misaligned shared
 * memory).  Synchronises `stream`.  A caller should poll it at least once per step: after a
 * non-zero status the step's outputs are undefined; the next cbkv_begin_step starts clean. */
int32_t cbkv_device_status(cbkv_arena* arena, void* stream, int32_t* status);
/* Kernel launches issued by this library in this process so far. */
int64_t cbkv_launch_count(void);
/* Per-kernel device timing: when on, CUDA events bracket every attention launch;
 * cbkv_profile_read returns their summed duration and count and clears them. */
int32_t cbkv_profile_enable(cbkv_arena* arena, int32_t on);
int32_t cbkv_profile_read(cbkv_arena* arena, double* total_ms, int64_t* launches);
/* Tuning knobs for measurements and tests (0 = built-in default): CTAs per SM of the
 * decode kernel, stages of its TMA ring (rounded down to a multiple of the consumer
 * count), consumer warps per CTA (4, 6, 8 or 12), an upper bound on the CTAs launched,
 * and whether consecutive decode launches may overlap (programmatic dependent
 * launch; 1 = default). */
int32_t cbkv_set_decode_tuning(cbkv_arena* arena, int32_t ctas_per_sm, int32_t stages, int32_t consumers,
                               int32_t max_ctas, int32_t overlap_launches);

/* cbkv_attention_host_async on decode steps: 1 (default) = the kernel reads its inputs' arrival from a
 * flag, 0 = `stream` waits for the input copies' event before every kernel (what other steps use). */
int32_t cbkv_set_host_route(cbkv_arena* arena, int32_t direct);

/* Two-tile tcgen05 chunk kernel: when the last wave of a launch (one CTA per SM at a time) would fill at
 * most half of the SMs, its items are cut along K/V into up to `max_parts` CTAs each, whose partial rows
 * the last finisher adds up.  1 = never cut; default 4. */
int32_t cbkv_set_chunk_split(cbkv_arena* arena, int32_t max_parts);

/* Which kernel runs a step that is not pure decode: 0 = the library chooses (tcgen05
 * tiles once the step has at least 64 new tokens), 1 = the mma.sync kernel, 2 = the
 * tcgen05/TMEM kernel with one 128-row query tile per CTA (head_dim 64, 128 or 256), 3 = the
 * tcgen05/TMEM kernel with two query tiles per CTA and P in tensor memory (head_dim 128).
 * Over int8 layers these kernels read a float copy of the step's pages made per layer and
 * step; 4 = as 3, but the kernel fetches the int8 records and converts them itself (no
 * float copy; slower so far, kept for measurement). */
int32_t cbkv_set_chunk_kernel(cbkv_arena* arena, int32_t mode);

/* ---- test hooks (host only, no device is touched) --------------------------- */

/* The bookkeeping half of cbkv_begin_step alone (no reference counterpart beyond
 * kv.rs:665-683 itself): lets the manager be exercised where no GPU exists. */
int32_t cbkv_debug_begin_step_host(cbkv_arena* arena, cbkv_seq* const* seqs, const int64_t* new_tokens,
                                   const int64_t* pos, int32_t n_seqs);
/* The boundary's own test: the body throws (1 = std::bad_alloc, 2 = std::runtime_error, 3 = a non-standard
 * object, anything else = nothing) and the call must come back with CBKV_ERR_INTERNAL and a message, as a
 * panic behind the reference's FFI comes back as rc = -1 (combs-ffi/src/lib.rs:173-183). */
int32_t cbkv_debug_raise(int32_t kind);

/* The decode work split for the step in flight, flattened into `out`:
 * [n_ctas, n_items, n_segs, n_units, n_parts, levels, segment records (n_segs + 1 of 8 ints:
 *  unit_begin, page_lo, q_pos, tok_off, nparts, part_base, tbl_off, 0), item records (n_items of
 *  4 ints: u_begin, u_end, first_seg, first_part) in claim order].  tail_pct / min_item: how the
 * tail of a CTA's range is cut into dynamically claimed items (negative = default).
 * Returns the number of words, or -1 without a step. */
int64_t cbkv_debug_decode_plan(cbkv_arena* arena, int64_t window, int32_t n_ctas, int32_t tail_pct, int32_t min_item,
                               int32_t* out, int64_t cap);

/* Tuning (no reference counterpart): the share of a CTA's range that is cut into dynamically
 * claimed tail items (percent), the smallest item (pages; 0 = no tail, a static equal split) and
 * the number of halvings + 2.  Negative / < 2 = keep. */
int32_t cbkv_set_decode_split(cbkv_arena* arena, int32_t tail_pct, int32_t min_item, int32_t max_levels);

/* Test hook for the kernels' failure path (the reference has no device-side failure path; its
 * host-side one is the panic fence above).  wait_us > 0 replaces the limit of the decode
 * kernel's bounded waits (default 100000 us).  fault_tile >= 0: the producer of CTA 0 never
 * issues the copy of that tile, so the wait of the warp that owns it runs out: the launch
 * returns, ST_WAIT_TIMEOUT (2) shows in cbkv_device_status, its output is undefined, and the
 * next step runs normally.  fault_tile = -1 switches the hook off.  Nothing is read or written
 * outside the kernel's own buffers either way. */
int32_t cbkv_debug_set_wait_limit(cbkv_arena* arena, int64_t wait_us, int32_t fault_tile);

#ifdef __cplusplus
}
#endif
#endif /* COMBS_KV_H */
