// Host-side cache manager: free-list, per-sequence block tables, refcounts, the
// per-step bookkeeping of the reference's `attention_opts` prologue, and the work
// partition handed to the kernels.  No CUDA in this file; the device side lives in
// device.cu.  Reference: engine/core/combs-models/src/kv.rs (lines cited inline).
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "../../include/combs_kv.h"

namespace cbkv {

// Thread-local error text (combs-ffi/src/lib.rs:41-58).
void set_error(const std::string& msg);
const char* last_error();

// PageAllocator (kv.rs:417-446): a stack of page ids.
class Allocator {
public:
    void init(int64_t n);
    int64_t alloc() {                       // kv.rs:431-433
        if (free_.empty()) return -1;
        int64_t p = free_.back();
        free_.pop_back();
        return p;
    }
    void free_page(int64_t id) { free_.push_back(id); }  // kv.rs:435-437
    int64_t num_free() const { return (int64_t)free_.size(); }
    void reset() { free_ = initial_; }      // kv.rs:443-445
    bool set_initial(const int64_t* ids, int64_t n);
    const std::vector<int64_t>& stack() const { return free_; }
private:
    std::vector<int64_t> free_, initial_;
};

struct Arena;

struct Seq {
    Arena* arena = nullptr;
    std::vector<int64_t> table;  // logical page -> physical page (kv.rs:481)
    int64_t seq_len = 0;
};

// Per-sequence record the kernels read (16 bytes).
struct SeqMeta {
    int32_t pos;      // tokens cached before this step
    int32_t snew;     // tokens appended this step
    int32_t tok_off;  // sum of snew over earlier sequences of the step
    int32_t tbl_off;  // offset of this sequence's block table in the flat table array
};

// Split of one decode launch over `n_ctas` CTAs.  A unit is one (sequence, kv head,
// visible page); a segment is all units of one (sequence, kv head).  CTAs get equal
// contiguous unit ranges, so a segment may be cut into several parts whose partial
// results are merged by the last CTA to finish one.
struct DecodePlan {
    int64_t window = 0;
    int32_t n_ctas = 0, n_segs = 0, n_units = 0, n_parts = 0;
    std::vector<int32_t> seg_unit_begin;  // n_segs + 1
    std::vector<int32_t> seg_page_lo;     // first visible logical page of the segment
    std::vector<int32_t> seg_first_cta;   // n_segs
    std::vector<int32_t> seg_nparts;      // n_segs
    std::vector<int32_t> seg_part_base;   // n_segs, slot of part 0 in the partial buffer
    std::vector<int32_t> cta_unit_begin;  // n_ctas + 1
    std::vector<int32_t> cta_first_seg;   // n_ctas
};

// Work list of the chunk (prefill) kernel: one item per (sequence, kv head, block of
// query columns); a column is one (new token, q head of the kv group).
struct ChunkPlan {
    int32_t cols_per_item = 0;
    int32_t n_items = 0;
    std::vector<int32_t> item_begin;  // n_seqs + 1
};

struct Arena {
    cbkv_config cfg{};
    std::vector<int64_t> windows;  // per layer, 0 = global
    int64_t num_pages = 0;
    Allocator alloc;
    std::vector<int32_t> refcnt;
    std::vector<Seq*> seqs;  // live sequences

    // the step in flight
    bool step_open = false;
    bool step_is_decode = false;  // every sequence appends exactly one token
    std::vector<Seq*> step_seqs;
    std::vector<SeqMeta> step_meta;
    std::vector<int32_t> step_tables;
    int64_t step_tokens = 0;
    uint64_t step_id = 0;

    void* dev = nullptr;  // device-side state (device.cu), created on first device use

    int n_rep() const { return cfg.n_q_heads / cfg.n_kv_heads; }
    // int8 pages: asked for, head_dim a multiple of the 32-value group, and not a layer with a window of
    // its own (those never reach the quantised branch in the reference, kv.rs:688-694)
    bool layer_quant(int layer) const { return cfg.quantize_kv && cfg.head_dim % 32 == 0 && windows[(size_t)layer] == 0; }
    int64_t layer_window(int layer, int64_t arg) const {  // the cache's own window wins, kv.rs:688-693
        return windows[layer] > 0 ? windows[layer] : arg;
    }
};

int32_t arena_create(const cbkv_config* cfg, Arena** out);
int32_t seq_create(Arena* a, Seq** out);
int32_t seq_destroy(Seq* s);
int32_t seq_fork_prefix(Seq* parent, int64_t n_tokens, Seq** out);
int32_t begin_step(Arena* a, Seq* const* seqs, const int64_t* new_tokens, const int64_t* pos, int32_t n);
int32_t popn(Seq* s, int64_t n, int64_t* popped);
int32_t reset(Seq* s);
void page_stats(const Seq* s, int64_t layers_materialized, cbkv_page_stats_t* out);

// Builders used by the device layer (pure functions of the step state).
void build_decode_plan(const Arena& a, int64_t window, int32_t n_ctas, DecodePlan* plan);
void build_chunk_plan(const Arena& a, int32_t cols_per_item, ChunkPlan* plan);
// Work list of the tcgen05 chunk kernel: one item per (sequence, kv head, tile of
// `tokens_per_tile` new tokens); `cols_per_item` records tokens_per_tile.
void build_chunk_tile_plan(const Arena& a, int32_t tokens_per_tile, ChunkPlan* plan);

}  // namespace cbkv
