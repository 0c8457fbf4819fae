// Host-side cache manager: free-list, per-sequence block tables, refcounts, the
// per-step bookkeeping of the reference's `attention_opts` prologue, and the work
// partition handed to the kernels.  No CUDA in this file; the device side lives in
// api.cu.  Reference: engine/core/combs-models/src/kv.rs (lines cited inline).
#pragma once
#include <cstdint>
#include <exception>
#include <new>
#include <string>
#include <vector>

#include "../../include/combs_kv.h"

namespace cbkv {

// Thread-local error text (combs-ffi/src/lib.rs:41-58).
void set_error(const std::string& msg);
void set_error_nothrow(const char* msg) noexcept;
const char* last_error();

// Every extern "C" entry point runs its body through one of these: a C++ exception (std::bad_alloc
// from a container, anything a callee throws) becomes CBKV_ERR_INTERNAL plus a message and never
// crosses the C boundary, where it would end the host process.  The reference's FFI wraps every
// entry point in catch_unwind for the same reason (combs-ffi/src/lib.rs:143,173-183).
template <typename F>
inline int32_t fenced(F&& body) noexcept {
    try {
        return body();
    } catch (const std::bad_alloc&) {
        set_error_nothrow("out of host memory");
    } catch (const std::exception& e) {
        set_error_nothrow(e.what());
    } catch (...) {
        set_error_nothrow("unknown C++ exception");
    }
    return CBKV_ERR_INTERNAL;
}
template <typename F>
inline int64_t fenced64(F&& body) noexcept {
    try {
        return body();
    } catch (const std::bad_alloc&) {
        set_error_nothrow("out of host memory");
    } catch (const std::exception& e) {
        set_error_nothrow(e.what());
    } catch (...) {
        set_error_nothrow("unknown C++ exception");
    }
    return CBKV_ERR_INTERNAL;
}

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
    uint64_t mark = 0;           // begin_step's duplicate check
};

// Per-sequence record the kernels read (16 bytes).
struct SeqMeta {
    int32_t pos;      // tokens cached before this step
    int32_t snew;     // tokens appended this step
    int32_t tok_off;  // sum of snew over earlier sequences of the step
    int32_t tbl_off;  // offset of this sequence's block table in the flat table array
};

// Work split of one decode launch.  A unit is one (sequence, kv head, visible page); a
// segment is all units of one (sequence, kv head).  The units are first divided into one
// contiguous range per CTA; each range is then cut into a large head item and a tail of
// items of decreasing size.  CTA c starts with head item c and afterwards claims items from
// a device counter in list order (larger tail items first), so that CTAs on slower SMs
// simply take fewer of them.  A segment cut by item boundaries leaves partial results that
// the last item to finish one merges.
struct SegInfo {        // 32 bytes, read by the kernels as two 16-byte words
    int32_t unit_begin; // first unit of the segment (entry n_segs holds n_units)
    int32_t page_lo;    // first visible logical page
    int32_t q_pos;      // absolute position of the sequence's decode query
    int32_t tok_off;    // index of the sequence's token in the packed q / k / v / out
    int32_t nparts;     // items that intersect the segment
    int32_t part_base;  // slot of part 0 in the partial buffers (-1: the segment is not cut)
    int32_t tbl_off;    // offset of the sequence's block table in the flat table array
    int32_t pad;
};
struct ItemInfo {       // 16 bytes
    int32_t u_begin, u_end;  // unit range
    int32_t first_seg;       // segment that holds u_begin
    int32_t first_part;      // index of the item's first piece among that segment's parts
};
struct DecodePlan {
    int64_t window = 0;
    int32_t n_ctas = 0, n_items = 0, n_segs = 0, n_units = 0, n_parts = 0, levels = 0;
    std::vector<SegInfo> segs;    // n_segs + 1
    std::vector<ItemInfo> items;  // n_items, in claim order: item c (c < n_ctas) is CTA c's first
};
// How the tail of a CTA's range is cut: `tail_pct` percent of the range, halved `levels - 1`
// times while the pieces stay >= min_item units.
struct DecodeSplit { int32_t tail_pct = 25, min_item = 0, max_levels = 5; };  // min_item 0: no tail, a static equal split

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
    uint64_t mark_gen = 0;

    // the step in flight
    bool step_open = false;
    bool step_is_decode = false;  // every sequence appends exactly one token
    std::vector<Seq*> step_seqs;
    std::vector<SeqMeta> step_meta;
    std::vector<int32_t> step_tables;
    int64_t step_tokens = 0;
    uint64_t step_id = 0;

    void* dev = nullptr;  // device-side state (api.cu), created on first device use

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
void build_decode_plan(const Arena& a, int64_t window, int32_t n_ctas, const DecodeSplit& split, DecodePlan* plan);
void build_chunk_plan(const Arena& a, int32_t cols_per_item, ChunkPlan* plan);
// Work list of the tcgen05 chunk kernel: one item per (sequence, kv head, tile of
// `tokens_per_tile` new tokens); `cols_per_item` records tokens_per_tile.
void build_chunk_tile_plan(const Arena& a, int32_t tokens_per_tile, ChunkPlan* plan);

}  // namespace cbkv
