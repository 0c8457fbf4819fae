// Kernel argument blocks and launchers (kernels.cu).  Plain C++ types only.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "manager.hpp"

namespace cbkv {

// Status bits the kernels OR into the arena's status word instead of trapping.
enum : int32_t {
    ST_BAD_PAGE = 1,       // a block-table entry was outside the arena
    ST_WAIT_TIMEOUT = 2,   // a bounded mbarrier wait ran out
    ST_SMEM_ALIGN = 4,     // dynamic shared memory was not 1024-byte aligned
    ST_BAD_ARG = 8
};

// One layer's arena in HBM: one (page, kv head) is 32 consecutive rows of d elements.
// Tiled arenas (16-token pages served by the TMA kernels) order them in groups of eight,
// [K slots 0-7][V slots 0-7][K slots 8-15][V slots 8-15], so that one 32-row TMA box brings
// K and V of a page and both still look like uniformly strided 8-row groups to the tensor
// cores (stride 2048 bytes per 64-element column block).  Other arenas (any page size,
// generic kernel) keep [K slots][V slots].
#if defined(__CUDACC__)
#define CBKV_HD __host__ __device__
#else
#define CBKV_HD
#endif
CBKV_HD inline int page_row(int kv, int slot, int page_size, bool tiled) {
    return tiled ? ((slot >> 3) * 16 + kv * 8 + (slot & 7)) : (kv * page_size + slot);
}
// Quantised layers keep one record per (page, kv head):
//   [K bytes: P rows x d][V bytes: P/2 token pairs x d x 2][K scales: P x d/32 elems][V scales: d/32 x P elems]
// Every value byte is q + 128 (the reference's packed words, kv.rs:276-283, keep their fourth lane
// signed; the export flips that byte's top bit back).  The layout inside a record is the decode
// kernel's, which copies a record to shared memory as it lies and reads it with 8-byte loads:
//   K: row = token, d order, the 32-byte groups of a row permuted (group g at position g ^ swizzle);
//   V: the two tokens of a pair interleaved per d (so the two numbers an MMA register needs are
//      neighbours), 64-byte units = one group of a pair, units and their halves permuted;
//   V scales group-major, so the scales of two neighbouring tokens are one 32-bit word.
CBKV_HD inline size_t qrec_bytes(int page_size, int d) { return (size_t)2 * page_size * d + (size_t)2 * page_size * (d / 32) * 2; }
CBKV_HD inline bool qrec_swizzled(int d) { return d == 64 || d == 128 || d == 256 || d == 512; }
CBKV_HD inline int qrec_swz(int slot, int d) {  // K rows
    if (d == 64) return (slot >> 1) & 1;
    return qrec_swizzled(d) ? (slot & 3) : 0;
}
CBKV_HD inline size_t qrec_value_off(int is_v, int slot, int j, int page_size, int d) {
    if (!is_v) return (size_t)slot * d + (size_t)((((j >> 5) ^ qrec_swz(slot, d)) << 5) + (j & 31));
    const int pair = slot >> 1, sw = qrec_swizzled(d) ? 1 : 0;
    const int unit = (j >> 5) ^ (sw * (pair & 1));               // 64-byte unit: one group of the pair
    const int chunk = ((j & 31) >> 2) ^ (sw * 4 * ((pair >> 1) & 1));  // 8-byte chunk: 4 d-values x 2 tokens
    return (size_t)page_size * d + (size_t)pair * 2 * d + (size_t)unit * 64 + (size_t)chunk * 8 + (size_t)(j & 3) * 2 + (slot & 1);
}
CBKV_HD inline size_t qrec_scale_off(int is_v, int slot, int group, int page_size, int d) {
    const size_t base = (size_t)2 * page_size * d;
    return is_v ? base + ((size_t)page_size * (d / 32) + (size_t)group * page_size + slot) * 2
                : base + ((size_t)slot * (d / 32) + group) * 2;
}

struct LayerArena {
    void* base = nullptr;
    bool quant = false;  // base holds quantised records
    CUtensorMap map_kv;  // 2-D view [rows = pages*n_kv*32][d], box 32 rows x 64 elems, 128B swizzle;
                         // quantised: bytes in 128-byte rows, one box = one record
    CUtensorMap map_k16; // same view, box 16 rows x 64 elems (one K or one V tile);
                         // quantised, head_dim 128: box = the 16 rows of a record's K values or of its V values
    CUtensorMap map_sc;  // quantised, head_dim 128: box = one row, a record's K scales or its V scales
};

struct StepDev {
    const SeqMeta* seq_meta;
    const int32_t* tables;
    int32_t n_seqs;
    int32_t n_tokens;
};

struct GeomDev {
    int32_t n_q, n_kv, n_rep, d, page_size, num_pages;
    int32_t tiled;  // 1: rows of a (page, kv head) in the 8-row K/V interleave (see page_row)
};

struct DecodeArgs {
    GeomDev geo;
    const SegInfo* segs;        // n_segs + 1 records (manager.hpp)
    const ItemInfo* items;      // n_items work items in claim order; item c < n_ctas is CTA c's first
    const int32_t* unit_row;    // per unit: page * n_kv + kv head (the record the tile lives in), -1 = bad table entry
    int32_t n_segs, n_items, n_ctas;
    int32_t n_units, tail_pct;  // with n_ctas: enough for CTA c to compute the unit range of its first item (tail_pct 0: one item per CTA)
    const void* q;
    void* out;
    const void* k_new;  // non-null: write the step's new row into its page and attend it (fused append)
    const void* v_new;
    void* arena;        // this layer's pages (for the fused append's global write)
    float* part_o;      // [n_parts][8][d] partial numerators
    float* part_ml;     // [n_parts][8][2] running max (log2 domain) and denominator
    int32_t* seg_counter;    // per segment: tickets of the parts that are done (0 between launches)
    int32_t* work_counters;  // four claim counters; launch i uses slot i % 4 and clears slot (i + 2) % 4
    int32_t work_slot;
    int32_t* status;
    int32_t window;
    float scale_log2;
    int32_t n_stages;   // stages of the CTA's TMA ring
    int32_t comb_cols;  // query columns kept in the merge buffers (n_rep rounded up to even)
    int32_t comb_bufs;  // 1 or 2 merge buffers
    int32_t kv_dep;     // 1: earlier work in the stream wrote this layer's pages or unit_row: the producer waits for it
    uint32_t wait_us;   // limit of every bounded wait on a tile, microseconds
    const uint32_t* in_flag;  // non-null: q, k_new, v_new arrive by copies on another stream, which writes in_seq here after them
    uint32_t in_seq;
    int32_t fault_tile; // test hook: the copy of this tile of CTA 0 is never issued (-1 = none), so its consumer's wait runs out
#ifdef CBKV_MEASURE
    unsigned long long* dbg_buf;  // per-CTA timestamps
    int32_t debug;                // 1 = skip the math, 4 = timestamps, 32/64/128 = skip phases of the int8 tile
#endif
};

struct ChunkArgs {
    StepDev step;
    GeomDev geo;
    const int32_t* item_begin;
    int32_t n_items;
    const void* q;
    void* out;
    int32_t* status;
    int32_t window;
    float scale_log2;
    int32_t rep_slots;  // tcgen05 kernel: q heads per kv head rounded up to a power of two (rows per token in a tile)
    const void* q8_arena;  // two-tile tcgen05 kernel: non-null = the layer's int8 records, read and converted by the kernel itself
    // two-tile tcgen05 kernel: the items from split_first on are cut along K/V into split_parts CTAs each (the
    // last wave of a launch would otherwise leave most SMs idle); each writes its un-normalised rows and their
    // (reference exponent, sum) to split_o / split_ml and draws a ticket from split_counter, the last one
    // merges.  split_parts <= 1: no item is cut.  n_items counts items, the grid has
    // split_first + (n_items - split_first) * split_parts CTAs.
    int32_t split_first, split_parts;
    float* split_o;         // float4 [(item - split_first) * split_parts + part][tile 2][column group 32][row 128]
    float2* split_ml;       // [(item - split_first) * split_parts + part][tile 2][row 128]
    int32_t* split_counter; // per cut item, zero between launches
#ifdef CBKV_MEASURE
    unsigned long long* dbg_buf;  // per-CTA cycle counters of the tcgen05 kernel
#endif
};

struct AppendArgs {
    StepDev step;
    GeomDev geo;
    const void* k;
    const void* v;
    void* arena;
    int32_t* status;
};

struct GenericArgs {
    StepDev step;
    GeomDev geo;
    const void* q;
    void* out;
    const void* arena;
    int32_t* status;
    int32_t window;
    float scale;
};

// Rotate-and-append (rope.cu).  `table` holds, per position, head_dim/2 cosines then head_dim/2 sines in
// the storage type; q_weight / k_weight (head_dim elements, storage type) are null without QK norm.
struct RopeArgs {
    StepDev step;
    GeomDev geo;
    const void* q;
    const void* k;
    const void* v;
    void* q_out;
    void* k_out;   // non-null: rotated k goes here (dense, same layout as k) and v is left alone; `arena` is unused
    void* arena;
    const void* table;
    int64_t max_position;
    const void* q_weight;
    const void* k_weight;
    float eps;
    int32_t gemma;
    int32_t* status;
};

// Decode kernel configuration for a head_dim (0 warps = not supported by the fast path).
struct DecodeConfig { int consumers, stages, smem_bytes, ctas_per_sm, comb_cols, comb_bufs; };
DecodeConfig decode_config(int d, int n_rep, int ctas_per_sm, int stages, int consumers, bool q8 = false);
struct ChunkConfig { int warps, stages, smem_bytes, cols_per_item; };
ChunkConfig chunk_config(int d);

cudaError_t launch_append(const AppendArgs& a, bool bf16, cudaStream_t st);
cudaError_t launch_decode(const CUtensorMap& map, const DecodeArgs& a, int n_ctas, int consumers, int smem_bytes, bool pdl, bool bf16, cudaStream_t st,
                          bool q8 = false);  // q8: the layer holds int8 records, `map` is the byte view with one record per box
cudaError_t launch_chunk(const CUtensorMap& map, const ChunkArgs& a, bool bf16, cudaStream_t st);
cudaError_t launch_generic(const GenericArgs& a, bool bf16, cudaStream_t st);
// unit_row of a decode plan from its segments and the step's block tables (once per step and window);
// zero_a / zero_b (may be null): counters the same launch sets to zero
cudaError_t launch_resolve_units(const SegInfo* segs, int n_segs, const int32_t* tables, int n_kv, int num_pages,
                                 int32_t* unit_row, int n_units, int32_t* status, cudaStream_t st,
                                 int32_t* zero_a = nullptr, int n_a = 0, int32_t* zero_b = nullptr, int n_b = 0);
cudaError_t launch_init_quant(void* arena, size_t n_records, int page_size, int d, cudaStream_t st);
cudaError_t launch_append_quant(const AppendArgs& a, bool bf16, cudaStream_t st);
cudaError_t launch_dequant_pages(const int32_t* tables, int n_entries, const GeomDev& geo, const void* arena, void* scratch,
                                 int32_t* status, bool bf16, cudaStream_t st);
cudaError_t launch_generic_quant(const GenericArgs& a, bool bf16, cudaStream_t st);
cudaError_t launch_rope_append(const RopeArgs& a, bool bf16, cudaStream_t st);
// host side of the rotary tables (rope.cu): frequencies, then [max_position][head_dim] f32 tables
int32_t rope_inv_freq(const cbkv_rope_config& c, std::vector<double>* inv, double* mscale);
void rope_tables(const cbkv_rope_config& c, const std::vector<double>& inv, double mscale, float* cos_out, float* sin_out);
// tcgen05 chunk kernel (prefill_tc.cu): head_dim 64 or 128; `map` is the 16-row box view
bool chunk_tc_supported(int d);
cudaError_t chunk_tc_init();
cudaError_t launch_chunk_tc(const CUtensorMap& map16, const CUtensorMap& map32, const ChunkArgs& a, bool bf16, cudaStream_t st);
// two query tiles per CTA, P in tensor memory (head_dim 128)
bool chunk_tc2_supported(int d);
// int8 layer (a.q8_arena non-null): `map32` = the layer's map_k16, `map_sc` = its map_sc; float layer: map_sc is not used
cudaError_t launch_chunk_tc2(const CUtensorMap& map32, const CUtensorMap& map_sc, const ChunkArgs& a, bool bf16, cudaStream_t st);
cudaError_t kernels_init();  // raises the dynamic shared memory limits once per process

}  // namespace cbkv
