// cbkv_decode_attention_static: decode attention over caller-owned pages that
// allocates no device memory.
//
// Who needs this: code that is not allowed to call cudaMalloc while it runs — a
// serving loop that has handed the whole GPU to its own pool allocator up front, a
// plugin loaded into a host process that forbids allocations after start-up, a
// latency-critical path where an allocation could block on the driver.  Such a
// caller already owns the KV pages and the block tables; all this entry point still
// needs is the decode kernel's working memory (work split, per-segment tickets,
// partial results).  Here that working memory is a fixed array that is part of the
// library image, so every GPU that loads the library pays for it once (about 10 MB)
// and nothing is ever allocated or freed.
//
// Consequences of the fixed array:
//   - problem sizes are capped (see the limits below) and larger ones are refused;
//   - all calls on a device share the one array and it keeps whatever the last call
//     left in it; the parts that must start at zero are cleared at the start of every
//     call, on the caller's stream;
//   - two calls that overlap on the GPU (different streams, no dependency between
//     them) would write the same array and corrupt each other: keep calls on one
//     stream or order them yourself;
//   - the first call on a device looks the array's address up and raises the kernel's
//     shared-memory limit; make that first call before starting any stream capture;
//   - the kernel's status word (a bad block-table entry, a wait that ran out) lives in the
//     same array and is cleared by every call: read it with cbkv_static_status afterwards.
#include <cuda.h>
#include <cuda_runtime.h>

#include <mutex>
#include <string>
#include <vector>

#include "kernels.hpp"
#include "manager.hpp"

using namespace cbkv;

namespace {

// ---- limits of the static working memory
constexpr int kMaxSeqs = 128;        // sequences per call
constexpr int kMaxSegs = 1024;       // sequences x kv heads
constexpr int kMaxItems = 296 * 8;   // work items the launch is cut into
constexpr int kMaxParts = 1024;      // partial results (segments cut across items)
constexpr int kMaxUnits = 1 << 18;   // (sequence, kv head, visible page) triples
constexpr int kMaxHeadDim = 256;

// ---- layout of the array (byte offsets, all multiples of 256)
constexpr size_t kOffStatus = 0;                                              // 1 int
constexpr size_t kOffWork = 64;                                               // 4 claim counters, 0 at launch
constexpr size_t kOffCounters = 256;                                          // kMaxSegs tickets, 0 at launch
constexpr size_t kOffSegs = kOffCounters + kMaxSegs * 4;                      // kMaxSegs + 1 segment records
constexpr size_t kOffItems = (kOffSegs + (kMaxSegs + 1) * sizeof(SegInfo) + 255) / 256 * 256;  // item records
constexpr size_t kOffUnits = (kOffItems + kMaxItems * sizeof(ItemInfo) + 255) / 256 * 256;     // kMaxUnits ints
constexpr size_t kOffPartMl = kOffUnits + (size_t)kMaxUnits * 4;              // kMaxParts x 8 x 2 floats
constexpr size_t kOffPartO = kOffPartMl + (size_t)kMaxParts * 16 * 4;         // kMaxParts x 8 x head_dim floats
constexpr size_t kScratchBytes = kOffPartO + (size_t)kMaxParts * 8 * kMaxHeadDim * 4;

// The working memory itself.  In host code this name is only a handle for
// cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) unsigned char g_static_scratch[kScratchBytes];

struct PerDevice {
    bool ready = false;
    unsigned char* scratch = nullptr;  // device address of g_static_scratch on this device
    int sm_count = 0;
};
PerDevice g_dev[64];
std::mutex g_mu;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int32_t fail(int32_t code, const std::string& msg) {
    set_error(msg);
    return code;
}

// Once per device, with that device current: resolve the array's device address.
int32_t setup_current_device(PerDevice** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(CBKV_ERR_CUDA, std::string("cudaGetDevice: ") + cudaGetErrorString(e));
    if (dev < 0 || dev >= 64) return fail(CBKV_ERR_ARG, "device ordinal out of range");
    std::lock_guard<std::mutex> lock(g_mu);
    PerDevice& pd = g_dev[dev];
    if (!pd.ready) {
        int major = 0;
        e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
        if (e != cudaSuccess) return fail(CBKV_ERR_CUDA, std::string("cudaDeviceGetAttribute: ") + cudaGetErrorString(e));
        if (major < 10) return fail(CBKV_ERR_CUDA, "this library is built for sm_100a (B200) only");
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || !p) return fail(CBKV_ERR_CUDA, std::string("cudaGetSymbolAddress: ") + cudaGetErrorString(e));
        e = cudaDeviceGetAttribute(&pd.sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return fail(CBKV_ERR_CUDA, std::string("cudaDeviceGetAttribute: ") + cudaGetErrorString(e));
        e = kernels_init();  // raises the kernels' dynamic shared memory limit; allocates nothing
        if (e != cudaSuccess) return fail(CBKV_ERR_CUDA, std::string("kernels_init: ") + cudaGetErrorString(e));
        pd.scratch = static_cast<unsigned char*>(p);
        pd.ready = true;
    }
    *out = &pd;
    return CBKV_OK;
}

}  // namespace

extern "C" int32_t cbkv_decode_attention_static(const void* kv_pages, int64_t num_pages, const int32_t* block_tables,
                                                int32_t table_stride, const int32_t* seq_lens_host, int32_t n_seqs,
                                                int32_t n_q_heads, int32_t n_kv_heads, int32_t head_dim, int32_t dtype,
                                                const void* q, void* out, double scale, int64_t window, void* stream) {
    return fenced([&]() -> int32_t {
    if (!kv_pages || !block_tables || !seq_lens_host || !q || !out) return fail(CBKV_ERR_ARG, "null argument");
    if (n_seqs < 1 || n_q_heads < 1 || n_kv_heads < 1 || n_q_heads % n_kv_heads != 0 || num_pages < 1 || table_stride < 1)
        return fail(CBKV_ERR_ARG, "invalid geometry");
    if (dtype != CBKV_F16 && dtype != CBKV_BF16) return fail(CBKV_ERR_ARG, "dtype must be CBKV_F16 or CBKV_BF16");
    if (window != 0 && window < 2) return fail(CBKV_ERR_ARG, "sliding window must be >= 2, got " + std::to_string(window));
    const int n_rep = n_q_heads / n_kv_heads;
    if (!(head_dim == 64 || head_dim == 128 || head_dim == 256) || n_rep > 8)
        return fail(CBKV_ERR_ARG, "static decode supports head_dim 64/128/256 and at most 8 q heads per kv head");
    if (n_seqs > kMaxSeqs || (int64_t)n_seqs * n_kv_heads > kMaxSegs)
        return fail(CBKV_ERR_ARG, "too large for the static working memory: at most " + std::to_string(kMaxSeqs) +
                                      " sequences and " + std::to_string(kMaxSegs) + " sequence x kv-head pairs per call");
    if ((uint64_t)num_pages * n_kv_heads * 32 >= (1ull << 32)) return fail(CBKV_ERR_ARG, "arena too large for one tensor map");

    PerDevice* pd = nullptr;
    int32_t rc = setup_current_device(&pd);
    if (rc) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);

    // host-side work split (host heap only)
    Arena tmp;
    tmp.cfg.page_size = 16;
    tmp.cfg.n_kv_heads = n_kv_heads;
    tmp.cfg.n_q_heads = n_q_heads;
    tmp.cfg.head_dim = head_dim;
    tmp.step_meta.resize((size_t)n_seqs);
    for (int b = 0; b < n_seqs; b++) {
        const int32_t L = seq_lens_host[b];
        if (L < 1 || (L + 15) / 16 > table_stride) return fail(CBKV_ERR_ARG, "sequence length outside its block table");
        tmp.step_meta[(size_t)b] = SeqMeta{L - 1, 1, b, b * table_stride};
    }
    const DecodeConfig dc = decode_config(head_dim, n_rep, 0, 0, 0);
    DecodePlan pl;
    DecodeSplit split;
    int n_ctas = pd->sm_count * dc.ctas_per_sm;
    for (;;) {
        build_decode_plan(tmp, window, n_ctas, split, &pl);
        const int want = std::max(1, (pl.n_units + dc.consumers - 1) / dc.consumers);
        if (want < pl.n_ctas) build_decode_plan(tmp, window, want, split, &pl);
        if ((pl.n_parts <= kMaxParts && pl.n_items <= kMaxItems) || (n_ctas == 1 && split.min_item == 0)) break;
        if (split.min_item != 0) split.min_item = 0;  // first give up the dynamically claimed tail items,
        else n_ctas = std::max(1, n_ctas / 2);        // then CTAs: fewer cuts either way
    }
    if (pl.n_parts > kMaxParts || pl.n_items > kMaxItems)
        return fail(CBKV_ERR_ARG, "too many partial results for the static working memory");
    if (pl.n_units > kMaxUnits)
        return fail(CBKV_ERR_ARG, "too large for the static working memory: at most " + std::to_string(kMaxUnits) +
                                      " (sequence, kv head, page) triples per call");

    unsigned char* S = pd->scratch;
    cudaError_t e;
    // what must start at zero: the status word, the claim counters and the per-segment tickets
    e = cudaMemsetAsync(S + kOffStatus, 0, kOffSegs - kOffStatus, st);
    if (e != cudaSuccess) return fail(CBKV_ERR_CUDA, std::string("cudaMemsetAsync: ") + cudaGetErrorString(e));
    e = cudaMemcpyAsync(S + kOffSegs, pl.segs.data(), pl.segs.size() * sizeof(SegInfo), cudaMemcpyHostToDevice, st);
    if (e != cudaSuccess) return fail(CBKV_ERR_CUDA, std::string("cudaMemcpyAsync: ") + cudaGetErrorString(e));
    e = cudaMemcpyAsync(S + kOffItems, pl.items.data(), pl.items.size() * sizeof(ItemInfo), cudaMemcpyHostToDevice, st);
    if (e != cudaSuccess) return fail(CBKV_ERR_CUDA, std::string("cudaMemcpyAsync: ") + cudaGetErrorString(e));
    // the host vectors go out of scope on return: the copies above come from pageable
    // memory, which the runtime stages before returning
    const SegInfo* segs = reinterpret_cast<const SegInfo*>(S + kOffSegs);
    int32_t* unit_row = reinterpret_cast<int32_t*>(S + kOffUnits);
    int32_t* status = reinterpret_cast<int32_t*>(S + kOffStatus);
    e = launch_resolve_units(segs, pl.n_segs, block_tables, n_kv_heads, (int)num_pages, unit_row, pl.n_units, status, st);
    if (e != cudaSuccess) return fail(CBKV_ERR_CUDA, std::string("launch: ") + cudaGetErrorString(e));

    // tensor map over the caller's pages: rows = pages x kv heads x 32, box 32 rows x 64 elements, 128-byte swizzle
    static EncodeTiledFn encode = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_mu);
        if (!encode) {
            void* fp = nullptr;
            cudaDriverEntryPointQueryResult qr;
            if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fp, cudaEnableDefault, &qr) != cudaSuccess || qr != cudaDriverEntryPointSuccess)
                return fail(CBKV_ERR_CUDA, "cuTensorMapEncodeTiled not available from the driver");
            encode = reinterpret_cast<EncodeTiledFn>(fp);
        }
    }
    CUtensorMap map;
    {
        cuuint64_t dims[2] = {(cuuint64_t)head_dim, (cuuint64_t)num_pages * n_kv_heads * 32};
        cuuint64_t strides[1] = {(cuuint64_t)head_dim * 2};
        cuuint32_t box[2] = {64, 32};
        cuuint32_t estr[2] = {1, 1};
        CUresult r = encode(&map, dtype == CBKV_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                            const_cast<void*>(kv_pages), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(CBKV_ERR_CUDA, "cuTensorMapEncodeTiled failed: " + std::to_string((int)r));
    }

    DecodeArgs args{};
    args.geo = GeomDev{n_q_heads, n_kv_heads, n_rep, head_dim, 16, (int32_t)num_pages, 1};
    args.segs = segs;
    args.items = reinterpret_cast<const ItemInfo*>(S + kOffItems);
    args.unit_row = unit_row;
    args.n_segs = pl.n_segs; args.n_items = pl.n_items; args.n_ctas = pl.n_ctas;
    args.n_units = pl.n_units; args.tail_pct = pl.levels > 1 ? split.tail_pct : 0;
    args.q = q; args.out = out; args.k_new = nullptr; args.v_new = nullptr; args.arena = nullptr;
    args.part_o = reinterpret_cast<float*>(S + kOffPartO);
    args.part_ml = reinterpret_cast<float*>(S + kOffPartMl);
    args.seg_counter = reinterpret_cast<int32_t*>(S + kOffCounters);
    args.work_counters = reinterpret_cast<int32_t*>(S + kOffWork);
    args.work_slot = 0;
    args.status = status;
    args.window = (int32_t)window;
    args.scale_log2 = (float)(scale * 1.4426950408889634);
    args.n_stages = dc.stages; args.comb_cols = dc.comb_cols; args.comb_bufs = dc.comb_bufs;
    args.kv_dep = 1;  // the pages are the caller's: assume the previous work in the stream wrote them
    args.wait_us = 100000; args.fault_tile = -1;
    e = launch_decode(map, args, pl.n_ctas, dc.consumers, dc.smem_bytes, /*pdl=*/false, dtype == CBKV_BF16, st);
    if (e != cudaSuccess) return fail(CBKV_ERR_CUDA, std::string("launch: ") + cudaGetErrorString(e));
    return CBKV_OK;
    });
}

// Reads and clears the status word of the entry point above on the current device.  Waits for
// `stream`; allocates nothing (one 4-byte copy each way).
extern "C" int32_t cbkv_static_status(void* stream, int32_t* status) {
    return fenced([&]() -> int32_t {
    if (!status) return fail(CBKV_ERR_ARG, "null argument");
    *status = 0;
    PerDevice* pd = nullptr;
    int32_t rc = setup_current_device(&pd);
    if (rc) return rc;
    cudaError_t e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(CBKV_ERR_CUDA, std::string("cudaStreamSynchronize: ") + cudaGetErrorString(e));
    e = cudaMemcpy(status, pd->scratch + kOffStatus, sizeof(int32_t), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return fail(CBKV_ERR_CUDA, std::string("cudaMemcpy: ") + cudaGetErrorString(e));
    if (*status) {
        e = cudaMemset(pd->scratch + kOffStatus, 0, sizeof(int32_t));
        if (e != cudaSuccess) return fail(CBKV_ERR_CUDA, std::string("cudaMemset: ") + cudaGetErrorString(e));
        return fail(CBKV_ERR_DEVICE, "kernel status word = " + std::to_string(*status));
    }
    return CBKV_OK;
    });
}
