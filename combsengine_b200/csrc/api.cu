// extern "C" boundary (include/combs_kv.h) and the device-side state behind it:
// lazily materialised per-layer arenas, TMA descriptors, per-step metadata upload,
// kernel selection and launch.  The host bookkeeping itself is manager.cpp.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <nvtx3/nvToolsExt.h>

#include <atomic>
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

#include "kernels.hpp"
#include "manager.hpp"

using namespace cbkv;

namespace {

std::atomic<int64_t> g_launches{0};

// NVTX range around the host side of an entry point (header-only NVTX: a no-op unless a profiler
// that collects NVTX is attached).
struct NvtxRange {
    explicit NvtxRange(const char* name) { nvtxRangePushA(name); }
    NvtxRange(const char* name, int layer) {
        char buf[48];
        snprintf(buf, sizeof buf, "%s L%d", name, layer);
        nvtxRangePushA(buf);
    }
    ~NvtxRange() { nvtxRangePop(); }
    NvtxRange(const NvtxRange&) = delete;
    NvtxRange& operator=(const NvtxRange&) = delete;
};

#define CU_TRY(expr)                                                                     \
    do {                                                                                 \
        cudaError_t e__ = (expr);                                                        \
        if (e__ != cudaSuccess) {                                                        \
            set_error(std::string(#expr) + ": " + cudaGetErrorString(e__));              \
            return CBKV_ERR_CUDA;                                                        \
        }                                                                                \
    } while (0)

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

constexpr int kSlots = 4;

struct StepSlot {
    uint8_t* host = nullptr;  // pinned
    uint8_t* dev = nullptr;
    size_t cap = 0, used = 0;
    size_t flushed = 0;       // bytes of `host` already on their way to `dev` (slot_upload only fills the pinned mirror;
                              // flush_uploads sends everything new in one copy, right before the kernel that needs it)
    cudaEvent_t ev = nullptr;
    bool pending = false;
};

struct DecodePlanDev {
    DecodePlan host;
    const SegInfo* segs = nullptr;     // in the step slot
    const ItemInfo* items = nullptr;   // in the step slot
    size_t unit_row_off = 0;           // offset (ints) of this plan's unit_row in DeviceState::unit_rows
    bool fresh = true;                 // unit_row was written by a kernel no decode launch has waited for yet
};

struct DeviceState {
    int device = 0;
    int sm_count = 148;
    bool fast = false;  // page 16, head_dim in {64,128,256}, n_rep <= 8: the TMA + mma kernels apply
    size_t layer_bytes = 0;
    std::vector<LayerArena> layers;
    StepSlot slots[kSlots];
    int cur = 0;
    uint64_t uploaded_step = 0;
    StepDev step{};
    std::map<std::pair<int64_t, int>, DecodePlanDev> decode_plans;  // by (window, consumer warps)
    int32_t* unit_rows = nullptr;  // unit_row arrays of the step's plans, one after the other
    size_t unit_rows_cap = 0, unit_rows_used = 0;
    int32_t* work_counters = nullptr;  // four claim counters of the decode kernel, rotating per launch
    uint32_t launch_seq = 0;
    DecodeSplit split;
    uint32_t wait_us = 100000;  // limit of the kernels' bounded waits
    int32_t fault_tile = -1;    // test hook, see cbkv_debug_set_wait_limit
    bool chunk_plan_ok = false;
    ChunkPlan chunk_host;
    const int32_t* chunk_item_begin = nullptr;
    bool tc_ok = false;       // the tcgen05 chunk kernel covers this geometry
    int chunk_mode = 0;       // cbkv_set_chunk_kernel: 0 = choose, 1 = mma.sync, 2 = tcgen05 one tile, 3 = two tiles, 4 = two tiles, int8 records converted in the kernel
    bool tile_plan_ok = false;
    int tile_plan_tokens = 0;  // tokens per work item the tile plan was built for
    ChunkPlan tile_host;
    const int32_t* tile_item_begin = nullptr;
    float* part_o = nullptr;
    float* part_ml = nullptr;
    size_t part_cap = 0;
    int32_t* seg_counter = nullptr;
    size_t counter_cap = 0;
    int32_t* status = nullptr;
    int decode_ctas_per_sm = 0, decode_stages = 0, decode_consumers = 0, decode_max_ctas = 0;
    bool pdl = true;
    bool host_direct = true;  // cbkv_set_host_route
    bool zero_pending = false; // the step's first unit-table kernel still has to zero the decode kernels' counters
    // two-tile chunk kernel: slices of the items of a launch's last, mostly empty wave (ChunkArgs::split_*)
    int chunk_split = 4;               // most slices per item, 1 = never cut (cbkv_set_chunk_split)
    float* split_o = nullptr;
    float2* split_ml = nullptr;
    int32_t* split_counter = nullptr;
    int split_cap = 0;                 // slices the buffers hold
    int last_kv_writer = -1;  // layer whose pages the most recent launch wrote (-1: none since the last upload)
    // host-buffer entry point staging
    uint8_t* io = nullptr;
    size_t io_cap = 0;
    // one float layer that int8 layers are de-quantised into for the tensor-core chunk kernels
    LayerArena qscratch;
    // rotated q of the current layer (cbkv_attention_rope)
    uint8_t* qrot = nullptr;
    size_t qrot_cap = 0;
    // pipelined host-buffer entry point: copy streams, rotating staging slots
    struct IoSlot {
        uint8_t* dev = nullptr;
        size_t cap = 0;
        cudaEvent_t in_done = nullptr, k_done = nullptr, out_done = nullptr;
        bool used = false;
    };
    static constexpr int kIoSlots = 32;
    IoSlot io_slots[kIoSlots];
    int io_cur = 0;
    cudaStream_t h2d = nullptr, d2h = nullptr;
    // Decode steps do not make the compute stream wait for the input copies' event (a wait between two
    // kernels ends the overlap of consecutive launches; an event record does not): the kernel itself waits for
    // a number that the copy stream writes behind its inputs (DecodeArgs::in_flag).
    uint32_t* in_flags = nullptr;      // device, one per slot
    uint32_t* in_seq_host = nullptr;   // pinned, the source of each slot's flag copy
    uint32_t in_seq = 0;
    const uint32_t* next_in_flag = nullptr;  // handed to the next decode launch
    uint32_t next_in_seq = 0;
#ifdef CBKV_MEASURE
    unsigned long long* dbg_buf = nullptr;  // per-CTA timestamps / cycle counters of the last launch
    int dbg_ctas = 0;
    int dbg_chain_last = -1;
#endif
    // profiling
    bool profile = false;
    std::vector<std::pair<cudaEvent_t, cudaEvent_t>> prof;
    size_t prof_used = 0;
};

DeviceState* dev_of(Arena* a) { return static_cast<DeviceState*>(a->dev); }

int32_t ensure_device(Arena* a) {
    if (a->dev) {
        CU_TRY(cudaSetDevice(dev_of(a)->device));
        return CBKV_OK;
    }
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) {
        set_error(std::string("no CUDA device: this library has no CPU path (") + cudaGetErrorString(e) + ")");
        return CBKV_ERR_CUDA;
    }
    CU_TRY(cudaSetDevice(a->cfg.device));
    cudaDeviceProp prop;
    CU_TRY(cudaGetDeviceProperties(&prop, a->cfg.device));
    if (prop.major < 10) {
        set_error("this library is built for sm_100a (B200) only; found sm_" + std::to_string(prop.major * 10 + prop.minor));
        return CBKV_ERR_CUDA;
    }
    auto* d = new DeviceState();
    d->device = a->cfg.device;
    d->sm_count = prop.multiProcessorCount;
    const int D = a->cfg.head_dim;
    d->fast = a->cfg.page_size == 16 && (D == 64 || D == 128 || D == 256) && a->n_rep() <= 8;
    if (!d->fast && D > 512) { delete d; set_error("head_dim > 512 is not supported"); return CBKV_ERR_ARG; }
    d->layer_bytes = (size_t)a->num_pages * a->cfg.n_kv_heads * 2 * a->cfg.page_size * D * 2;
    d->layers.resize((size_t)a->cfg.num_layers);
    if (d->fast) {
        cudaError_t ke = kernels_init();
        if (ke != cudaSuccess) { delete d; set_error(std::string("kernels_init: ") + cudaGetErrorString(ke)); return CBKV_ERR_CUDA; }
        if (!encode_fn()) { delete d; set_error("cuTensorMapEncodeTiled not available from the driver"); return CBKV_ERR_CUDA; }
        if (chunk_tc_supported(D)) {
            ke = chunk_tc_init();
            if (ke != cudaSuccess) { delete d; set_error(std::string("chunk_tc_init: ") + cudaGetErrorString(ke)); return CBKV_ERR_CUDA; }
            d->tc_ok = true;
        }
    }
    cudaError_t se = cudaMalloc(&d->status, sizeof(int32_t));
    if (se != cudaSuccess) { delete d; set_error(std::string("cudaMalloc: ") + cudaGetErrorString(se)); return CBKV_ERR_CUDA; }
    cudaMemset(d->status, 0, sizeof(int32_t));
    for (auto& s : d->slots) cudaEventCreateWithFlags(&s.ev, cudaEventDisableTiming);
    a->dev = d;
    return CBKV_OK;
}

#ifdef CBKV_MEASURE
// Measurement build only (python -m combsengine_b200._build --measure): switches read from CBKV_DEBUG.
int debug_flags() {
    static int f = -1;
    if (f < 0) { const char* e = getenv("CBKV_DEBUG"); f = e ? atoi(e) : 0; }
    return f;
}
#else
constexpr int debug_flags() { return 0; }  // the product build ignores the environment
#endif

int32_t encode_map(CUtensorMap* map, bool bf16, void* base, uint64_t rows, int D, int box_rows) {
    cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)D * 2};
    cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = encode_fn()(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, base, dims,
                             strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed: " + std::to_string((int)r)); return CBKV_ERR_CUDA; }
    return CBKV_OK;
}

int32_t alloc_float_layer(Arena* a, LayerArena* Lp, cudaStream_t st);

// Arenas appear on a layer's first write, zero-filled (kv.rs:695-713).
int32_t materialize(Arena* a, int layer, cudaStream_t st) {
    DeviceState* d = dev_of(a);
    LayerArena& L = d->layers[(size_t)layer];
    if (L.base) return CBKV_OK;
    if (a->layer_quant(layer)) {  // Arena::Quant, zero-filled (kv.rs:699-705)
        const size_t bytes = (size_t)a->num_pages * a->cfg.n_kv_heads * qrec_bytes(a->cfg.page_size, a->cfg.head_dim);
        CU_TRY(cudaMalloc(&L.base, bytes));
        CU_TRY(launch_init_quant(L.base, (size_t)a->num_pages * a->cfg.n_kv_heads, a->cfg.page_size, a->cfg.head_dim, st));
        L.quant = true;
        if (d->fast) {
            // the decode kernel fetches one record per copy: a byte tensor of 128-byte rows, one box = one record
            const uint64_t rec_rows = qrec_bytes(16, a->cfg.head_dim) / 128;
            const uint64_t rows = (uint64_t)a->num_pages * a->cfg.n_kv_heads * rec_rows;
            if (rows >= (1ull << 31)) { set_error("arena too large for one tensor map"); return CBKV_ERR_ARG; }
            cuuint64_t dims[2] = {128, (cuuint64_t)rows};
            cuuint64_t strides[1] = {128};
            cuuint32_t box[2] = {128, (cuuint32_t)rec_rows};
            cuuint32_t estr[2] = {1, 1};
            CUresult r = encode_fn()(&L.map_kv, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, L.base, dims, strides, box, estr,
                                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled (int8 records) failed: " + std::to_string((int)r)); return CBKV_ERR_CUDA; }
            if (a->cfg.head_dim == 128) {
                // the two-tile chunk kernel fetches K and V of a record separately: rows 0-15 K values, 16-31 V
                // values, row 32 K scales, row 33 V scales
                cuuint32_t box_values[2] = {128, 16}, box_scales[2] = {128, 1};
                r = encode_fn()(&L.map_k16, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, L.base, dims, strides, box_values, estr,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
                if (r == CUDA_SUCCESS)
                    r = encode_fn()(&L.map_sc, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, L.base, dims, strides, box_scales, estr,
                                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
                if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled (int8 half-records) failed: " + std::to_string((int)r)); return CBKV_ERR_CUDA; }
            }
        }
        return CBKV_OK;
    }
    return alloc_float_layer(a, &L, st);
}

int32_t alloc_float_layer(Arena* a, LayerArena* Lp, cudaStream_t st) {
    DeviceState* d = dev_of(a);
    LayerArena& L = *Lp;
    CU_TRY(cudaMalloc(&L.base, d->layer_bytes));
    CU_TRY(cudaMemsetAsync(L.base, 0, d->layer_bytes, st));
    if (d->fast) {
        uint64_t rows = (uint64_t)a->num_pages * a->cfg.n_kv_heads * 32;
        if (rows >= (1ull << 32)) { set_error("arena too large for one tensor map"); return CBKV_ERR_ARG; }
        bool bf16 = a->cfg.dtype == CBKV_BF16;
        int32_t rc = encode_map(&L.map_kv, bf16, L.base, rows, a->cfg.head_dim, 32);
        if (rc) return rc;
        rc = encode_map(&L.map_k16, bf16, L.base, rows, a->cfg.head_dim, 16);
        if (rc) return rc;
    }
    return CBKV_OK;
}

// Bump-allocate `bytes` in the current step slot, copy `src` there and enqueue the
// upload; returns the device address.
int32_t slot_upload(DeviceState* d, const void* src, size_t bytes, cudaStream_t st, const void** dev_out) {
    StepSlot& s = d->slots[d->cur];
    size_t off = (s.used + 255) & ~(size_t)255;
    if (off + bytes > s.cap) {
        // grow: nothing of this slot may still be in flight
        CU_TRY(cudaStreamSynchronize(st));
        size_t ncap = std::max<size_t>((off + bytes) * 2, 1 << 20);
        uint8_t *nh = nullptr, *nd = nullptr;
        CU_TRY(cudaMallocHost(&nh, ncap));
        CU_TRY(cudaMalloc(&nd, ncap));
        if (s.used) {
            memcpy(nh, s.host, s.used);
            CU_TRY(cudaMemcpy(nd, s.dev, s.used, cudaMemcpyDeviceToDevice));
        }
        // earlier uploads of this step keep their offsets; re-point what was handed out
        ptrdiff_t delta = nd - s.dev;
        if (s.dev) {
            auto fix = [&](const void*& p) { if (p) p = (const uint8_t*)p + delta; };
            const void* p;
            p = d->step.seq_meta; fix(p); d->step.seq_meta = (const SeqMeta*)p;
            p = d->step.tables; fix(p); d->step.tables = (const int32_t*)p;
            for (auto& kv : d->decode_plans) {
                DecodePlanDev& pd = kv.second;
                p = pd.segs; fix(p); pd.segs = (const SegInfo*)p;
                p = pd.items; fix(p); pd.items = (const ItemInfo*)p;
            }
            p = d->chunk_item_begin; fix(p); d->chunk_item_begin = (const int32_t*)p;
            p = d->tile_item_begin; fix(p); d->tile_item_begin = (const int32_t*)p;
            cudaFreeHost(s.host);
            cudaFree(s.dev);
        }
        s.host = nh; s.dev = nd; s.cap = ncap;
    }
    memcpy(s.host + off, src, bytes);
    s.used = off + bytes;
    *dev_out = s.dev + off;
    return CBKV_OK;
}

// Everything slot_upload has put into the current step slot since the last call goes to the device in one
// copy (a decode step uploads the sequences' records, the block tables and the work split: three pieces, one
// copy).  Called in front of every launch that reads the slot.
int32_t flush_uploads(DeviceState* d, cudaStream_t st) {
    StepSlot& s = d->slots[d->cur];
    if (s.flushed >= s.used) return CBKV_OK;
    CU_TRY(cudaMemcpyAsync(s.dev + s.flushed, s.host + s.flushed, s.used - s.flushed, cudaMemcpyHostToDevice, st));
    CU_TRY(cudaEventRecord(s.ev, st));
    s.pending = true;
    s.flushed = s.used;
    return CBKV_OK;
}

int32_t upload_step(Arena* a, cudaStream_t st) {
    DeviceState* d = dev_of(a);
    d->cur = (d->cur + 1) % kSlots;
    StepSlot& s = d->slots[d->cur];
    if (s.pending) { CU_TRY(cudaEventSynchronize(s.ev)); s.pending = false; }
    s.used = 0;
    s.flushed = 0;
    d->decode_plans.clear();
    d->chunk_plan_ok = false;
    d->chunk_item_begin = nullptr;
    d->tile_plan_ok = false;
    d->tile_item_begin = nullptr;
    d->step = StepDev{};
    d->last_kv_writer = -1;  // the upload is a full stream dependency
    d->unit_rows_used = 0;
    // tickets and claim counters start every step at zero, whatever an earlier launch that gave up left behind:
    // the decode kernels' by the step's first unit-table kernel (get_decode_plan), the chunk kernel's here
    d->zero_pending = true;
    if (d->split_counter && !a->step_is_decode) CU_TRY(cudaMemsetAsync(d->split_counter, 0, (size_t)d->split_cap * sizeof(int32_t), st));
    if (a->step_meta.empty()) {  // an empty step: nothing to upload, nothing will launch
        d->uploaded_step = a->step_id;
        return CBKV_OK;
    }
    const void* p = nullptr;
    int32_t rc = slot_upload(d, a->step_meta.data(), a->step_meta.size() * sizeof(SeqMeta), st, &p);
    if (rc) return rc;
    d->step.seq_meta = (const SeqMeta*)p;
    rc = slot_upload(d, a->step_tables.data(), std::max<size_t>(1, a->step_tables.size()) * sizeof(int32_t), st, &p);
    if (rc) return rc;
    d->step.tables = (const int32_t*)p;
    d->step.n_seqs = (int32_t)a->step_meta.size();
    d->step.n_tokens = (int32_t)a->step_tokens;
    d->uploaded_step = a->step_id;
    return CBKV_OK;
}

GeomDev geom(const Arena* a) {
    return GeomDev{a->cfg.n_q_heads, a->cfg.n_kv_heads, a->cfg.n_q_heads / a->cfg.n_kv_heads, a->cfg.head_dim,
                   a->cfg.page_size, (int32_t)a->num_pages, (a->dev && dev_of(const_cast<Arena*>(a))->fast) ? 1 : 0};
}

int32_t get_decode_plan(Arena* a, int64_t window, bool quant, cudaStream_t st, DecodePlanDev** out) {
    DeviceState* d = dev_of(a);
    DecodeConfig dc = decode_config(a->cfg.head_dim, a->n_rep(), d->decode_ctas_per_sm, d->decode_stages, d->decode_consumers, quant);
    const auto key = std::make_pair(window, dc.consumers);
    auto it = d->decode_plans.find(key);
    if (it != d->decode_plans.end()) { *out = &it->second; return CBKV_OK; }
    DecodePlanDev pd{};
    // at least one page per consumer warp, at most one resident wave of CTAs
    int max_ctas = d->sm_count * dc.ctas_per_sm;
    if (d->decode_max_ctas > 0) max_ctas = std::min(max_ctas, d->decode_max_ctas);
    build_decode_plan(*a, window, max_ctas, d->split, &pd.host);
    {
        int want = std::max(1, (pd.host.n_units + dc.consumers - 1) / dc.consumers);
        if (want < pd.host.n_ctas) build_decode_plan(*a, window, want, d->split, &pd.host);
    }
    // segment and item records in one upload
    const size_t seg_bytes = pd.host.segs.size() * sizeof(SegInfo), item_bytes = pd.host.items.size() * sizeof(ItemInfo);
    std::vector<uint8_t> flat(seg_bytes + item_bytes);
    memcpy(flat.data(), pd.host.segs.data(), seg_bytes);
    memcpy(flat.data() + seg_bytes, pd.host.items.data(), item_bytes);
    const void* p = nullptr;
    int32_t rc = slot_upload(d, flat.data(), flat.size(), st, &p);
    if (rc) return rc;
    pd.segs = reinterpret_cast<const SegInfo*>(p);
    pd.items = reinterpret_cast<const ItemInfo*>(reinterpret_cast<const uint8_t*>(p) + seg_bytes);
    // scratch for partial results and the per-segment tickets
    if ((size_t)pd.host.n_parts > d->part_cap) {
        CU_TRY(cudaStreamSynchronize(st));
        if (d->part_o) { cudaFree(d->part_o); cudaFree(d->part_ml); }
        d->part_o = d->part_ml = nullptr;
        d->part_cap = std::max<size_t>((size_t)pd.host.n_parts * 2, 2048);
        CU_TRY(cudaMalloc(&d->part_o, d->part_cap * 8 * a->cfg.head_dim * sizeof(float)));
        CU_TRY(cudaMalloc(&d->part_ml, d->part_cap * 16 * sizeof(float)));
    }
    if ((size_t)pd.host.n_segs > d->counter_cap) {
        CU_TRY(cudaStreamSynchronize(st));
        if (d->seg_counter) cudaFree(d->seg_counter);
        d->seg_counter = nullptr;
        d->counter_cap = std::max<size_t>((size_t)pd.host.n_segs * 2, 1024);
        CU_TRY(cudaMalloc(&d->seg_counter, d->counter_cap * sizeof(int32_t)));
        CU_TRY(cudaMemsetAsync(d->seg_counter, 0, d->counter_cap * sizeof(int32_t), st));
    }
    if (!d->work_counters) {
        CU_TRY(cudaMalloc(&d->work_counters, 4 * sizeof(int32_t)));
        CU_TRY(cudaMemsetAsync(d->work_counters, 0, 4 * sizeof(int32_t), st));
    }
    // the record index of every unit, resolved through the block tables once for all layers of the step
    const size_t need = d->unit_rows_used + (size_t)pd.host.n_units;
    if (need > d->unit_rows_cap) {
        CU_TRY(cudaStreamSynchronize(st));
        const size_t ncap = std::max<size_t>(need * 2, (size_t)1 << 18);
        int32_t* nb = nullptr;
        CU_TRY(cudaMalloc(&nb, ncap * sizeof(int32_t)));
        if (d->unit_rows) {
            if (d->unit_rows_used) CU_TRY(cudaMemcpy(nb, d->unit_rows, d->unit_rows_used * sizeof(int32_t), cudaMemcpyDeviceToDevice));
            cudaFree(d->unit_rows);
        }
        d->unit_rows = nb;
        d->unit_rows_cap = ncap;
    }
    pd.unit_row_off = d->unit_rows_used;
    d->unit_rows_used = need;
    { int32_t frc = flush_uploads(d, st); if (frc) return frc; }
    CU_TRY(launch_resolve_units(pd.segs, pd.host.n_segs, d->step.tables, a->cfg.n_kv_heads, (int)a->num_pages,
                                d->unit_rows + pd.unit_row_off, pd.host.n_units, d->status, st,
                                d->zero_pending ? d->seg_counter : nullptr, (int)d->counter_cap,
                                d->zero_pending ? d->work_counters : nullptr, 4));
    d->zero_pending = false;
    g_launches++;
    pd.fresh = true;
    auto ins = d->decode_plans.emplace(key, std::move(pd));
    *out = &ins.first->second;
    return CBKV_OK;
}

int32_t get_chunk_plan(Arena* a, cudaStream_t st) {
    DeviceState* d = dev_of(a);
    if (d->chunk_plan_ok) return CBKV_OK;
    build_chunk_plan(*a, chunk_config(a->cfg.head_dim).cols_per_item, &d->chunk_host);
    const void* p = nullptr;
    int32_t rc = slot_upload(d, d->chunk_host.item_begin.data(), d->chunk_host.item_begin.size() * sizeof(int32_t), st, &p);
    if (rc) return rc;
    d->chunk_item_begin = (const int32_t*)p;
    d->chunk_plan_ok = true;
    return CBKV_OK;
}

int rep_slots_of(int n_rep) {
    int rs = 1;
    while (rs < n_rep) rs <<= 1;
    return rs;
}

int32_t get_tile_plan(Arena* a, int tokens_per_item, cudaStream_t st) {
    DeviceState* d = dev_of(a);
    if (d->tile_plan_ok && d->tile_plan_tokens == tokens_per_item) return CBKV_OK;
    build_chunk_tile_plan(*a, tokens_per_item, &d->tile_host);
    d->tile_plan_tokens = tokens_per_item;
    const void* p = nullptr;
    int32_t rc = slot_upload(d, d->tile_host.item_begin.data(), d->tile_host.item_begin.size() * sizeof(int32_t), st, &p);
    if (rc) return rc;
    d->tile_item_begin = (const int32_t*)p;
    d->tile_plan_ok = true;
    return CBKV_OK;
}

struct ProfScope {
    DeviceState* d;
    cudaStream_t st;
    size_t idx = 0;
    bool on;
    ProfScope(DeviceState* d_, cudaStream_t s) : d(d_), st(s), on(d_->profile) {
        if (!on) return;
        if (d->prof_used == d->prof.size()) {
            cudaEvent_t a, b;
            cudaEventCreate(&a); cudaEventCreate(&b);
            d->prof.emplace_back(a, b);
        }
        idx = d->prof_used++;
        cudaEventRecord(d->prof[idx].first, st);
    }
    ~ProfScope() { if (on) cudaEventRecord(d->prof[idx].second, st); }
};

int32_t check_step(Arena* a, int32_t layer) {
    if (!a) { set_error("null arena"); return CBKV_ERR_ARG; }
    if (layer < 0 || layer >= a->cfg.num_layers) { set_error("layer out of range"); return CBKV_ERR_ARG; }
    if (!a->step_open || !a->dev || dev_of(a)->uploaded_step != a->step_id) {
        set_error("no step begun (call cbkv_begin_step first)"); return CBKV_ERR_STATE;
    }
    return CBKV_OK;
}

int32_t run_append(Arena* a, int layer, const void* k, const void* v, cudaStream_t st) {
    DeviceState* d = dev_of(a);
    { int32_t frc = flush_uploads(d, st); if (frc) return frc; }
    AppendArgs args{d->step, geom(a), k, v, d->layers[(size_t)layer].base, d->status};
    if (d->layers[(size_t)layer].quant) {
        args.geo.tiled = 0;
        CU_TRY(launch_append_quant(args, a->cfg.dtype == CBKV_BF16, st));
    } else {
        CU_TRY(launch_append(args, a->cfg.dtype == CBKV_BF16, st));
    }
    g_launches++;
    d->last_kv_writer = layer;
    return CBKV_OK;
}

// k, v non-null on a decode step => the append rides inside the decode kernel.
int32_t run_attention(Arena* a, int layer, const void* q, const void* k_fused, const void* v_fused, void* out,
                      double scale, int64_t window, cudaStream_t st) {
    DeviceState* d = dev_of(a);
    const bool bf16 = a->cfg.dtype == CBKV_BF16;
    const int64_t w = a->layer_window(layer, window);
    if (w != 0 && w < 2) { set_error("sliding window must be >= 2, got " + std::to_string(w)); return CBKV_ERR_ARG; }
    LayerArena& L = d->layers[(size_t)layer];
    const float scale_log2 = (float)(scale * 1.4426950408889634);
    // tensor-core chunk kernels: worth it once the step has enough new tokens to fill 128-row tiles
    // (their softmax takes row maxima before scaling, which needs a positive scale)
    const bool tc_able = d->fast && d->tc_ok && scale > 0 && !a->step_is_decode;
    const bool use_tc2 = tc_able && chunk_tc2_supported(a->cfg.head_dim) &&
                         (d->chunk_mode == 3 || d->chunk_mode == 4 || (d->chunk_mode == 0 && a->step_tokens >= 128));
    const bool use_tc = tc_able && !use_tc2 && (d->chunk_mode == 2 || (d->chunk_mode == 0 && a->step_tokens >= 64));
    // int8 pages: decode steps stream the records through the decode kernel; the chunk kernels read a float
    // copy made per layer and step (mode 4: the two-tile kernel converts the records itself, slower so far);
    // shapes outside the fast path de-quantise on the fly in the generic kernel
    const bool q8_direct = L.quant && use_tc2 && d->chunk_mode == 4;
    LayerArena* KV = &L;  // where the chunk kernels read K/V from
    if (L.quant && d->fast && !a->step_is_decode && !q8_direct && !(debug_flags() & 16)) {
        // de-quantise the pages of the step's sequences into the scratch layer (kv_dequantize,
        // kv.rs:771-780) and run the float chunk kernels over that
        if (!d->qscratch.base) {
            int32_t rc = alloc_float_layer(a, &d->qscratch, st);
            if (rc) return rc;
        }
        GeomDev g = geom(a);
        { int32_t frc = flush_uploads(d, st); if (frc) return frc; }
        CU_TRY(launch_dequant_pages(d->step.tables, (int)a->step_tables.size(), g, L.base, d->qscratch.base, d->status, bf16, st));
        g_launches++;
        KV = &d->qscratch;
    } else if (L.quant && !q8_direct && !(d->fast && a->step_is_decode && !(debug_flags() & 16))) {
        GenericArgs args{d->step, geom(a), q, out, L.base, d->status, (int32_t)w, (float)scale};
        ProfScope ps(d, st);
        { int32_t frc = flush_uploads(d, st); if (frc) return frc; }
        CU_TRY(launch_generic_quant(args, bf16, st));
        g_launches++;
        return CBKV_OK;
    }
    if (d->fast && a->step_is_decode) {
        DecodePlanDev* pd = nullptr;
        int32_t rc = get_decode_plan(a, w, L.quant, st, &pd);
        if (rc) return rc;
        DecodeConfig dc = decode_config(a->cfg.head_dim, a->n_rep(), d->decode_ctas_per_sm, d->decode_stages, d->decode_consumers, L.quant);
        DecodeArgs args{};
        args.geo = geom(a);
        args.segs = pd->segs; args.items = pd->items; args.unit_row = d->unit_rows + pd->unit_row_off;
        args.n_segs = pd->host.n_segs; args.n_items = pd->host.n_items; args.n_ctas = pd->host.n_ctas;
        args.n_units = pd->host.n_units; args.tail_pct = pd->host.levels > 1 ? d->split.tail_pct : 0;
        args.q = q; args.out = out; args.k_new = k_fused; args.v_new = v_fused; args.arena = L.base;
        args.part_o = d->part_o; args.part_ml = d->part_ml; args.seg_counter = d->seg_counter; args.status = d->status;
        args.work_counters = d->work_counters; args.work_slot = (int32_t)(d->launch_seq++ & 3u);
        args.window = (int32_t)w; args.scale_log2 = scale_log2;
        args.n_stages = dc.stages; args.comb_cols = dc.comb_cols; args.comb_bufs = dc.comb_bufs;
        // the producer may run ahead of earlier work in the stream unless that work wrote what it reads
        args.kv_dep = (d->last_kv_writer == layer || pd->fresh) ? 1 : 0;
        pd->fresh = false;
        args.wait_us = d->wait_us; args.fault_tile = d->fault_tile;
        args.in_flag = d->next_in_flag; args.in_seq = d->next_in_seq;
#ifdef CBKV_MEASURE
        args.debug = debug_flags();
        if (args.debug & 256) {  // timestamps of the last eight launches, no memset in between (launch overlap stays intact)
            if (!d->dbg_buf) { CU_TRY(cudaMalloc(&d->dbg_buf, 4096 * 16 * sizeof(unsigned long long))); CU_TRY(cudaMemset(d->dbg_buf, 0, 4096 * 16 * sizeof(unsigned long long))); }
            args.debug |= 4;
            args.dbg_buf = d->dbg_buf + (size_t)((d->launch_seq - 1) & 7u) * 512 * 16;
            d->dbg_ctas = std::min(512, pd->host.n_ctas);
            d->dbg_chain_last = (int)((d->launch_seq - 1) & 7u);
        } else if (args.debug & 4) {
            if (!d->dbg_buf) { CU_TRY(cudaMalloc(&d->dbg_buf, 4096 * 16 * sizeof(unsigned long long))); }
            CU_TRY(cudaMemsetAsync(d->dbg_buf, 0, 4096 * 16 * sizeof(unsigned long long), st));
            args.dbg_buf = d->dbg_buf;
            d->dbg_ctas = pd->host.n_ctas;
        }
#endif
        ProfScope ps(d, st);
        { int32_t frc = flush_uploads(d, st); if (frc) return frc; }
        CU_TRY(launch_decode(L.map_kv, args, pd->host.n_ctas, dc.consumers, dc.smem_bytes, d->pdl, bf16, st, L.quant));
        g_launches++;
        d->last_kv_writer = k_fused ? layer : -1;
        return CBKV_OK;
    }
    if (use_tc || use_tc2) {
        const int rs = rep_slots_of(a->n_rep());
        int32_t rc = get_tile_plan(a, (use_tc2 ? 2 : 1) * (128 / rs), st);
        if (rc) return rc;
        ChunkArgs args{};
        args.step = d->step; args.geo = geom(a); args.item_begin = d->tile_item_begin; args.n_items = d->tile_host.n_items;
        args.q = q; args.out = out; args.status = d->status; args.window = (int32_t)w; args.scale_log2 = scale_log2; args.rep_slots = rs;
        args.q8_arena = q8_direct ? L.base : nullptr;
        if (use_tc2 && d->chunk_split > 1) {
            // The grid runs one CTA per SM at a time.  When the last wave would fill at most half of the SMs, its
            // items are cut along K/V so that the wave is full and ends sooner (the slices are merged by whichever
            // CTA of an item finishes last).  Only worth it when every slice still has a few K/V tiles.
            const int n_items = d->tile_host.n_items, rem = n_items % d->sm_count;
            int parts = rem > 0 ? std::min(d->chunk_split, d->sm_count / rem) : 1;
            int64_t min_keys = INT64_MAX;
            for (const auto& m : a->step_meta) {
                const int64_t keys = w > 0 ? std::min<int64_t>(w, (int64_t)m.pos + m.snew) : (int64_t)m.pos + m.snew;
                min_keys = std::min(min_keys, keys);
            }
            while (parts > 1 && min_keys < (int64_t)parts * 8 * 128) parts--;  // measured: below 8 tiles per slice the merge costs more than the wave saves
            if (parts > 1) {
                const int slices = rem * parts;
                if (slices > d->split_cap) {
                    CU_TRY(cudaStreamSynchronize(st));
                    if (d->split_o) { cudaFree(d->split_o); cudaFree(d->split_ml); cudaFree(d->split_counter); }
                    d->split_cap = std::max(slices, d->sm_count);
                    CU_TRY(cudaMalloc(&d->split_o, (size_t)d->split_cap * 2 * 128 * 128 * sizeof(float)));
                    CU_TRY(cudaMalloc(&d->split_ml, (size_t)d->split_cap * 2 * 128 * sizeof(float2)));
                    CU_TRY(cudaMalloc(&d->split_counter, (size_t)d->split_cap * sizeof(int32_t)));
                    CU_TRY(cudaMemsetAsync(d->split_counter, 0, (size_t)d->split_cap * sizeof(int32_t), st));
                }
                args.split_first = n_items - rem; args.split_parts = parts;
                args.split_o = d->split_o; args.split_ml = d->split_ml; args.split_counter = d->split_counter;
            }
        }
#ifdef CBKV_MEASURE
        if (debug_flags() & 8) {  // per-role cycle counters of the first 4096 CTAs
            if (!d->dbg_buf) { CU_TRY(cudaMalloc(&d->dbg_buf, 4096 * 16 * sizeof(unsigned long long))); }
            CU_TRY(cudaMemsetAsync(d->dbg_buf, 0, 4096 * 16 * sizeof(unsigned long long), st));
            if (d->tile_host.n_items + d->sm_count * 4 <= 4096) { args.dbg_buf = d->dbg_buf; d->dbg_ctas = -d->tile_host.n_items; }
        }
#endif
        ProfScope ps(d, st);
        { int32_t frc = flush_uploads(d, st); if (frc) return frc; }
        if (use_tc2) CU_TRY(q8_direct ? launch_chunk_tc2(L.map_k16, L.map_sc, args, bf16, st) : launch_chunk_tc2(KV->map_kv, KV->map_kv, args, bf16, st));
        else CU_TRY(launch_chunk_tc(KV->map_k16, KV->map_kv, args, bf16, st));
        g_launches++;
        d->last_kv_writer = -1;
        return CBKV_OK;
    }
    if (d->fast) {
        int32_t rc = get_chunk_plan(a, st);
        if (rc) return rc;
        ChunkArgs args{};
        args.step = d->step; args.geo = geom(a); args.item_begin = d->chunk_item_begin; args.n_items = d->chunk_host.n_items;
        args.q = q; args.out = out; args.status = d->status; args.window = (int32_t)w; args.scale_log2 = scale_log2;
        ProfScope ps(d, st);
        { int32_t frc = flush_uploads(d, st); if (frc) return frc; }
        CU_TRY(launch_chunk(KV->map_kv, args, bf16, st));
        g_launches++;
        return CBKV_OK;
    }
    GenericArgs args{d->step, geom(a), q, out, L.base, d->status, (int32_t)w, (float)scale};
    ProfScope ps(d, st);
    { int32_t frc = flush_uploads(d, st); if (frc) return frc; }
    CU_TRY(launch_generic(args, bf16, st));
    g_launches++;
    return CBKV_OK;
}

}  // namespace

extern "C" {

const char* cbkv_last_error(void) { return last_error(); }

int32_t cbkv_arena_create(const cbkv_config* cfg, cbkv_arena** out) {
    return fenced([&]() -> int32_t {
    Arena* a = nullptr;
    int32_t rc = arena_create(cfg, &a);
    if (rc == CBKV_OK) *out = reinterpret_cast<cbkv_arena*>(a);
    return rc;
    });
}

int32_t cbkv_arena_destroy(cbkv_arena* arena) {
    return fenced([&]() -> int32_t {
    Arena* a = reinterpret_cast<Arena*>(arena);
    if (!a) return CBKV_OK;
    if (a->dev) {
        DeviceState* d = dev_of(a);
        cudaSetDevice(d->device);
        cudaDeviceSynchronize();
        for (auto& L : d->layers) if (L.base) cudaFree(L.base);
        for (auto& s : d->slots) { if (s.host) cudaFreeHost(s.host); if (s.dev) cudaFree(s.dev); if (s.ev) cudaEventDestroy(s.ev); }
        if (d->part_o) { cudaFree(d->part_o); cudaFree(d->part_ml); }
        if (d->seg_counter) cudaFree(d->seg_counter);
        if (d->unit_rows) cudaFree(d->unit_rows);
        if (d->work_counters) cudaFree(d->work_counters);
#ifdef CBKV_MEASURE
        if (d->dbg_buf) cudaFree(d->dbg_buf);
#endif
        if (d->status) cudaFree(d->status);
        if (d->io) cudaFree(d->io);
        if (d->qrot) cudaFree(d->qrot);
        if (d->qscratch.base) cudaFree(d->qscratch.base);
        for (auto& sl : d->io_slots) {
            if (sl.dev) cudaFree(sl.dev);
            if (sl.in_done) { cudaEventDestroy(sl.in_done); cudaEventDestroy(sl.k_done); cudaEventDestroy(sl.out_done); }
        }
        if (d->h2d) { cudaStreamDestroy(d->h2d); cudaStreamDestroy(d->d2h); }
        if (d->split_o) { cudaFree(d->split_o); cudaFree(d->split_ml); cudaFree(d->split_counter); }
        if (d->in_flags) cudaFree(d->in_flags);
        if (d->in_seq_host) cudaFreeHost(d->in_seq_host);
        for (auto& p : d->prof) { cudaEventDestroy(p.first); cudaEventDestroy(p.second); }
        delete d;
    }
    while (!a->seqs.empty()) seq_destroy(a->seqs.back());
    delete a;
    return CBKV_OK;
    });
}

int32_t cbkv_set_free_list(cbkv_arena* arena, const int64_t* ids, int64_t n) {
    return fenced([&]() -> int32_t {
    Arena* a = reinterpret_cast<Arena*>(arena);
    if (!a || !ids) { set_error("null argument"); return CBKV_ERR_ARG; }
    if (!a->alloc.set_initial(ids, n)) {
        set_error("set_free_list needs a full permutation of the page ids on an unused arena");
        return CBKV_ERR_ARG;
    }
    return CBKV_OK;
    });
}

int32_t cbkv_seq_create(cbkv_arena* arena, cbkv_seq** out) {
    return fenced([&]() -> int32_t {
    Seq* s = nullptr;
    int32_t rc = seq_create(reinterpret_cast<Arena*>(arena), &s);
    if (rc == CBKV_OK) *out = reinterpret_cast<cbkv_seq*>(s);
    return rc;
    });
}
int32_t cbkv_seq_destroy(cbkv_seq* seq) {
    return fenced([&]() -> int32_t { return seq_destroy(reinterpret_cast<Seq*>(seq)); });
}

int32_t cbkv_seq_fork_prefix(cbkv_seq* parent, int64_t n_tokens, cbkv_seq** out) {
    return fenced([&]() -> int32_t {
    Seq* c = nullptr;
    int32_t rc = seq_fork_prefix(reinterpret_cast<Seq*>(parent), n_tokens, &c);
    if (rc == CBKV_OK) *out = reinterpret_cast<cbkv_seq*>(c);
    return rc;
    });
}

int32_t cbkv_begin_step(cbkv_arena* arena, cbkv_seq* const* seqs, const int64_t* new_tokens, const int64_t* pos,
                        int32_t n_seqs, void* stream) {
    return fenced([&]() -> int32_t {
    NvtxRange nvtx_range("cbkv_begin_step");
    Arena* a = reinterpret_cast<Arena*>(arena);
    if (!a) { set_error("null arena"); return CBKV_ERR_ARG; }
    // The device must be reachable before any state is advanced: there is no CPU path.
    int32_t rc = ensure_device(a);
    if (rc) return rc;
    rc = begin_step(a, reinterpret_cast<Seq* const*>(seqs), new_tokens, pos, n_seqs);
    if (rc) return rc;
    return upload_step(a, static_cast<cudaStream_t>(stream));
    });
}

int32_t cbkv_append(cbkv_arena* arena, int32_t layer, const void* k, const void* v, void* stream) {
    return fenced([&]() -> int32_t {
    NvtxRange nvtx_range("cbkv_append", layer);
    Arena* a = reinterpret_cast<Arena*>(arena);
    int32_t rc = check_step(a, layer);
    if (rc) return rc;
    if (a->step_tokens == 0) return CBKV_OK;  // empty step
    if (!k || !v) { set_error("null k/v"); return CBKV_ERR_ARG; }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    CU_TRY(cudaSetDevice(dev_of(a)->device));
    if ((rc = materialize(a, layer, st))) return rc;
    return run_append(a, layer, k, v, st);
    });
}

int32_t cbkv_paged_attention(cbkv_arena* arena, int32_t layer, const void* q, void* out, double scale, int64_t window,
                             void* stream) {
    return fenced([&]() -> int32_t {
    NvtxRange nvtx_range("cbkv_paged_attention", layer);
    Arena* a = reinterpret_cast<Arena*>(arena);
    int32_t rc = check_step(a, layer);
    if (rc) return rc;
    if (a->step_tokens == 0) return CBKV_OK;  // empty step
    if (!q || !out) { set_error("null q/out"); return CBKV_ERR_ARG; }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    CU_TRY(cudaSetDevice(dev_of(a)->device));
    if ((rc = materialize(a, layer, st))) return rc;
    return run_attention(a, layer, q, nullptr, nullptr, out, scale, window, st);
    });
}

int32_t cbkv_attention(cbkv_arena* arena, int32_t layer, const void* q, const void* k, const void* v, void* out,
                       double scale, int64_t window, void* stream) {
    return fenced([&]() -> int32_t {
    NvtxRange nvtx_range("cbkv_attention", layer);
    Arena* a = reinterpret_cast<Arena*>(arena);
    int32_t rc = check_step(a, layer);
    if (rc) return rc;
    if (a->step_tokens == 0) return CBKV_OK;  // empty step
    if (!q || !k || !v || !out) { set_error("null tensor"); return CBKV_ERR_ARG; }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    DeviceState* d = dev_of(a);
    CU_TRY(cudaSetDevice(d->device));
    if ((rc = materialize(a, layer, st))) return rc;
    if (d->fast && a->step_is_decode && !(d->layers[(size_t)layer].quant && (debug_flags() & 16)))
        return run_attention(a, layer, q, k, v, out, scale, window, st);  // the append rides inside the decode kernel
    if ((rc = run_append(a, layer, k, v, st))) return rc;
    return run_attention(a, layer, q, nullptr, nullptr, out, scale, window, st);
    });
}

// ---- rotary embedding + QK norm fused into the append (rope.cu) ----------------
struct Rope {
    Arena* arena;
    int device;
    int head_dim;
    int64_t max_position;
    void* table;  // [max_position][cos: head_dim/2 | sin: head_dim/2] in the arena's element type
};

static int32_t check_rope_cfg(const cbkv_rope_config* c) {
    if (!c) { set_error("null rope config"); return CBKV_ERR_ARG; }
    if (c->head_dim < 4 || c->head_dim % 4 != 0 || c->head_dim > 512) {
        set_error("rope head_dim must be a multiple of 4 in [4, 512]"); return CBKV_ERR_ARG;
    }
    if (c->max_position < 1 || !(c->theta > 0.0)) { set_error("rope needs max_position >= 1 and theta > 0"); return CBKV_ERR_ARG; }
    if (c->scaling < CBKV_ROPE_NONE || c->scaling > CBKV_ROPE_LONGROPE) { set_error("unknown rope scaling"); return CBKV_ERR_ARG; }
    return CBKV_OK;
}

int32_t cbkv_rope_inv_freq_host(const cbkv_rope_config* cfg, double* inv_out, double* mscale_out) {
    return fenced([&]() -> int32_t {
    int32_t rc = check_rope_cfg(cfg);
    if (rc) return rc;
    if (!inv_out || !mscale_out) { set_error("null output"); return CBKV_ERR_ARG; }
    std::vector<double> inv;
    if ((rc = rope_inv_freq(*cfg, &inv, mscale_out))) return rc;
    std::copy(inv.begin(), inv.end(), inv_out);
    return CBKV_OK;
    });
}

int32_t cbkv_rope_tables_host(const cbkv_rope_config* cfg, float* cos_out, float* sin_out) {
    return fenced([&]() -> int32_t {
    int32_t rc = check_rope_cfg(cfg);
    if (rc) return rc;
    if (!cos_out || !sin_out) { set_error("null output"); return CBKV_ERR_ARG; }
    std::vector<double> inv;
    double mscale = 1.0;
    if ((rc = rope_inv_freq(*cfg, &inv, &mscale))) return rc;
    rope_tables(*cfg, inv, mscale, cos_out, sin_out);
    return CBKV_OK;
    });
}

int32_t cbkv_rope_create(cbkv_arena* arena, const cbkv_rope_config* cfg, cbkv_rope** out) {
    return fenced([&]() -> int32_t {
    Arena* a = reinterpret_cast<Arena*>(arena);
    if (!a || !out) { set_error("null argument"); return CBKV_ERR_ARG; }
    int32_t rc = check_rope_cfg(cfg);
    if (rc) return rc;
    if (cfg->head_dim != a->cfg.head_dim) { set_error("rope head_dim differs from the arena's"); return CBKV_ERR_ARG; }
    if ((rc = ensure_device(a))) return rc;
    const int64_t n = cfg->max_position * cfg->head_dim;
    std::vector<float> cosv((size_t)n), sinv((size_t)n);
    if ((rc = cbkv_rope_tables_host(cfg, cosv.data(), sinv.data()))) return rc;
    // device layout: per position head_dim/2 cosines then head_dim/2 sines, f32 -> element type
    // (rope.rs:167-176)
    const int half = cfg->head_dim / 2;
    std::vector<uint16_t> packed((size_t)cfg->max_position * half * 2);
    const bool bf16 = a->cfg.dtype == CBKV_BF16;
    auto conv = [&](float f) -> uint16_t {
        if (bf16) { __nv_bfloat16 h = __float2bfloat16_rn(f); uint16_t u; memcpy(&u, &h, 2); return u; }
        __half h = __float2half_rn(f); uint16_t u; memcpy(&u, &h, 2); return u;
    };
    for (int64_t p = 0; p < cfg->max_position; p++)
        for (int i = 0; i < half; i++) {
            packed[(size_t)(p * 2 * half + i)] = conv(cosv[(size_t)(p * cfg->head_dim + i)]);
            packed[(size_t)(p * 2 * half + half + i)] = conv(sinv[(size_t)(p * cfg->head_dim + i)]);
        }
    auto* r = new Rope{a, dev_of(a)->device, cfg->head_dim, cfg->max_position, nullptr};
    cudaError_t e = cudaMalloc(&r->table, packed.size() * 2);
    if (e == cudaSuccess) e = cudaMemcpy(r->table, packed.data(), packed.size() * 2, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
        if (r->table) cudaFree(r->table);
        delete r;
        set_error(std::string("rope table upload: ") + cudaGetErrorString(e));
        return CBKV_ERR_CUDA;
    }
    *out = reinterpret_cast<cbkv_rope*>(r);
    return CBKV_OK;
    });
}

int32_t cbkv_rope_destroy(cbkv_rope* rope) {
    return fenced([&]() -> int32_t {
    Rope* r = reinterpret_cast<Rope*>(rope);
    if (!r) return CBKV_OK;
    cudaSetDevice(r->device);
    if (r->table) cudaFree(r->table);
    delete r;
    return CBKV_OK;
    });
}

// k_out non-null: rotated k goes to that dense buffer and nothing is written to pages (int8 layers,
// whose append quantises afterwards).
static int32_t run_rope_append(Arena* a, int layer, const Rope* r, const cbkv_qk_norm* norm, const void* q, const void* k,
                               const void* v, void* q_out, void* k_out, cudaStream_t st) {
    DeviceState* d = dev_of(a);
    if (r->arena != a) { set_error("rope tables belong to another arena"); return CBKV_ERR_ARG; }
    for (const SeqMeta& m : a->step_meta)
        if ((int64_t)m.pos + m.snew > r->max_position) {
            set_error("rope table shorter than the step's positions: " + std::to_string((int64_t)m.pos + m.snew) + " > " +
                      std::to_string(r->max_position));
            return CBKV_ERR_ARG;
        }
    RopeArgs args{};
    args.step = d->step; args.geo = geom(a);
    args.q = q; args.k = k; args.v = v; args.q_out = q_out; args.k_out = k_out;
    args.arena = d->layers[(size_t)layer].base;
    args.table = r->table; args.max_position = r->max_position;
    args.q_weight = norm ? norm->q_weight : nullptr;
    args.k_weight = norm ? norm->k_weight : nullptr;
    args.eps = norm ? (float)norm->eps : 0.f;
    args.gemma = norm ? norm->gemma : 0;
    args.status = d->status;
    { int32_t frc = flush_uploads(d, st); if (frc) return frc; }
    CU_TRY(launch_rope_append(args, a->cfg.dtype == CBKV_BF16, st));
    g_launches++;
    if (!k_out) d->last_kv_writer = layer;
    return CBKV_OK;
}

// Scratch for the rotated q (and, for int8 layers, the rotated k) of the current layer.
static int32_t rope_scratch(Arena* a, cudaStream_t st, size_t bytes) {
    DeviceState* d = dev_of(a);
    if (bytes <= d->qrot_cap) return CBKV_OK;
    CU_TRY(cudaStreamSynchronize(st));  // an earlier layer may still read the old buffer
    if (d->qrot) cudaFree(d->qrot);
    d->qrot = nullptr;
    d->qrot_cap = 0;
    CU_TRY(cudaMalloc(&d->qrot, bytes * 2));
    d->qrot_cap = bytes * 2;
    return CBKV_OK;
}

int32_t cbkv_rope_append(cbkv_arena* arena, int32_t layer, const cbkv_rope* rope, const cbkv_qk_norm* norm,
                         const void* q, const void* k, const void* v, void* q_out, void* stream) {
    return fenced([&]() -> int32_t {
    NvtxRange nvtx_range("cbkv_rope_append", layer);
    Arena* a = reinterpret_cast<Arena*>(arena);
    int32_t rc = check_step(a, layer);
    if (rc) return rc;
    if (a->step_tokens == 0) return CBKV_OK;  // empty step
    if (!rope || !q || !k || !v || !q_out) { set_error("null argument"); return CBKV_ERR_ARG; }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    CU_TRY(cudaSetDevice(dev_of(a)->device));
    if ((rc = materialize(a, layer, st))) return rc;
    DeviceState* d = dev_of(a);
    if (d->layers[(size_t)layer].quant) {  // rotate k to scratch, then the quantising append (kv.rs:746-768)
        const size_t kb = ((size_t)a->step_tokens * a->cfg.n_kv_heads * a->cfg.head_dim * 2 + 255) & ~(size_t)255;
        if ((rc = rope_scratch(a, st, kb))) return rc;
        if ((rc = run_rope_append(a, layer, reinterpret_cast<const Rope*>(rope), norm, q, k, v, q_out, d->qrot, st))) return rc;
        return run_append(a, layer, d->qrot, v, st);
    }
    return run_rope_append(a, layer, reinterpret_cast<const Rope*>(rope), norm, q, k, v, q_out, nullptr, st);
    });
}

int32_t cbkv_attention_rope(cbkv_arena* arena, int32_t layer, const cbkv_rope* rope, const cbkv_qk_norm* norm,
                            const void* q, const void* k, const void* v, void* out, double scale, int64_t window,
                            void* stream) {
    return fenced([&]() -> int32_t {
    NvtxRange nvtx_range("cbkv_attention_rope", layer);
    Arena* a = reinterpret_cast<Arena*>(arena);
    int32_t rc = check_step(a, layer);
    if (rc) return rc;
    if (a->step_tokens == 0) return CBKV_OK;  // empty step
    if (!rope || !q || !k || !v || !out) { set_error("null argument"); return CBKV_ERR_ARG; }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    DeviceState* d = dev_of(a);
    CU_TRY(cudaSetDevice(d->device));
    if ((rc = materialize(a, layer, st))) return rc;
    const size_t qb = ((size_t)a->step_tokens * a->cfg.n_q_heads * a->cfg.head_dim * 2 + 255) & ~(size_t)255;
    const size_t kb = ((size_t)a->step_tokens * a->cfg.n_kv_heads * a->cfg.head_dim * 2 + 255) & ~(size_t)255;
    const bool quant = d->layers[(size_t)layer].quant;
    if ((rc = rope_scratch(a, st, qb + (quant ? kb : 0)))) return rc;
    if (quant) {  // int8 pages: rotate q and k to scratch; the append (fused into the decode kernel when it can be) quantises
        uint8_t* krot = d->qrot + qb;
        if ((rc = run_rope_append(a, layer, reinterpret_cast<const Rope*>(rope), norm, q, k, v, d->qrot, krot, st))) return rc;
        if (d->fast && a->step_is_decode && !(debug_flags() & 16))
            return run_attention(a, layer, d->qrot, krot, v, out, scale, window, st);
        if ((rc = run_append(a, layer, krot, v, st))) return rc;
        return run_attention(a, layer, d->qrot, nullptr, nullptr, out, scale, window, st);
    }
    if ((rc = run_rope_append(a, layer, reinterpret_cast<const Rope*>(rope), norm, q, k, v, d->qrot, nullptr, st))) return rc;
    return run_attention(a, layer, d->qrot, nullptr, nullptr, out, scale, window, st);
    });
}

int32_t cbkv_attention_host(cbkv_arena* arena, int32_t layer, const void* q_host, const void* k_host,
                            const void* v_host, void* out_host, double scale, int64_t window, void* stream) {
    return fenced([&]() -> int32_t {
    Arena* a = reinterpret_cast<Arena*>(arena);
    int32_t rc = check_step(a, layer);
    if (rc) return rc;
    if (a->step_tokens == 0) return CBKV_OK;  // empty step
    if (!q_host || !k_host || !v_host || !out_host) { set_error("null tensor"); return CBKV_ERR_ARG; }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    DeviceState* d = dev_of(a);
    CU_TRY(cudaSetDevice(d->device));
    const size_t qb = (size_t)a->step_tokens * a->cfg.n_q_heads * a->cfg.head_dim * 2;
    const size_t kb = (size_t)a->step_tokens * a->cfg.n_kv_heads * a->cfg.head_dim * 2;
    auto up = [](size_t x) { return (x + 255) & ~(size_t)255; };
    const size_t need = 2 * up(qb) + 2 * up(kb);
    if (need > d->io_cap) {
        CU_TRY(cudaStreamSynchronize(st));
        if (d->io) cudaFree(d->io);
        d->io_cap = need * 2;
        CU_TRY(cudaMalloc(&d->io, d->io_cap));
    }
    uint8_t* qd = d->io;
    uint8_t* od = qd + up(qb);
    uint8_t* kd = od + up(qb);
    uint8_t* vd = kd + up(kb);
    CU_TRY(cudaMemcpyAsync(qd, q_host, qb, cudaMemcpyHostToDevice, st));
    CU_TRY(cudaMemcpyAsync(kd, k_host, kb, cudaMemcpyHostToDevice, st));
    CU_TRY(cudaMemcpyAsync(vd, v_host, kb, cudaMemcpyHostToDevice, st));
    rc = cbkv_attention(arena, layer, qd, kd, vd, od, scale, window, stream);
    if (rc) return rc;
    CU_TRY(cudaMemcpyAsync(out_host, od, qb, cudaMemcpyDeviceToHost, st));
    CU_TRY(cudaStreamSynchronize(st));
    return CBKV_OK;
    });
}

int32_t cbkv_attention_host_async(cbkv_arena* arena, int32_t layer, const void* q_host, const void* k_host,
                                  const void* v_host, void* out_host, double scale, int64_t window, void* stream) {
    return fenced([&]() -> int32_t {
    NvtxRange nvtx_range("cbkv_attention_host_async", layer);
    Arena* a = reinterpret_cast<Arena*>(arena);
    int32_t rc = check_step(a, layer);
    if (rc) return rc;
    if (a->step_tokens == 0) return CBKV_OK;  // empty step
    if (!q_host || !k_host || !v_host || !out_host) { set_error("null tensor"); return CBKV_ERR_ARG; }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    DeviceState* d = dev_of(a);
    CU_TRY(cudaSetDevice(d->device));
    if (!d->h2d) {
        CU_TRY(cudaStreamCreateWithFlags(&d->h2d, cudaStreamNonBlocking));
        CU_TRY(cudaStreamCreateWithFlags(&d->d2h, cudaStreamNonBlocking));
    }
    const size_t qb = (size_t)a->step_tokens * a->cfg.n_q_heads * a->cfg.head_dim * 2;
    const size_t kb = (size_t)a->step_tokens * a->cfg.n_kv_heads * a->cfg.head_dim * 2;
    auto up = [](size_t x) { return (x + 255) & ~(size_t)255; };
    const size_t need = 2 * up(qb) + 2 * up(kb);
    const int si = d->io_cur;
    DeviceState::IoSlot& sl = d->io_slots[si];
    d->io_cur = (d->io_cur + 1) % DeviceState::kIoSlots;
    if (!sl.in_done) {
        CU_TRY(cudaEventCreateWithFlags(&sl.in_done, cudaEventDisableTiming));
        CU_TRY(cudaEventCreateWithFlags(&sl.k_done, cudaEventDisableTiming));
        CU_TRY(cudaEventCreateWithFlags(&sl.out_done, cudaEventDisableTiming));
    }
    if (sl.used) CU_TRY(cudaEventSynchronize(sl.out_done));  // the slot's previous round trip is over
    if (need > sl.cap) {
        if (sl.dev) CU_TRY(cudaFree(sl.dev));
        sl.cap = need * 2;
        CU_TRY(cudaMalloc(&sl.dev, sl.cap));
    }
    uint8_t* qd = sl.dev;
    uint8_t* od = qd + up(qb);
    uint8_t* kd = od + up(qb);
    uint8_t* vd = kd + up(kb);
    CU_TRY(cudaMemcpyAsync(qd, q_host, qb, cudaMemcpyHostToDevice, d->h2d));
    CU_TRY(cudaMemcpyAsync(kd, k_host, kb, cudaMemcpyHostToDevice, d->h2d));
    CU_TRY(cudaMemcpyAsync(vd, v_host, kb, cudaMemcpyHostToDevice, d->h2d));
    if (d->fast && a->step_is_decode && d->host_direct) {
        // the decode kernel waits for this number itself (bounded), after its wait for the previous launch
        if (!d->in_flags) {
            CU_TRY(cudaMalloc(&d->in_flags, DeviceState::kIoSlots * sizeof(uint32_t)));
            CU_TRY(cudaMemset(d->in_flags, 0, DeviceState::kIoSlots * sizeof(uint32_t)));
            CU_TRY(cudaMallocHost(&d->in_seq_host, DeviceState::kIoSlots * sizeof(uint32_t)));
        }
        const uint32_t seq = ++d->in_seq;
        d->in_seq_host[si] = seq;  // stable until the slot comes round again, by when this copy is long done
        CU_TRY(cudaMemcpyAsync(d->in_flags + si, d->in_seq_host + si, sizeof(uint32_t), cudaMemcpyHostToDevice, d->h2d));
        d->next_in_flag = d->in_flags + si;
        d->next_in_seq = seq;
    } else {
        CU_TRY(cudaEventRecord(sl.in_done, d->h2d));
        CU_TRY(cudaStreamWaitEvent(st, sl.in_done, 0));
    }
    rc = cbkv_attention(arena, layer, qd, kd, vd, od, scale, window, stream);
    d->next_in_flag = nullptr;
    if (rc) return rc;
    CU_TRY(cudaEventRecord(sl.k_done, st));
    CU_TRY(cudaStreamWaitEvent(d->d2h, sl.k_done, 0));
    CU_TRY(cudaMemcpyAsync(out_host, od, qb, cudaMemcpyDeviceToHost, d->d2h));
    CU_TRY(cudaEventRecord(sl.out_done, d->d2h));
    sl.used = true;
    return CBKV_OK;
    });
}

int32_t cbkv_host_sync(cbkv_arena* arena) {
    return fenced([&]() -> int32_t {
    Arena* a = reinterpret_cast<Arena*>(arena);
    if (!a) { set_error("null arena"); return CBKV_ERR_ARG; }
    if (!a->dev) return CBKV_OK;
    DeviceState* d = dev_of(a);
    CU_TRY(cudaSetDevice(d->device));
    // every output copy runs on the one output stream, in order: waiting for the stream is waiting for all of them
    if (d->d2h) CU_TRY(cudaStreamSynchronize(d->d2h));
    return CBKV_OK;
    });
}

int32_t cbkv_host_alloc(size_t bytes, void** out) {
    return fenced([&]() -> int32_t {
    if (!out) { set_error("null argument"); return CBKV_ERR_ARG; }
    CU_TRY(cudaMallocHost(out, bytes));
    return CBKV_OK;
    });
}
int32_t cbkv_host_free(void* p) {
    return fenced([&]() -> int32_t {
    if (p) CU_TRY(cudaFreeHost(p));
    return CBKV_OK;
    });
}

int32_t cbkv_popn(cbkv_seq* seq, int64_t n, int64_t* popped) {
    return fenced([&]() -> int32_t { return popn(reinterpret_cast<Seq*>(seq), n, popped); });
}
int32_t cbkv_reset(cbkv_seq* seq) {
    return fenced([&]() -> int32_t { return reset(reinterpret_cast<Seq*>(seq)); });
}
int64_t cbkv_seq_len(const cbkv_seq* seq) {
    return fenced64([&]() -> int64_t {
        if (!seq) { set_error("null sequence"); return (int64_t)CBKV_ERR_ARG; }
        return reinterpret_cast<const Seq*>(seq)->seq_len;
    });
}
int64_t cbkv_pages_used(const cbkv_seq* seq) {
    return fenced64([&]() -> int64_t {
        if (!seq) { set_error("null sequence"); return (int64_t)CBKV_ERR_ARG; }
        return (int64_t)reinterpret_cast<const Seq*>(seq)->table.size();
    });
}
int64_t cbkv_num_free_pages(const cbkv_arena* arena) {
    return fenced64([&]() -> int64_t {
        if (!arena) { set_error("null arena"); return (int64_t)CBKV_ERR_ARG; }
        return reinterpret_cast<const Arena*>(arena)->alloc.num_free();
    });
}

int32_t cbkv_page_stats(const cbkv_seq* seq, cbkv_page_stats_t* out) {
    return fenced([&]() -> int32_t {
    const Seq* s = reinterpret_cast<const Seq*>(seq);
    if (!s || !out) { set_error("null argument"); return CBKV_ERR_ARG; }
    int64_t mat = 0;
    if (s->arena->dev)
        for (auto& L : static_cast<DeviceState*>(s->arena->dev)->layers) if (L.base) mat++;
    page_stats(s, mat, out);
    return CBKV_OK;
    });
}

int64_t cbkv_page_bytes(const cbkv_arena* arena) {
    return fenced64([&]() -> int64_t {
    const Arena* a = reinterpret_cast<const Arena*>(arena);
    if (!a) { set_error("null arena"); return (int64_t)CBKV_ERR_ARG; }
    int64_t total = 0;  // what one page id costs over all layers: float pages, or records with bytes + scales
    for (int l = 0; l < a->cfg.num_layers; l++)
        total += a->layer_quant(l) ? (int64_t)a->cfg.n_kv_heads * (int64_t)qrec_bytes(a->cfg.page_size, a->cfg.head_dim)
                                   : (int64_t)a->cfg.page_size * a->cfg.n_kv_heads * a->cfg.head_dim * 2 * 2;
    return total;
    });
}

int64_t cbkv_export_block_table(const cbkv_seq* seq, int64_t* out, int64_t cap) {
    return fenced64([&]() -> int64_t {
    const Seq* s = reinterpret_cast<const Seq*>(seq);
    if (!s || (!out && cap > 0)) { set_error("null argument"); return (int64_t)CBKV_ERR_ARG; }
    for (int64_t i = 0; i < (int64_t)s->table.size() && i < cap; i++) out[i] = s->table[(size_t)i];
    return (int64_t)s->table.size();
    });
}

int64_t cbkv_export_free_list(const cbkv_arena* arena, int64_t* out, int64_t cap) {
    return fenced64([&]() -> int64_t {
    if (!arena || (!out && cap > 0)) { set_error("null argument"); return (int64_t)CBKV_ERR_ARG; }
    const auto& st = reinterpret_cast<const Arena*>(arena)->alloc.stack();
    for (int64_t i = 0; i < (int64_t)st.size() && i < cap; i++) out[i] = st[(size_t)i];
    return (int64_t)st.size();
    });
}

int32_t cbkv_export_page(cbkv_arena* arena, int32_t layer, int64_t page, void* k_out_host, void* v_out_host, void* stream) {
    return fenced([&]() -> int32_t {
    Arena* a = reinterpret_cast<Arena*>(arena);
    if (!a || !k_out_host || !v_out_host) { set_error("null argument"); return CBKV_ERR_ARG; }
    if (layer < 0 || layer >= a->cfg.num_layers || page < 0 || page >= a->num_pages) { set_error("layer or page out of range"); return CBKV_ERR_ARG; }
    const size_t tile = (size_t)a->cfg.page_size * a->cfg.head_dim * 2;  // one head's K (or V) rows, bytes
    const int H = a->cfg.n_kv_heads;
    if (!a->dev || !dev_of(a)->layers[(size_t)layer].base) {
        memset(k_out_host, 0, tile * H);
        memset(v_out_host, 0, tile * H);
        return CBKV_OK;
    }
    DeviceState* d = dev_of(a);
    if (d->layers[(size_t)layer].quant) { set_error("layer holds int8 pages: use cbkv_export_page_quant"); return CBKV_ERR_STATE; }
    CU_TRY(cudaSetDevice(d->device));
    CU_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    std::vector<uint8_t> buf(tile * 2 * H);
    CU_TRY(cudaMemcpy(buf.data(), (uint8_t*)d->layers[(size_t)layer].base + (size_t)page * tile * 2 * H, buf.size(),
                      cudaMemcpyDeviceToHost));
    const size_t rowb = (size_t)a->cfg.head_dim * 2;
    const int P = a->cfg.page_size;
    for (int h = 0; h < H; h++)  // the arena's row order (page_row) -> K [h][slot][d], V [h][slot][d]
        for (int slot = 0; slot < P; slot++) {
            memcpy((uint8_t*)k_out_host + ((size_t)h * P + slot) * rowb,
                   buf.data() + ((size_t)h * 2 * P + page_row(0, slot, P, d->fast)) * rowb, rowb);
            memcpy((uint8_t*)v_out_host + ((size_t)h * P + slot) * rowb,
                   buf.data() + ((size_t)h * 2 * P + page_row(1, slot, P, d->fast)) * rowb, rowb);
        }
    return CBKV_OK;
    });
}

int32_t cbkv_layer_is_quantized(const cbkv_arena* arena, int32_t layer) {
    return fenced([&]() -> int32_t {
    const Arena* a = reinterpret_cast<const Arena*>(arena);
    if (!a || layer < 0 || layer >= a->cfg.num_layers) { set_error("layer out of range"); return CBKV_ERR_ARG; }
    return a->layer_quant(layer) ? 1 : 0;
    });
}

int32_t cbkv_export_page_quant(cbkv_arena* arena, int32_t layer, int64_t page, int32_t* kp, void* ks, int32_t* vp, void* vs,
                               void* stream) {
    return fenced([&]() -> int32_t {
    Arena* a = reinterpret_cast<Arena*>(arena);
    if (!a || !kp || !ks || !vp || !vs) { set_error("null argument"); return CBKV_ERR_ARG; }
    if (layer < 0 || layer >= a->cfg.num_layers || page < 0 || page >= a->num_pages) { set_error("layer or page out of range"); return CBKV_ERR_ARG; }
    if (!a->layer_quant(layer)) { set_error("layer holds float pages: use cbkv_export_page"); return CBKV_ERR_STATE; }
    const int H = a->cfg.n_kv_heads, P = a->cfg.page_size, D = a->cfg.head_dim, G = D / 32;
    const size_t rows = (size_t)H * P;
    if (!a->dev || !dev_of(a)->layers[(size_t)layer].base) {  // never written: zeros (kv.rs:699-705)
        memset(kp, 0, rows * D); memset(vp, 0, rows * D);
        memset(ks, 0, rows * G * 2); memset(vs, 0, rows * G * 2);
        return CBKV_OK;
    }
    DeviceState* d = dev_of(a);
    CU_TRY(cudaSetDevice(d->device));
    CU_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    const size_t rec = qrec_bytes(P, D);
    std::vector<uint8_t> buf(rec * H);
    CU_TRY(cudaMemcpy(buf.data(), (uint8_t*)d->layers[(size_t)layer].base + (size_t)page * H * rec, buf.size(), cudaMemcpyDeviceToHost));
    for (int h = 0; h < H; h++)
        for (int slot = 0; slot < P; slot++)
            for (int is_v = 0; is_v < 2; is_v++) {
                uint8_t* pk = reinterpret_cast<uint8_t*>(is_v ? vp : kp) + ((size_t)h * P + slot) * D;
                uint8_t* sc = reinterpret_cast<uint8_t*>(is_v ? vs : ks) + ((size_t)h * P + slot) * G * 2;
                const uint8_t* r = buf.data() + (size_t)h * rec;
                // records hold q + 128 in every byte; the reference's words keep lane 3 signed (kv.rs:276-283)
                for (int j = 0; j < D; j++) pk[j] = r[qrec_value_off(is_v, slot, j, P, D)] ^ ((j & 3) == 3 ? 0x80 : 0x00);
                for (int g = 0; g < G; g++) memcpy(sc + 2 * g, r + qrec_scale_off(is_v, slot, g, P, D), 2);
}
    return CBKV_OK;
    });
}

int32_t cbkv_page_refcount(const cbkv_arena* arena, int64_t page) {
    return fenced([&]() -> int32_t {
    const Arena* a = reinterpret_cast<const Arena*>(arena);
    if (!a) { set_error("null arena"); return CBKV_ERR_ARG; }
    if (page < 0 || page >= a->num_pages) return -1;
    return a->refcnt[(size_t)page];
    });
}

int32_t cbkv_device_status(cbkv_arena* arena, void* stream, int32_t* status) {
    return fenced([&]() -> int32_t {
    Arena* a = reinterpret_cast<Arena*>(arena);
    if (!a || !status) { set_error("null argument"); return CBKV_ERR_ARG; }
    *status = 0;
    if (!a->dev) return CBKV_OK;
    DeviceState* d = dev_of(a);
    CU_TRY(cudaSetDevice(d->device));
    CU_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    CU_TRY(cudaMemcpy(status, d->status, sizeof(int32_t), cudaMemcpyDeviceToHost));
#ifdef CBKV_MEASURE
    if ((debug_flags() & 256) && d->dbg_buf && d->dbg_chain_last >= 0) {  // the last eight decode launches as they overlapped
        std::vector<unsigned long long> h((size_t)8 * 512 * 16);
        cudaMemcpy(h.data(), d->dbg_buf, h.size() * 8, cudaMemcpyDeviceToHost);
        unsigned long long t0 = ~0ull;
        const int n = d->dbg_ctas;
        for (int l = 0; l < 8; l++) for (int c = 0; c < n; c++) { unsigned long long v = h[((size_t)l * 512 + c) * 16]; if (v) t0 = std::min(t0, v); }
        double prev_exit = 0;
        for (int k = 1; k <= 8; k++) {
            const int l = (d->dbg_chain_last + k) & 7;
            const int slots[5] = {0, 4, 7, 5, 6};
            const char* names[5] = {"entry", "first_tile", "prod_done", "last_piece", "exit"};
            char line[512]; int off = snprintf(line, sizeof line, "[cbkv chain] launch %d:", k);
            double this_exit = 0;
            for (int s2 = 0; s2 < 5; s2++) {
                double mn = 1e18, mx = 0, av = 0; int cnt = 0;
                for (int c = 0; c < n; c++) { unsigned long long v = h[((size_t)l * 512 + c) * 16 + slots[s2]]; if (!v) continue; double x = (double)(v - t0) * 1e-3; mn = std::min(mn, x); mx = std::max(mx, x); av += x; cnt++; }
                if (cnt) off += snprintf(line + off, sizeof line - off, " %s %.1f/%.1f/%.1f", names[s2], mn, av / cnt, mx);
                if (s2 == 4) this_exit = mx;
            }
            fprintf(stderr, "%s | period %.1f us\n", line, this_exit - prev_exit);
            {   // the same times by quarter of the CTA index (CTAs are dispatched in index order as SMs come free)
                char q[256]; int qo = snprintf(q, sizeof q, "[cbkv chain]   by index quarter, entry / exit:");
                for (int part = 0; part < 4; part++) {
                    double en = 0, ex = 0; int cnt = 0;
                    for (int c = n * part / 4; c < n * (part + 1) / 4; c++) {
                        const unsigned long long e0 = h[((size_t)l * 512 + c) * 16 + 0], e1 = h[((size_t)l * 512 + c) * 16 + 6];
                        if (!e0 || !e1) continue;
                        en += (double)(e0 - t0) * 1e-3; ex += (double)(e1 - t0) * 1e-3; cnt++;
                    }
                    if (cnt) qo += snprintf(q + qo, sizeof q - qo, "  %.1f / %.1f", en / cnt, ex / cnt);
                }
                fprintf(stderr, "%s\n", q);
            }
            prev_exit = this_exit;
        }
        {   // is a CTA's streaming time a property of the SM it ran on?  per SM: mean and spread over the eight launches
            std::map<int, std::vector<double>> by_sm;
            for (int l = 0; l < 8; l++)
                for (int c = 0; c < n; c++) {
                    const unsigned long long* r = &h[((size_t)l * 512 + c) * 16];
                    if (r[4] && r[7]) by_sm[(int)r[11]].push_back((double)(r[7] - r[4]) * 1e-3);
                }
            std::vector<std::pair<double, int>> order;
            double within = 0; int nw = 0;
            for (auto& kv : by_sm) {
                double m = 0; for (double x : kv.second) m += x; m /= kv.second.size();
                for (double x : kv.second) { within += (x - m) * (x - m); nw++; }
                order.push_back({m, kv.first});
            }
            std::sort(order.begin(), order.end());
            double gm = 0; for (auto& o : order) gm += o.first; gm /= std::max<size_t>(1, order.size());
            double between = 0; for (auto& o : order) between += (o.first - gm) * (o.first - gm);
            fprintf(stderr, "[cbkv chain] streaming time per SM (first tile -> last copy issued): mean %.2f us, std between SMs %.2f, std within an SM %.2f\n",
                    gm, std::sqrt(between / std::max<size_t>(1, order.size())), std::sqrt(within / std::max(1, nw)));
            char line[1024]; int off = snprintf(line, sizeof line, "[cbkv chain] fastest SMs:");
            for (size_t i = 0; i < std::min<size_t>(10, order.size()); i++) off += snprintf(line + off, sizeof line - off, " %d:%.1f", order[i].second, order[i].first);
            off += snprintf(line + off, sizeof line - off, " | slowest:");
            for (size_t i = order.size() > 10 ? order.size() - 10 : 0; i < order.size(); i++) off += snprintf(line + off, sizeof line - off, " %d:%.1f", order[i].second, order[i].first);
            fprintf(stderr, "%s\n", line);
        }
        d->dbg_chain_last = -1;
    }
#endif
    if (*status) {
        CU_TRY(cudaMemset(d->status, 0, sizeof(int32_t)));
        if (d->seg_counter) CU_TRY(cudaMemset(d->seg_counter, 0, d->counter_cap * sizeof(int32_t)));
        if (d->work_counters) CU_TRY(cudaMemset(d->work_counters, 0, 4 * sizeof(int32_t)));
        set_error("kernel status word = " + std::to_string(*status));
        return CBKV_ERR_DEVICE;
    }
    return CBKV_OK;
    });
}

int64_t cbkv_launch_count(void) {
    return fenced64([&]() -> int64_t { return g_launches.load(); });
}

int32_t cbkv_profile_enable(cbkv_arena* arena, int32_t on) {
    return fenced([&]() -> int32_t {
    Arena* a = reinterpret_cast<Arena*>(arena);
    if (!a) { set_error("null arena"); return CBKV_ERR_ARG; }
    int32_t rc = ensure_device(a);
    if (rc) return rc;
    dev_of(a)->profile = on != 0;
    dev_of(a)->prof_used = 0;
    return CBKV_OK;
    });
}

int32_t cbkv_profile_read(cbkv_arena* arena, double* total_ms, int64_t* launches) {
    return fenced([&]() -> int32_t {
    Arena* a = reinterpret_cast<Arena*>(arena);
    if (!a || !a->dev || !total_ms || !launches) { set_error("null argument"); return CBKV_ERR_ARG; }
    DeviceState* d = dev_of(a);
    CU_TRY(cudaSetDevice(d->device));
    CU_TRY(cudaDeviceSynchronize());
    double sum = 0;
    for (size_t i = 0; i < d->prof_used; i++) {
        float ms = 0;
        CU_TRY(cudaEventElapsedTime(&ms, d->prof[i].first, d->prof[i].second));
        sum += ms;
    }
#ifdef CBKV_MEASURE
    if ((debug_flags() & 8) && d->dbg_buf && d->dbg_ctas < 0) {
        const int n = -d->dbg_ctas;
        std::vector<unsigned long long> h((size_t)n * 16);
        cudaMemcpy(h.data(), d->dbg_buf, h.size() * 8, cudaMemcpyDeviceToHost);
        const char* names[15] = {"producer wait_empty", "producer issue", "mma wait_kv", "mma wait_p", "mma issue (QK)", "softmax wait_s",
                                 "softmax ld+max", "softmax exp+store", "softmax wait_o", "softmax rescale+arrive", "softmax total",
                                 "mma issue (PV, two-tile kernel)", "int8 loader: convert", "int8 loader: warp meets", "int8 loader: next copy"};
        double tiles = 0;
        for (int c = 0; c < n; c++) tiles += (double)h[(size_t)c * 16 + 15];
        for (int s2 = 0; s2 < 15; s2++) {
            double sum = 0;
            for (int c = 0; c < n; c++) sum += (double)h[(size_t)c * 16 + s2];
            fprintf(stderr, "[cbkv tc] %-26s %9.0f cycles per KV tile (mean over %d CTAs, %.1f tiles each)\n", names[s2], sum / tiles, n, tiles / n);
        }
        if (h[12] == 0x7c2) {  // float layers of the two-tile kernel: what a CTA spends outside its tiles
            double pro = 0, epi = 0, loop = 0;
            for (int c = 0; c < n; c++) { pro += (double)h[(size_t)c * 16 + 13]; epi += (double)h[(size_t)c * 16 + 14]; loop += (double)h[(size_t)c * 16 + 10]; }
            fprintf(stderr, "[cbkv tc] per CTA: %.0f cycles from entry to the softmax loop, %.0f in the loop, %.0f from the loop's end to the output written\n",
                    pro / n, loop / n, epi / n);
        }
    }
    if ((debug_flags() & 4) && d->dbg_buf && d->dbg_ctas > 0 && d->dbg_ctas <= 4096) {
        std::vector<unsigned long long> h((size_t)d->dbg_ctas * 16);
        cudaMemcpy(h.data(), d->dbg_buf, h.size() * 8, cudaMemcpyDeviceToHost);
        unsigned long long t0 = ~0ull;
        for (int c = 0; c < d->dbg_ctas; c++) if (h[(size_t)c * 16]) t0 = std::min(t0, h[(size_t)c * 16]);
        const char* names[8] = {"entry", "-", "first_round_issued", "q_loaded", "first_tile_ready", "last_piece_arrived", "merger_exit", "producer_done"};
        for (int s2 = 0; s2 < 8; s2++) {
            double mn = 1e18, mx = 0, av = 0; int cnt = 0;
            for (int c = 0; c < d->dbg_ctas; c++) { unsigned long long v = h[(size_t)c * 16 + s2]; if (!v) continue; double x = (double)(v - t0) * 1e-3; mn = std::min(mn, x); mx = std::max(mx, x); av += x; cnt++; }
            if (cnt) fprintf(stderr, "[cbkv timeline] %-22s min %7.2f avg %7.2f max %7.2f us (%d CTAs)\n", names[s2], mn, av / cnt, mx, cnt);
        }
        std::vector<int> order(d->dbg_ctas);
        for (int c = 0; c < d->dbg_ctas; c++) order[c] = c;
        std::sort(order.begin(), order.end(), [&](int x, int y) { return h[(size_t)x * 16 + 6] > h[(size_t)y * 16 + 6]; });
        auto us = [&](int c, int s2) { return h[(size_t)c * 16 + s2] ? (double)(h[(size_t)c * 16 + s2] - t0) * 1e-3 : -1.0; };
        for (int i = 0; i < d->dbg_ctas; i += (i < 8 ? 1 : d->dbg_ctas / 8)) {
            int c = order[i];
            fprintf(stderr, "[cbkv cta] rank %3d cta %3d sm %3llu tiles %3llu items %llu pieces %llu merges %llu parts %llu | first_tile %.1f prod_done %.1f last_piece %.1f exit %.1f\n",
                    i, c, h[(size_t)c * 16 + 11], h[(size_t)c * 16 + 12], h[(size_t)c * 16 + 13], h[(size_t)c * 16 + 8], h[(size_t)c * 16 + 9], h[(size_t)c * 16 + 10],
                    us(c, 4), us(c, 7), us(c, 5), us(c, 6));
        }
    }
#endif
    *total_ms = sum;
    *launches = (int64_t)d->prof_used;
    d->prof_used = 0;
    return CBKV_OK;
    });
}

int32_t cbkv_set_decode_tuning(cbkv_arena* arena, int32_t ctas_per_sm, int32_t stages, int32_t consumers,
                               int32_t max_ctas, int32_t overlap_launches) {
    return fenced([&]() -> int32_t {
    Arena* a = reinterpret_cast<Arena*>(arena);
    if (!a || ctas_per_sm < 0 || ctas_per_sm > 8 || stages < 0 || stages > 64 || max_ctas < 0 ||
        !(consumers == 0 || consumers == 4 || consumers == 6 || consumers == 8 || consumers == 12)) {
        set_error("bad argument"); return CBKV_ERR_ARG;
    }
    int32_t rc = ensure_device(a);
    if (rc) return rc;
    DeviceState* d = dev_of(a);
    if (d->fast) {
        DecodeConfig dc = decode_config(a->cfg.head_dim, a->n_rep(), ctas_per_sm, stages, consumers);
        if (dc.smem_bytes > 227 * 1024) { set_error("that many stages do not fit in shared memory"); return CBKV_ERR_ARG; }
    }
    d->decode_ctas_per_sm = ctas_per_sm;
    d->decode_stages = stages;
    d->decode_consumers = consumers;
    d->decode_max_ctas = max_ctas;
    d->pdl = overlap_launches != 0;
    d->decode_plans.clear();  // the split depends on the CTA count
    return CBKV_OK;
    });
}

int32_t cbkv_set_host_route(cbkv_arena* arena, int32_t direct) {
    return fenced([&]() -> int32_t {
    Arena* a = reinterpret_cast<Arena*>(arena);
    if (!a) { set_error("null arena"); return CBKV_ERR_ARG; }
    int32_t rc = ensure_device(a);
    if (rc) return rc;
    dev_of(a)->host_direct = direct != 0;
    return CBKV_OK;
    });
}

int32_t cbkv_set_chunk_split(cbkv_arena* arena, int32_t max_parts) {
    return fenced([&]() -> int32_t {
    Arena* a = reinterpret_cast<Arena*>(arena);
    if (!a || max_parts < 1 || max_parts > 8) { set_error("bad argument"); return CBKV_ERR_ARG; }
    int32_t rc = ensure_device(a);
    if (rc) return rc;
    dev_of(a)->chunk_split = max_parts;
    return CBKV_OK;
    });
}

int32_t cbkv_set_chunk_kernel(cbkv_arena* arena, int32_t mode) {
    return fenced([&]() -> int32_t {
    Arena* a = reinterpret_cast<Arena*>(arena);
    if (!a || mode < 0 || mode > 4) { set_error("bad argument"); return CBKV_ERR_ARG; }
    int32_t rc = ensure_device(a);
    if (rc) return rc;
    if (mode >= 3 && !(dev_of(a)->tc_ok && chunk_tc2_supported(a->cfg.head_dim))) {
        set_error("the two-tile tensor-core chunk kernel covers head_dim 128 with 16-token pages only"); return CBKV_ERR_ARG;
    }
    if (mode == 2 && !dev_of(a)->tc_ok) { set_error("the tensor-core chunk kernel covers head_dim 64, 128 and 256 with 16-token pages only"); return CBKV_ERR_ARG; }
    dev_of(a)->chunk_mode = mode;
    return CBKV_OK;
    });
}

// Host-only view of the decode work split for the step in flight (used by the CPU tests of
// the partition): out = [n_ctas, n_items, n_segs, n_units, n_parts, levels,
// segs (n_segs + 1 records of 8 ints), items (n_items records of 4 ints)].
int64_t cbkv_debug_decode_plan(cbkv_arena* arena, int64_t window, int32_t n_ctas, int32_t tail_pct, int32_t min_item,
                               int32_t* out, int64_t cap) {
    return fenced64([&]() -> int64_t {
    Arena* a = reinterpret_cast<Arena*>(arena);
    if (!a || a->step_meta.empty() || !out) return -1;
    DecodePlan pl;
    DecodeSplit sp;
    if (tail_pct >= 0) sp.tail_pct = tail_pct;
    if (min_item >= 0) sp.min_item = min_item;
    build_decode_plan(*a, window, n_ctas, sp, &pl);
    std::vector<int32_t> flat = {pl.n_ctas, pl.n_items, pl.n_segs, pl.n_units, pl.n_parts, pl.levels};
    const int32_t* sp32 = reinterpret_cast<const int32_t*>(pl.segs.data());
    flat.insert(flat.end(), sp32, sp32 + pl.segs.size() * 8);
    const int32_t* ip32 = reinterpret_cast<const int32_t*>(pl.items.data());
    flat.insert(flat.end(), ip32, ip32 + pl.items.size() * 4);
    for (int64_t i = 0; i < (int64_t)flat.size() && i < cap; i++) out[i] = flat[(size_t)i];
    return (int64_t)flat.size();
    });
}

// How a CTA's share of a decode launch is cut into a head item and a tail of dynamically claimed
// items (manager.hpp, DecodeSplit); negative = keep.  min_item = 0 switches the tail off.
int32_t cbkv_set_decode_split(cbkv_arena* arena, int32_t tail_pct, int32_t min_item, int32_t max_levels) {
    return fenced([&]() -> int32_t {
    Arena* a = reinterpret_cast<Arena*>(arena);
    if (!a || tail_pct > 90 || max_levels > 8) { set_error("bad argument"); return CBKV_ERR_ARG; }
    int32_t rc = ensure_device(a);
    if (rc) return rc;
    DeviceState* d = dev_of(a);
    if (tail_pct >= 0) d->split.tail_pct = tail_pct;
    if (min_item >= 0) d->split.min_item = min_item;
    if (max_levels >= 2) d->split.max_levels = max_levels;
    d->decode_plans.clear();
    return CBKV_OK;
    });
}

// Test hook for the kernels' failure path.  wait_us > 0 replaces the limit of the decode kernel's
// bounded waits (default 100000); fault_tile >= 0 makes the producer of CTA 0 skip the copy of that
// tile, so the consumer that owns it finds its wait running out, the status word gets
// ST_WAIT_TIMEOUT and the launch returns without a result; -1 switches the hook off.  Nothing is
// read or written outside the kernel's own buffers either way.
int32_t cbkv_debug_set_wait_limit(cbkv_arena* arena, int64_t wait_us, int32_t fault_tile) {
    return fenced([&]() -> int32_t {
    Arena* a = reinterpret_cast<Arena*>(arena);
    if (!a || wait_us < 0 || wait_us > 10000000) { set_error("bad argument"); return CBKV_ERR_ARG; }
    int32_t rc = ensure_device(a);
    if (rc) return rc;
    if (wait_us > 0) dev_of(a)->wait_us = (uint32_t)wait_us;
    dev_of(a)->fault_tile = fault_tile;
    return CBKV_OK;
    });
}

// Test hook for the boundary itself: the body throws, the caller must see a return code.
int32_t cbkv_debug_raise(int32_t kind) {
    return fenced([&]() -> int32_t {
        if (kind == 1) throw std::bad_alloc();
        if (kind == 2) throw std::runtime_error("raised on request");
        if (kind == 3) throw 42;
        return CBKV_OK;
    });
}

// Host-only bookkeeping of a step without touching a device (CPU tests of the manager).
int32_t cbkv_debug_begin_step_host(cbkv_arena* arena, cbkv_seq* const* seqs, const int64_t* new_tokens,
                                   const int64_t* pos, int32_t n_seqs) {
    return fenced([&]() -> int32_t { return begin_step(reinterpret_cast<Arena*>(arena), reinterpret_cast<Seq* const*>(seqs), new_tokens, pos, n_seqs); });
}

}  // extern "C"
