// Chunk (prefill) attention on the 5th-generation tensor cores: tcgen05.mma with
// accumulators in tensor memory, operands staged in shared memory by TMA.
// Reference math: attend() with seq > 1, kv.rs:243-268 — scores = q k^T * scale, causal
// mask aligned to the chunk's position (kv.rs:247-251), optional window (kv.rs:252-257),
// softmax over keys, P V — here as a flash-style loop over 128-token KV tiles.
//
// One CTA = one (sequence, kv head, tile of query tokens).  The 128 rows of the MMA are
// "columns" of the problem: row m = rep * TPT + i is q head `rep` of the kv group at
// the tile's i-th token (TPT = 128 / RS tokens, RS = n_rep rounded up to a power of
// two), so the K/V tiles are shared by the whole q-head group.
//
//   warp 0        TMA producer: one 32-row box per (page, 64-column block) brings K and V of a
//                 page in the arena's 8-row interleave; 8 pages per tile, two stages
//   warp 1        one thread issues tcgen05.mma: S = Q K^T (two S buffers), O += P V
//   warps 2..5    softmax: one TMEM lane (row) per thread, P written to shared memory
//                 in the K-major swizzled layout, O rescaled in TMEM when a row max moves
//
// KV tiles hold KT tokens: 128 for head_dim 64 and 128; 64 for head_dim 256, where a 128-token tile of K
// and V (128 KB) would not leave room for two stages next to the Q tile (S = Q K^T is then 128 x 64 and
// O += P V one 128 x 256 MMA per 16 keys).
//
// Tensor memory: S0 [0,KT), S1 [128,128+KT), O [256, 256 + D) -> 512 columns allocated.
// Shared memory: Q and P tiles of 128 rows stored as 64-column blocks of 128 rows x 128 bytes
// (128-byte swizzle); two K/V stages, each D/64 blocks of 8 pages x 32 rows x 128 bytes in
// the arena's row order [K 0-7][V 0-7][K 8-15][V 8-15], so K and V are both 8-row groups
// 2048 bytes apart (V starts 1024 bytes in).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>

#include "kernels.hpp"
#include "q8_unpack.cuh"

namespace cbkv {

namespace {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}
__device__ __forceinline__ uint64_t global_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Bounded: gives up after a wall-clock limit (the caller records it and winds down).
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, uint64_t limit_ns = 200000000ull) {
    for (int i = 0; i < 64; i++)
        if (mbar_try_wait(bar, parity)) return true;
    // the timer is slow to read, and a read in flight would hold up the return: look at it once per 64 polls
    const uint64_t t0 = global_ns();
    for (;;) {
        for (int i = 0; i < 64; i++)
            if (mbar_try_wait(bar, parity)) return true;
        if (global_ns() - t0 > limit_ns) return false;
    }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Shared-memory matrix descriptor (tcgen05): start address, leading / stride byte
// offsets (all >> 4), descriptor version 1, 128-byte swizzle.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFF) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;  // version
    d |= (uint64_t)2 << 61;  // SWIZZLE_128B
    return d;
}
// Instruction descriptor, kind::f16: f32 accumulate, A/B f16 or bf16, M x N, operand majors.
__device__ __forceinline__ uint32_t instr_desc(bool bf16, int M, int N, bool b_mn_major) {
    uint32_t d = 0;
    d |= 1u << 4;                       // D format: f32
    d |= (bf16 ? 1u : 0u) << 7;         // A format
    d |= (bf16 ? 1u : 0u) << 10;        // B format
    d |= 0u << 15;                      // A: K-major
    d |= (b_mn_major ? 1u : 0u) << 16;  // B: K-major or MN-major
    d |= (uint32_t)(N >> 3) << 17;
    d |= (uint32_t)(M >> 4) << 24;
    return d;
}
__device__ __forceinline__ void umma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
          "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
          "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
          "r"(r[30]), "r"(r[31])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// 128 consecutive columns of this thread's lane: four 32-column loads in flight, one wait
__device__ __forceinline__ void tmem_ld128(uint32_t taddr, uint32_t (&r)[128]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%128];\n\t"
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%32,%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47,%48,%49,%50,%51,%52,%53,%54,%55,%56,%57,%58,%59,%60,%61,%62,%63}, [%129];\n\t"
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%64,%65,%66,%67,%68,%69,%70,%71,%72,%73,%74,%75,%76,%77,%78,%79,%80,%81,%82,%83,%84,%85,%86,%87,%88,%89,%90,%91,%92,%93,%94,%95}, [%130];\n\t"
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%96,%97,%98,%99,%100,%101,%102,%103,%104,%105,%106,%107,%108,%109,%110,%111,%112,%113,%114,%115,%116,%117,%118,%119,%120,%121,%122,%123,%124,%125,%126,%127}, [%131];\n\t"
        "tcgen05.wait::ld.sync.aligned;"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63]), "=r"(r[64]), "=r"(r[65]), "=r"(r[66]), "=r"(r[67]), "=r"(r[68]), "=r"(r[69]), "=r"(r[70]), "=r"(r[71]), "=r"(r[72]), "=r"(r[73]), "=r"(r[74]), "=r"(r[75]), "=r"(r[76]), "=r"(r[77]), "=r"(r[78]), "=r"(r[79]), "=r"(r[80]), "=r"(r[81]), "=r"(r[82]), "=r"(r[83]), "=r"(r[84]), "=r"(r[85]), "=r"(r[86]), "=r"(r[87]), "=r"(r[88]), "=r"(r[89]), "=r"(r[90]), "=r"(r[91]), "=r"(r[92]), "=r"(r[93]), "=r"(r[94]), "=r"(r[95]), "=r"(r[96]), "=r"(r[97]), "=r"(r[98]), "=r"(r[99]), "=r"(r[100]), "=r"(r[101]), "=r"(r[102]), "=r"(r[103]), "=r"(r[104]), "=r"(r[105]), "=r"(r[106]), "=r"(r[107]), "=r"(r[108]), "=r"(r[109]), "=r"(r[110]), "=r"(r[111]), "=r"(r[112]), "=r"(r[113]), "=r"(r[114]), "=r"(r[115]), "=r"(r[116]), "=r"(r[117]), "=r"(r[118]), "=r"(r[119]), "=r"(r[120]), "=r"(r[121]), "=r"(r[122]), "=r"(r[123]), "=r"(r[124]), "=r"(r[125]), "=r"(r[126]), "=r"(r[127])
        : "r"(taddr), "r"(taddr + 32), "r"(taddr + 64), "r"(taddr + 96) : "memory");
}
__device__ __forceinline__ void tmem_st128(uint32_t taddr, const uint32_t (&r)[128]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32,%33,%34,%35};\n\t"
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%1], {%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47,%48,%49,%50,%51,%52,%53,%54,%55,%56,%57,%58,%59,%60,%61,%62,%63,%64,%65,%66,%67};\n\t"
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%2], {%68,%69,%70,%71,%72,%73,%74,%75,%76,%77,%78,%79,%80,%81,%82,%83,%84,%85,%86,%87,%88,%89,%90,%91,%92,%93,%94,%95,%96,%97,%98,%99};\n\t"
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%3], {%100,%101,%102,%103,%104,%105,%106,%107,%108,%109,%110,%111,%112,%113,%114,%115,%116,%117,%118,%119,%120,%121,%122,%123,%124,%125,%126,%127,%128,%129,%130,%131};\n\t"
        "tcgen05.wait::st.sync.aligned;"
        :: "r"(taddr), "r"(taddr + 32), "r"(taddr + 64), "r"(taddr + 96), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]), "r"(r[32]), "r"(r[33]), "r"(r[34]), "r"(r[35]), "r"(r[36]), "r"(r[37]), "r"(r[38]), "r"(r[39]), "r"(r[40]), "r"(r[41]), "r"(r[42]), "r"(r[43]), "r"(r[44]), "r"(r[45]), "r"(r[46]), "r"(r[47]), "r"(r[48]), "r"(r[49]), "r"(r[50]), "r"(r[51]), "r"(r[52]), "r"(r[53]), "r"(r[54]), "r"(r[55]), "r"(r[56]), "r"(r[57]), "r"(r[58]), "r"(r[59]), "r"(r[60]), "r"(r[61]), "r"(r[62]), "r"(r[63]), "r"(r[64]), "r"(r[65]), "r"(r[66]), "r"(r[67]), "r"(r[68]), "r"(r[69]), "r"(r[70]), "r"(r[71]), "r"(r[72]), "r"(r[73]), "r"(r[74]), "r"(r[75]), "r"(r[76]), "r"(r[77]), "r"(r[78]), "r"(r[79]), "r"(r[80]), "r"(r[81]), "r"(r[82]), "r"(r[83]), "r"(r[84]), "r"(r[85]), "r"(r[86]), "r"(r[87]), "r"(r[88]), "r"(r[89]), "r"(r[90]), "r"(r[91]), "r"(r[92]), "r"(r[93]), "r"(r[94]), "r"(r[95]), "r"(r[96]), "r"(r[97]), "r"(r[98]), "r"(r[99]), "r"(r[100]), "r"(r[101]), "r"(r[102]), "r"(r[103]), "r"(r[104]), "r"(r[105]), "r"(r[106]), "r"(r[107]), "r"(r[108]), "r"(r[109]), "r"(r[110]), "r"(r[111]), "r"(r[112]), "r"(r[113]), "r"(r[114]), "r"(r[115]), "r"(r[116]), "r"(r[117]), "r"(r[118]), "r"(r[119]), "r"(r[120]), "r"(r[121]), "r"(r[122]), "r"(r[123]), "r"(r[124]), "r"(r[125]), "r"(r[126]), "r"(r[127]) : "memory");
}
__device__ __forceinline__ float ex2_approx(float x) {  // one MUFU op; -inf -> 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    if constexpr (BF16) {
        __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&v);
    } else {
        __half2 v = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&v);
    }
}

// Cycle counters per role, 16 slots per CTA: measurement build only (-DCBKV_MEASURE).
#ifdef CBKV_MEASURE
#define TC_NOW() clock64()
#define TC_ACC(var) do { if (a.dbg_buf) { const long long t1__ = clock64(); var += t1__ - tprev; tprev = t1__; } } while (0)
#define TC_DUMP(...) do { if (a.dbg_buf) { __VA_ARGS__ } } while (0)
#else
#define TC_NOW() 0ll
#define TC_ACC(var) do { (void)var; (void)tprev; } while (0)
#define TC_DUMP(...) do { } while (0)
#endif

constexpr int kThreads = 192;
constexpr int kTmemCols = 512;
constexpr int kPageCap = 2560;   // block-table entries staged in shared memory (40960 tokens); longer ranges read the rest from global memory

template <int D>
struct TcKeys { static constexpr int value = D == 256 ? 64 : 128; };  // tokens per KV tile

template <int D>
constexpr int tc_smem_bytes() {
    // Q tile of 128 rows x D, two stages of K and V tiles of KT tokens x D, P tile of 128 rows x KT keys, barriers
    // and the staged block table; at least 120 KB so that two CTAs never share an SM (each allocates all 512
    // tensor-memory columns)
    constexpr int need = 128 * D * 2 + 2 * 2 * TcKeys<D>::value * D * 2 + 128 * TcKeys<D>::value * 2 + 256 + kPageCap * 4;
    return need < 120 * 1024 ? 120 * 1024 : need;
}

// KT consecutive columns of this thread's lane
template <int KT>
__device__ __forceinline__ void tmem_ld_row(uint32_t taddr, uint32_t (&r)[KT]) {
    if constexpr (KT == 128) {
        tmem_ld128(taddr, r);
    } else {
        static_assert(KT == 64, "KV tiles of 64 or 128 tokens");
        uint32_t lo[32], hi[32];
        tmem_ld32(taddr, lo);
        tmem_ld32(taddr + 32, hi);
#pragma unroll
        for (int e = 0; e < 32; e++) { r[e] = lo[e]; r[32 + e] = hi[e]; }
    }
}

}  // namespace

template <int D, bool BF16>
__global__ void __launch_bounds__(kThreads) chunk_tc_kernel(const __grid_constant__ CUtensorMap tmap, const __grid_constant__ CUtensorMap tmap32, const ChunkArgs a) {
    constexpr uint32_t TILE = 128u * D * 2u;   // one operand tile (Q, K or V)
    constexpr uint32_t BLK = 128u * 128u;      // one 64-element column block of a tile: 128 rows x 128 bytes
    constexpr int XB = D / 64;                 // column blocks per row
    extern __shared__ __align__(1024) uint8_t smem[];
    constexpr int KT = TcKeys<D>::value;           // tokens per KV tile
    constexpr int PPT = KT / 16;               // pages per KV tile
    constexpr uint32_t BLKKV = PPT * 4096u;    // one 64-column block of a K/V stage: PPT pages x 32 rows x 128 bytes
    constexpr uint32_t STAGE = 2u * KT * D * 2u;  // K and V of KT tokens
    uint8_t* sQ = smem;
    uint8_t* sKV = sQ + TILE;           // 2 stages
    uint8_t* sP = sKV + 2 * STAGE;      // 128 rows x KT keys
    uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 128 * KT * 2);
    // barriers: kv_full[2], kv_empty[2], s_full[2], p_full, o_done
    const uint32_t b_kv_full = smem_u32(bars + 0), b_kv_empty = smem_u32(bars + 2), b_s_full = smem_u32(bars + 4);
    const uint32_t b_p_full = smem_u32(bars + 6), b_o_done = smem_u32(bars + 7);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
    volatile int* failed = reinterpret_cast<volatile int*>(bars + 9);
    int* s_pages = reinterpret_cast<int*>(bars + 16);   // [kPageCap] physical pages of the KV range

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if ((smem_u32(smem) & 1023u) != 0) {
        if (tid == 0) atomicOr(a.status, ST_SMEM_ALIGN);
        return;
    }
    // ---- which (sequence, kv head, query tile)
    const int item = blockIdx.x;
    int lo = 0, hi = a.step.n_seqs - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (a.item_begin[mid] <= item) lo = mid; else hi = mid - 1;
    }
    const SeqMeta sm = a.step.seq_meta[lo];
    const int Hkv = a.geo.n_kv, n_rep = a.geo.n_rep, RS = a.rep_slots, TPT = 128 / RS;
    const int n_qt = (sm.snew + TPT - 1) / TPT;
    const int local = item - a.item_begin[lo];
    const int h = local / n_qt, qt = local - h * n_qt;
    const int r0 = qt * TPT;                               // first new token of the tile
    const int r_last = min(r0 + TPT, sm.snew) - 1;
    const int q_min = sm.pos + r0, q_max = sm.pos + r_last;
    const int lo_key = a.window > 0 ? max(0, q_min - a.window + 1) : 0;
    const int p_lo = lo_key >> 4, p_hi = q_max >> 4;
    const int n_tiles = (p_hi - p_lo + 1 + PPT - 1) / PPT;
    const int k0 = p_lo * 16;                               // absolute position of key 0 of tile 0

    if (tid == 0) {
        for (int i = 0; i < 2; i++) { mbar_init(b_kv_full + i * 8, 1); mbar_init(b_kv_empty + i * 8, 1); mbar_init(b_s_full + i * 8, 1); }
        mbar_init(b_p_full, 128);
        mbar_init(b_o_done, 1);
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap) : "memory");
    }
    if (warp == 0) {  // tensor memory for this CTA
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    for (int i = tid; i <= p_hi - p_lo && i < kPageCap; i += kThreads) s_pages[i] = a.step.tables[sm.tbl_off + p_lo + i];
    // ---- Q tile: rows m = rep * TPT + i, K-major swizzled blocks; rows past the data are zero
    {
        const uint16_t* qbase = reinterpret_cast<const uint16_t*>(a.q) + (size_t)sm.tok_off * a.geo.n_q * D;
        for (int c = tid; c < 128 * (D / 8); c += kThreads) {
            const int m = c / (D / 8), j = c - m * (D / 8);   // row, 16-byte piece
            const int rep = m / TPT, r = r0 + (m - rep * TPT);
            uint4 val = make_uint4(0, 0, 0, 0);
            if (rep < n_rep && r < sm.snew)
                val = *reinterpret_cast<const uint4*>(qbase + ((size_t)(h * n_rep + rep) * sm.snew + r) * D + j * 8);
            const uint32_t off = (j >> 3) * BLK + m * 128u + (((j & 7) ^ (m & 7)) << 4);
            *reinterpret_cast<uint4*>(sQ + off) = val;
        }
    }
    fence_proxy_async();   // Q was written through the generic proxy, the MMA reads it through the async proxy
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tS0 = tmem, tO = tmem + 256;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        // The block-table entries of the whole KV range were staged in shared memory by all
        // threads (below the Q load); every lane issues one box of a tile: lane = page * (2 XB) +
        // column block * 2 + (K or V).
        bool ok = true;
        long long tprev = TC_NOW(), c_wait = 0, c_issue = 0;
#pragma unroll 1
        for (int j = 0; j < n_tiles && ok; j++) {
            const int st = j & 1;
            if (lane == 0) {
                if (j >= 2 && !mbar_wait_bounded(b_kv_empty + st * 8, ((j >> 1) - 1) & 1)) ok = false;
                TC_ACC(c_wait);
                if (*failed) ok = false;
                if (ok) mbar_expect_tx(b_kv_full + st * 8, STAGE);
                else { *failed = 1; atomicOr(a.status, ST_WAIT_TIMEOUT); }
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            for (int bx = lane; bx < PPT * XB; bx += 32) {
                const int pg = bx / XB, x = bx - pg * XB;
                // pages past the last visible one repeat it: finite data that the causal mask hides
                const int idx = min(j * PPT + pg, p_hi - p_lo);
                int phys = idx < kPageCap ? s_pages[idx] : a.step.tables[sm.tbl_off + p_lo + idx];
                if (phys < 0 || phys >= a.geo.num_pages) { atomicOr(a.status, ST_BAD_PAGE); phys = 0; }
                tma_load_2d(smem_u32(sKV + st * STAGE + x * BLKKV + pg * 4096), &tmap32, x * 64, (phys * Hkv + h) * 32, b_kv_full + st * 8);
            }
            if (lane == 0) TC_ACC(c_issue);
        }
        TC_DUMP(if (lane == 0) { a.dbg_buf[(size_t)blockIdx.x * 16 + 0] = c_wait; a.dbg_buf[(size_t)blockIdx.x * 16 + 1] = c_issue; a.dbg_buf[(size_t)blockIdx.x * 16 + 15] = n_tiles; });
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t id_qk = instr_desc(BF16, 128, KT, false);
            const uint32_t id_pv = instr_desc(BF16, 128, D, true);
            // descriptors differ only in the start address field (bits 0-13, address >> 4)
            // K: 8-row groups 2048 bytes apart; V: the same groups 1024 bytes further, 64-wide d blocks BLKKV apart
            const uint64_t dq = smem_desc(smem_u32(sQ), 16, 1024), dk = smem_desc(smem_u32(sKV), 16, 2048);
            const uint64_t dp = smem_desc(smem_u32(sP), 16, 1024), dv = smem_desc(smem_u32(sKV) + 1024, BLKKV, 2048);
            auto issue_qk = [&](int j) {
                const uint64_t kst = (uint64_t)(((j & 1) * STAGE) >> 4);
#pragma unroll
                for (int ks = 0; ks < D / 16; ks++) {
                    // 16 elements = 32 bytes inside the swizzled row, four steps per 64-column block
                    const uint64_t qoff = (uint64_t)(((ks >> 2) * BLK + (ks & 3) * 32) >> 4);
                    const uint64_t koff = (uint64_t)(((ks >> 2) * BLKKV + (ks & 3) * 32) >> 4);
                    umma(tS0 + (j & 1) * 128, dq + qoff, dk + kst + koff, id_qk, ks > 0);
                }
                umma_commit(b_s_full + (j & 1) * 8);
            };
            long long tprev = TC_NOW(), c_wkv = 0, c_wp = 0, c_iss = 0;
            bool ok = mbar_wait_bounded(b_kv_full, 0);
            if (ok) { tc_fence_after(); issue_qk(0); }
            for (int j = 0; ok && j < n_tiles; j++) {
                if (j + 1 < n_tiles) {
                    TC_ACC(c_iss);
                    ok = mbar_wait_bounded(b_kv_full + ((j + 1) & 1) * 8, ((j + 1) >> 1) & 1);
                    TC_ACC(c_wkv);
                    if (!ok) break;
                    tc_fence_after();
                    issue_qk(j + 1);
                }
                TC_ACC(c_iss);
                ok = mbar_wait_bounded(b_p_full, j & 1) && !*failed;
                TC_ACC(c_wp);
                if (!ok) break;
                tc_fence_after();
                const int st = j & 1;
                const uint64_t vst = (uint64_t)((st * STAGE) >> 4);
#pragma unroll
                for (int ks = 0; ks < PPT; ks++) {  // 16 keys per step = one page
                    // P: K-major, keys 16 ks.. inside key block ks / 4; V: MN-major, one page (4096 bytes) per step
                    umma(tO, dp + (uint64_t)(((ks >> 2) * BLK + (ks & 3) * 32) >> 4), dv + vst + (uint64_t)((ks * 4096) >> 4), id_pv,
                         (j > 0 || ks > 0));
                }
                umma_commit(b_kv_empty + st * 8);
                umma_commit(b_o_done);
            }
            if (!ok) { *failed = 1; atomicOr(a.status, ST_WAIT_TIMEOUT); }
            TC_DUMP(a.dbg_buf[(size_t)blockIdx.x * 16 + 2] = c_wkv; a.dbg_buf[(size_t)blockIdx.x * 16 + 3] = c_wp; a.dbg_buf[(size_t)blockIdx.x * 16 + 4] = c_iss;);
        }
    } else {
        // ------------------------------------------------------------ softmax + epilogue, one row per thread
        const int lane_base = (warp & 3) * 32;             // the TMEM lanes this warp may touch
        const int m = lane_base + lane;                    // row of the tile
        const int rep = m / TPT, r = r0 + (m - rep * TPT);
        const bool row_ok = rep < n_rep && r < sm.snew;
        const int q_pos = sm.pos + min(r, sm.snew - 1);    // rows past the data mimic the last token
        const uint32_t lane_addr = (uint32_t)lane_base << 16;
        // Exponents are taken against a reference maximum that is only moved when a row's maximum
        // exceeds it by more than 8 (a factor 256): probabilities then stay below 256, exact enough in
        // f16/bf16 with f32 sums, and O needs rescaling only on those rare moves.
        float m_ref = -INFINITY, l_run = 0.f;
        bool ok = true;
        long long tprev = TC_NOW(), c_ws = 0, c_ld = 0, c_exp = 0, c_wo = 0, c_st = 0;
        const long long tstart = tprev;
#pragma unroll 1
        for (int j = 0; j < n_tiles; j++) {
            ok = mbar_wait_bounded(b_s_full + (j & 1) * 8, (j >> 1) & 1) && !*failed;
            ok = __all_sync(0xffffffffu, ok);  // the tensor-memory accesses below need the whole warp
            TC_ACC(c_ws);
            if (!ok) break;
            tc_fence_after();
            const uint32_t tS = tS0 + (j & 1) * 128 + lane_addr;
            const int kbase = k0 + j * KT;
            const bool need_mask = (kbase + KT - 1 > q_min) || (a.window > 0 && kbase + a.window <= q_max);
            uint32_t sv[KT];
            tmem_ld_row<KT>(tS, sv);
            TC_ACC(c_ld);
            float mx = -INFINITY;
            if (need_mask) {
#pragma unroll
                for (int e = 0; e < KT; e++) {
                    const int kp = kbase + e;
                    if (!(kp <= q_pos && (a.window <= 0 || kp + a.window > q_pos))) sv[e] = 0xff800000u;  // -inf
                }
            }
            {
                float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
                for (int e = 0; e < KT; e += 4) {
                    m0 = fmaxf(m0, __uint_as_float(sv[e])); m1 = fmaxf(m1, __uint_as_float(sv[e + 1]));
                    m2 = fmaxf(m2, __uint_as_float(sv[e + 2])); m3 = fmaxf(m3, __uint_as_float(sv[e + 3]));
                }
                mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
            }
            mx *= a.scale_log2;  // scale > 0: the maximum commutes with the scaling
            float alpha = 1.f;
            if (mx > m_ref + 8.f || m_ref == -INFINITY) {
                const float m_new = mx;
                alpha = (m_ref == -INFINITY) ? 0.f : exp2f(m_ref - m_new);
                m_ref = m_new;
            }
            const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
            float sum = 0.f, sum2 = 0.f;
            uint32_t pk[KT / 2];
#pragma unroll
            for (int e = 0; e < KT; e += 2) {
                const float p0 = ex2_approx(fmaf(__uint_as_float(sv[e]), a.scale_log2, -m_use));
                const float p1 = ex2_approx(fmaf(__uint_as_float(sv[e + 1]), a.scale_log2, -m_use));
                if (e & 2) sum2 += p0 + p1; else sum += p0 + p1;  // two chains
                pk[e >> 1] = pack2<BF16>(p0, p1);
            }
            l_run = l_run * alpha + (sum + sum2);
            TC_ACC(c_exp);
            // the previous P V must be finished before P is overwritten and O rescaled
            if (j > 0) {
                ok = mbar_wait_bounded(b_o_done, (j - 1) & 1) && !*failed;
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
            }
            TC_ACC(c_wo);
#pragma unroll
            for (int u = 0; u < KT / 8; u++) {  // 16-byte pieces of 8 keys, K-major swizzled
                const uint32_t off = (u >> 3) * BLK + m * 128u + (((u & 7) ^ (m & 7)) << 4);
                *reinterpret_cast<uint4*>(sP + off) = make_uint4(pk[u * 4], pk[u * 4 + 1], pk[u * 4 + 2], pk[u * 4 + 3]);
            }
            if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
                if constexpr (D == 128) {
                    uint32_t ov[128];
                    tmem_ld128(tO + lane_addr, ov);
#pragma unroll
                    for (int e = 0; e < 128; e++) ov[e] = __float_as_uint(__uint_as_float(ov[e]) * alpha);
                    tmem_st128(tO + lane_addr, ov);
                } else {
#pragma unroll 1
                    for (int c = 0; c < D / 32; c++) {
                        uint32_t v[32];
                        tmem_ld32(tO + lane_addr + c * 32, v);
#pragma unroll
                        for (int e = 0; e < 32; e++) v[e] = __float_as_uint(__uint_as_float(v[e]) * alpha);
                        tmem_st32(tO + lane_addr + c * 32, v);
                    }
                }
            }
            fence_proxy_async();   // P for the async proxy
            tc_fence_before();     // the tensor-memory traffic above is ordered before the hand-over
            mbar_arrive(b_p_full);
            TC_ACC(c_st);
        }
        TC_DUMP(if (tid == 64) {
            unsigned long long* b = a.dbg_buf + (size_t)blockIdx.x * 16;
            b[5] = c_ws; b[6] = c_ld; b[7] = c_exp; b[8] = c_wo; b[9] = c_st; b[10] = TC_NOW() - tstart;
        });
        (void)tstart; (void)c_wo;
        // ---- epilogue: O / l -> out
        if (ok) ok = mbar_wait_bounded(b_o_done, (n_tiles - 1) & 1) && !*failed;
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
            tc_fence_after();
            const float inv = 1.f / l_run;
            uint16_t* orow = reinterpret_cast<uint16_t*>(a.out) +
                             ((size_t)sm.tok_off * a.geo.n_q + (size_t)(h * n_rep + (row_ok ? rep : 0)) * sm.snew + (row_ok ? r : 0)) * D;
#pragma unroll 1
            for (int c = 0; c < D / 32; c++) {
                uint32_t v[32];
                tmem_ld32(tO + lane_addr + c * 32, v);
                if (row_ok) {
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        uint4 w;
                        w.x = pack2<BF16>(__uint_as_float(v[u * 8 + 0]) * inv, __uint_as_float(v[u * 8 + 1]) * inv);
                        w.y = pack2<BF16>(__uint_as_float(v[u * 8 + 2]) * inv, __uint_as_float(v[u * 8 + 3]) * inv);
                        w.z = pack2<BF16>(__uint_as_float(v[u * 8 + 4]) * inv, __uint_as_float(v[u * 8 + 5]) * inv);
                        w.w = pack2<BF16>(__uint_as_float(v[u * 8 + 6]) * inv, __uint_as_float(v[u * 8 + 7]) * inv);
                        *reinterpret_cast<uint4*>(orow + c * 32 + u * 8) = w;
                    }
                }
            }
        } else if (lane == 0) {
            *failed = 1;
            atomicOr(a.status, ST_WAIT_TIMEOUT);
        }
    }
    // ---- wind down: everybody meets, then the allocating warp frees the tensor memory
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
}

template <int D, bool BF16>
static cudaError_t launch_tc(const CUtensorMap& map, const CUtensorMap& map32, const ChunkArgs& a, cudaStream_t st) {
    if (a.n_items <= 0) return cudaSuccess;
    chunk_tc_kernel<D, BF16><<<a.n_items, kThreads, tc_smem_bytes<D>(), st>>>(map, map32, a);
    return cudaGetLastError();
}


// ------------------------------------------------------------------ two query tiles per CTA
// The second-generation kernel: each CTA works on two 128-row query tiles (A and B) that
// share every K/V tile, which halves the shared-memory fill per FLOP, and keeps P in tensor
// memory (it overwrites the first 64 columns of its S tile as packed 16-bit pairs and is the
// A operand of the P V product), so no shared memory is spent on P.
//
//   warp 0        TMA producer (as above)
//   warp 1        MMA issuer:  QK_A, QK_B, then per K/V tile  PV_A, QK_A', PV_B, QK_B'
//   warps 2..9    softmax of tile A        warps 10..17  softmax of tile B
//
// A tile's softmax is the longest link of the chain QK -> softmax -> PV, and that chain, not the tensor pipe,
// set the pace with one thread per row.  Two threads share a row now: the warps of a tile come in pairs that
// may touch the same quarter of the tensor-memory lanes; one takes keys 0-63 of the tile, the other keys
// 64-127 (and, when the row maximum moves, the matching half of the O columns).  They exchange their half-row
// maxima through shared memory once per tile and their half-row sums once at the end.
//
// Tensor memory: S_A [0,128), S_B [128,256), O_A [256,384), O_B [384,512).
constexpr int kThreads2 = 576;

template <int D>
constexpr int tc2_smem_bytes() {
    return 2 * 128 * D * 2 /* Q_A, Q_B */ + 2 * 2 * 128 * D * 2 /* two K/V stages */ + 256 + kPageCap * 4 +
           2 * 2 * 128 * 2 * 4 /* half-row maxima of both tiles, double-buffered */ + 64 /* the pairs' failure flags */;
}

__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

// Q8: the layer holds int8 records (kernels.hpp, qrec_*) and the kernel converts them itself
// (cbkv_set_chunk_kernel mode 4; by default int8 layers go through a float copy, which is faster so far).
// Two warps after the softmax warps take the TMA producer's place, one for K and one for V.  Each keeps a
// ring of raw half-records (a record's K bytes and K scales, or its V bytes and V scales: two boxes of
// the layer's byte tensor maps) in flight, turns a landed half-record into q * scale in registers
// (q8_unpack.cuh: kv_dequantize, kv.rs:319-358), stores that where the tensor pipe reads it, and refills
// the slot itself.  Shared memory is cut differently from the float kernel: K is double-buffered as there
// (the scores of the next tile are issued a tile ahead), V has one buffer (P.V of a tile is the last thing
// that reads it), and the 32 KB this frees plus the tail of the allocation hold 8 K and 14 V half-records.
// Measured on 8 prompts x 8192 tokens: 2.4 times the float-copy route's time.  The V buffer can only be
// refilled between the last P.V of a tile and the first of the next, and one warp needs about 1400 cycles
// per half-record there (wait, convert, refill), eight times per tile; 640 threads at 96 registers leave no
// room for more converting warps, and 227 KB no room for a second V buffer beside the raw rings.
constexpr int kLoaders2 = 2;
constexpr int kThreads2Q8 = kThreads2 + kLoaders2 * 32;
constexpr int kRawK = 8, kRawV = 14;       // half-records per ring
constexpr int kRawVInStage = 7;            // V slots that fit behind the K ring in the freed stage quarter
template <int D>
constexpr int tc2_half_rec() { return 16 * D + 16 * (D / 32) * 2; }  // values + scales of K or of V
template <int D>
constexpr int tc2_smem_bytes_q8() { return tc2_smem_bytes<D>() + 64 + (kRawV - kRawVInStage) * tc2_half_rec<D>() + (kRawK + kRawV + 2) * 8; }

template <int D, bool BF16, bool Q8>
__global__ void __launch_bounds__(Q8 ? kThreads2Q8 : kThreads2) chunk_tc2_kernel(const __grid_constant__ CUtensorMap tmap32, const __grid_constant__ CUtensorMap tmap_sc, const ChunkArgs a) {
    static_assert(D == 128, "two-tile kernel: head_dim 128");
    constexpr uint32_t TILE = 128u * D * 2u;   // one Q tile
    constexpr uint32_t BLK = 128u * 128u;      // 64-column block of a Q tile
    constexpr int XB = D / 64;
    constexpr uint32_t BLKKV = 8u * 4096u;     // 64-column block of a K/V stage
    constexpr uint32_t STAGE = 2u * TILE;
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sQ = smem;                 // Q_A then Q_B
    uint8_t* sKV = sQ + 2 * TILE;       // 2 stages
    uint64_t* bars = reinterpret_cast<uint64_t*>(sKV + 2 * STAGE);
    // barriers: kv_full[2], kv_empty[2], s_full[A,B], p_full[A,B], o_done[A,B]
    const uint32_t b_kv_full = smem_u32(bars + 0), b_kv_empty = smem_u32(bars + 2), b_s_full = smem_u32(bars + 4);
    const uint32_t b_p_full = smem_u32(bars + 6), b_o_done = smem_u32(bars + 8);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);
    volatile int* failed = reinterpret_cast<volatile int*>(bars + 11);
    int* s_pages = reinterpret_cast<int*>(bars + 16);
    float* s_xch = reinterpret_cast<float*>(s_pages + kPageCap);  // [2 buffers][2 tiles][128 rows][2 halves]
    // Q8 layout of the stage area: K buffers [0, 64 KB), V buffer [64, 96 KB), raw K ring and the first raw V
    // slots [96, 128 KB); the other raw V slots and the Q8 barriers follow the exchange area.  A K or V buffer
    // is [64-column block][page][8-token group][8 rows of 128 bytes], 128-byte swizzle.
    constexpr uint32_t REC = 2u * 16u * D + 2u * 16u * (D / 32) * 2u;  // an int8 record
    constexpr uint32_t HALF = 16u * D + 16u * (D / 32) * 2u;              // a record's K or V values with their scales
    static_assert(HALF == (uint32_t)(REC / 2), "half a record");
    constexpr uint32_t QBUF = 128u * D * 2u, QBLK = QBUF / 2;          // one K or V buffer, one 64-column block of it
    static_assert(!Q8 || kRawK * HALF + kRawVInStage * HALF <= 2 * STAGE - 3 * QBUF, "raw rings in the freed quarter");
    uint8_t* sRawK = sKV + 3 * QBUF;
    uint8_t* sRawV0 = sRawK + kRawK * HALF;
    uint8_t* sRawV1 = reinterpret_cast<uint8_t*>(s_xch + 2 * 2 * 128 * 2) + 128;  // 128-byte aligned, as every slot is
    const uint32_t b_q8 = smem_u32(sRawV1 + (kRawV - kRawVInStage) * HALF);
    const uint32_t b_v_full = b_q8, b_v_empty = b_q8 + 8, b_rawk = b_q8 + 16, b_rawv = b_rawk + kRawK * 8;
    (void)sRawK; (void)sRawV0; (void)sRawV1; (void)b_v_full; (void)b_v_empty; (void)b_rawk; (void)b_rawv; (void)REC;

    const long long t_entry = TC_NOW();
    (void)t_entry;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if ((smem_u32(smem) & 1023u) != 0) {
        if (tid == 0) atomicOr(a.status, ST_SMEM_ALIGN);
        return;
    }
    // CTAs past split_first share items: `parts` of them per item, each with a slice of the item's K/V tiles
    const int parts = (a.split_parts > 1 && (int)blockIdx.x >= a.split_first) ? a.split_parts : 1;
    const int item = parts > 1 ? a.split_first + ((int)blockIdx.x - a.split_first) / parts : (int)blockIdx.x;
    const int part = parts > 1 ? ((int)blockIdx.x - a.split_first) % parts : 0;
    int lo = 0, hi = a.step.n_seqs - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (a.item_begin[mid] <= item) lo = mid; else hi = mid - 1;
    }
    const SeqMeta sm = a.step.seq_meta[lo];
    const int Hkv = a.geo.n_kv, n_rep = a.geo.n_rep, RS = a.rep_slots, TPT = 128 / RS;
    const int n_qt = (sm.snew + 2 * TPT - 1) / (2 * TPT);        // pairs of tiles
    const int local = item - a.item_begin[lo];
    const int h = local / n_qt, qt = local - h * n_qt;
    const int r0 = qt * 2 * TPT;                                  // first new token of tile A
    const int q_first = sm.pos + r0, q_last = sm.pos + min(r0 + 2 * TPT, sm.snew) - 1;
    const int lo_key = a.window > 0 ? max(0, q_first - a.window + 1) : 0;
    int p_lo = lo_key >> 4, p_hi = q_last >> 4;
    int n_tiles = (p_hi - p_lo + 1 + 7) >> 3;
    if (parts > 1) {  // this CTA's slice of the tiles (possibly empty: it then hands over rows with sum 0)
        const int per = (n_tiles + parts - 1) / parts;
        const int t0 = min(n_tiles, part * per), t1 = min(n_tiles, t0 + per);
        if (t1 < n_tiles) p_hi = p_lo + 8 * t1 - 1;  // inner slices end on a tile boundary: every page is real
        p_lo += 8 * t0;
        n_tiles = t1 - t0;
    }
    const int k0 = p_lo * 16;

    if (tid == 0) {
        for (int i = 0; i < 2; i++) {
            mbar_init(b_kv_full + i * 8, 1); mbar_init(b_kv_empty + i * 8, 1); mbar_init(b_s_full + i * 8, 1);
            mbar_init(b_p_full + i * 8, 256); mbar_init(b_o_done + i * 8, 1);
        }
        if constexpr (Q8) {  // kv_full / kv_empty above are K's here
            mbar_init(b_v_full, 1); mbar_init(b_v_empty, 1);
            for (int i = 0; i < kRawK + kRawV; i++) mbar_init(b_rawk + i * 8, 1);
        }
        *failed = 0;
        for (int i = 0; i < 8; i++) reinterpret_cast<int*>(s_xch + 2 * 2 * 128 * 2)[i] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap32) : "memory");
        if constexpr (Q8) asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_sc) : "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    for (int i = tid; i <= p_hi - p_lo && i < kPageCap; i += (int)blockDim.x) s_pages[i] = a.step.tables[sm.tbl_off + p_lo + i];
    // ---- Q tiles: row m of tile X is q head (m / TPT) at token r0 + X TPT + m % TPT
    {
        const uint16_t* qbase = reinterpret_cast<const uint16_t*>(a.q) + (size_t)sm.tok_off * a.geo.n_q * D;
        for (int c = tid; c < 256 * (D / 8); c += (int)blockDim.x) {
            const int mm = c / (D / 8), j = c - mm * (D / 8);
            const int X = mm >> 7, m = mm & 127;
            const int rep = m / TPT, r = r0 + X * TPT + (m - rep * TPT);
            uint4 val = make_uint4(0, 0, 0, 0);
            if (rep < n_rep && r < sm.snew)
                val = *reinterpret_cast<const uint4*>(qbase + ((size_t)(h * n_rep + rep) * sm.snew + r) * D + j * 8);
            const uint32_t off = X * TILE + (j >> 3) * BLK + m * 128u + (((j & 7) ^ (m & 7)) << 4);
            *reinterpret_cast<uint4*>(sQ + off) = val;
        }
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (Q8 && warp >= 18) {
        // ------------------------------------------------------------ int8 layer: warp 18 feeds K, warp 19 feeds V
        const bool is_v = warp == 19;
        const int n_slots = is_v ? kRawV : kRawK;
        const uint32_t b_raw = is_v ? b_rawv : b_rawk;
        auto slot_ptr = [&](int sl) -> uint8_t* {
            if (!is_v) return sRawK + sl * HALF;
            return sl < kRawVInStage ? sRawV0 + sl * HALF : sRawV1 + (sl - kRawVInStage) * HALF;
        };
        const int n_recs = 8 * n_tiles;
        // lane 0: the half-record of page n of the CTA's range into its slot (values, then scales behind them).
        // Two boxes of the layer's byte tensor maps (128-byte rows, REC / 128 rows per record: K values, V values,
        // one row of K scales, one of V scales); plain bulk copies of the same bytes cost the issuing thread about
        // a thousand cycles per record, tensor-map copies a few dozen.
        auto issue = [&](int n, int sl) {
            const int idx = min(n, p_hi - p_lo);  // pages past the end repeat the last one (masked)
            int phys = idx < kPageCap ? s_pages[idx] : a.step.tables[sm.tbl_off + p_lo + idx];
            if (phys < 0 || phys >= a.geo.num_pages) { atomicOr(a.status, ST_BAD_PAGE); phys = 0; }
            const int row0 = (phys * Hkv + h) * (int)(REC / 128u);
            const uint32_t dst = smem_u32(slot_ptr(sl)), bar = b_raw + sl * 8;
            mbar_expect_tx(bar, HALF);
            tma_load_2d(dst, &tmap32, 0, row0 + (is_v ? 16 : 0), bar);
            tma_load_2d(dst + 16u * D, &tmap_sc, 0, row0 + 32 + (is_v ? 1 : 0), bar);
        };
        // Lane l takes the 16-byte pieces l, l + 32, l + 64, l + 96 of a half-record's 2048 value bytes.
        // K: 16 consecutive d of token l / 8 + 4 i, one scale group.  V: 8 consecutive d of token pair
        // l / 16 + 2 i.  Both permutations of qrec_value_off repeat every eight tokens, so piece i + 2 lands
        // one 8-token group (1024 bytes) after piece i, and pieces i = 0, 1 differ by four rows.
        uint32_t src_sc, d0[2], d1[2];  // scale offset of piece 0; where the piece's two 16-byte results go (i even, i odd)
        if (!is_v) {
            const int s0 = lane >> 3, grp = ((lane & 7) >> 1) ^ (s0 & 3), j0 = grp * 32 + (lane & 1) * 16, cc = (j0 & 63) >> 3;
            src_sc = 16u * D + (uint32_t)(s0 * (D / 32) + grp) * 2u;  // + 4 i tokens = + 4 i (D / 32) * 2 bytes
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const int row = s0 + 4 * e;
                const uint32_t base = (uint32_t)(j0 >> 6) * QBLK + (uint32_t)row * 128u;
                d0[e] = base + (uint32_t)((cc ^ row) << 4); d1[e] = base + (uint32_t)(((cc + 1) ^ row) << 4);
            }
        } else {
            const int p0 = lane >> 4, grp = ((lane & 15) >> 2) ^ (p0 & 1);
            src_sc = 16u * D + (uint32_t)(grp * 8 + p0) * 4u;          // + 2 i pairs = + 8 i bytes
#pragma unroll
            for (int e = 0; e < 2; e++) {  // pair p0 + 2 i: (pair >> 1) & 1 = i & 1
                const int chunk = (2 * (lane & 3)) ^ (4 * e), j0 = grp * 32 + chunk * 4, cc = (j0 & 63) >> 3;
                const int t0 = 2 * p0 + 4 * e, t1 = t0 + 1;            // rows inside the 8-token group
                const uint32_t base = (uint32_t)(j0 >> 6) * QBLK;
                d0[e] = base + (uint32_t)t0 * 128u + (uint32_t)((cc ^ t0) << 4); d1[e] = base + (uint32_t)t1 * 128u + (uint32_t)((cc ^ t1) << 4);
            }
        }
        int issued = 0;
        if (lane == 0)
            for (; issued < n_slots && issued < n_recs; issued++) issue(issued, issued);
        issued = __shfl_sync(0xffffffffu, issued, 0);
        bool ok = true;
        int n = 0, sl = 0, ph = 0;  // record, its slot, the slot's phase
        long long tprev = TC_NOW(), c_wait = 0, c_issue = 0, c_conv = 0, c_meet = 0;
#pragma unroll 1
        for (; n < n_recs; n++) {
            const int j = n >> 3, pg = n & 7;
            if (lane == 0) {
                if (pg == 0) {  // the buffer this tile goes to must have been read to the end
                    if (!is_v && j >= 2 && !mbar_wait_bounded(b_kv_empty + (j & 1) * 8, ((j >> 1) - 1) & 1)) ok = false;
                    if (is_v && j >= 1 && !mbar_wait_bounded(b_v_empty, (j - 1) & 1)) ok = false;
                }
                if (ok && !mbar_wait_bounded(b_raw + sl * 8, ph)) ok = false;
                if (*failed) ok = false;
                if (!ok) { *failed = 1; atomicOr(a.status, ST_WAIT_TIMEOUT); }
                TC_ACC(c_wait);
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            const uint8_t* rp = slot_ptr(sl);
            uint8_t* out = sKV + (is_v ? 2 * QBUF : (uint32_t)(j & 1) * QBUF) + (uint32_t)pg * 2048u;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const uint4 raw = *reinterpret_cast<const uint4*>(rp + lane * 16 + i * 512);
                uint8_t* o = out + (i >> 1) * 1024;
                uint4 x, y;
                if (!is_v) {
                    const uint32_t sc = *reinterpret_cast<const uint16_t*>(rp + src_sc + i * (4 * (D / 32) * 2));
                    q8_unpack_k16<BF16>(raw, sc | (sc << 16), x, y);
                } else {
                    const uint32_t sc = *reinterpret_cast<const uint32_t*>(rp + src_sc + i * 8);
                    q8_unpack_v8x2<BF16>(raw, sc, x, y);
                }
                *reinterpret_cast<uint4*>(o + d0[i & 1]) = x;
                *reinterpret_cast<uint4*>(o + d1[i & 1]) = y;
            }
            // A finished tile goes to the tensor pipe's proxy.  The slot's next copy needs no fence: every lane's
            // loads from the slot have returned their values (the stores above used them) before the warp meets.
            if (lane == 0) TC_ACC(c_conv);
            if (pg == 7) fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
                TC_ACC(c_meet);
                if (issued < n_recs) issue(issued, sl);
                if (pg == 7) mbar_arrive(is_v ? b_v_full : b_kv_full + (j & 1) * 8);
                TC_ACC(c_issue);
            }
            if (issued < n_recs) issued++;
            if (++sl == n_slots) { sl = 0; ph ^= 1; }
        }
        // never leave with a copy in flight: the records n .. issued - 1 have been asked for and not taken
        if (lane == 0)
            for (; n < issued; n++) {
                if (!mbar_wait_bounded(b_raw + sl * 8, ph)) { *failed = 1; atomicOr(a.status, ST_WAIT_TIMEOUT); }
                if (++sl == n_slots) { sl = 0; ph ^= 1; }
            }
        TC_DUMP(if (tid == 18 * 32) { unsigned long long* b = a.dbg_buf + (size_t)blockIdx.x * 16; b[0] = c_wait; b[1] = c_issue + c_conv + c_meet; b[12] = c_conv; b[13] = c_meet; b[14] = c_issue; b[15] = n_tiles; });
        (void)c_wait; (void)c_issue; (void)c_conv; (void)c_meet; (void)tprev;
    } else if (!Q8 && warp == 0) {
        // ------------------------------------------------------------ TMA producer
        bool ok = true;
        long long tprev = TC_NOW(), c_wait = 0, c_issue = 0;
#pragma unroll 1
        for (int j = 0; j < n_tiles && ok; j++) {
            const int st = j & 1;
            if (lane == 0) {
                if (j >= 2 && !mbar_wait_bounded(b_kv_empty + st * 8, ((j >> 1) - 1) & 1)) ok = false;
                TC_ACC(c_wait);
                if (*failed) ok = false;
                if (ok) mbar_expect_tx(b_kv_full + st * 8, STAGE);
                else { *failed = 1; atomicOr(a.status, ST_WAIT_TIMEOUT); }
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            for (int bx = lane; bx < 8 * XB; bx += 32) {
                const int pg = bx / XB, x = bx - pg * XB;
                const int idx = min(j * 8 + pg, p_hi - p_lo);  // pages past the end repeat the last one (masked)
                int phys = idx < kPageCap ? s_pages[idx] : a.step.tables[sm.tbl_off + p_lo + idx];
                if (phys < 0 || phys >= a.geo.num_pages) { atomicOr(a.status, ST_BAD_PAGE); phys = 0; }
                tma_load_2d(smem_u32(sKV + st * STAGE + x * BLKKV + pg * 4096), &tmap32, x * 64, (phys * Hkv + h) * 32, b_kv_full + st * 8);
            }
            if (lane == 0) TC_ACC(c_issue);
        }
        TC_DUMP(if (lane == 0) { a.dbg_buf[(size_t)blockIdx.x * 16 + 0] = c_wait; a.dbg_buf[(size_t)blockIdx.x * 16 + 1] = c_issue; a.dbg_buf[(size_t)blockIdx.x * 16 + 15] = n_tiles; });
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t id_qk = instr_desc(BF16, 128, 128, false);
            const uint32_t id_pv = instr_desc(BF16, 128, D, true);
            // float layer: a stage holds pages as they lie in device memory (K and V rows of a page interleaved in
            // groups of eight); int8 layer: the loader warps lay K and V out separately (see the shared memory map)
            constexpr uint32_t KBUF = Q8 ? QBUF : STAGE, KBLK = Q8 ? QBLK : BLKKV, GRP = Q8 ? 1024u : 2048u, VPAGE = Q8 ? 2048u : 4096u;
            const uint64_t dq = smem_desc(smem_u32(sQ), 16, 1024), dk = smem_desc(smem_u32(sKV), 16, GRP);
            const uint64_t dv = smem_desc(smem_u32(sKV) + (Q8 ? 2 * QBUF : 1024u), KBLK, GRP);
            auto issue_qk = [&](int X, int j) {
                const uint64_t kst = (uint64_t)(((j & 1) * KBUF) >> 4), qst = (uint64_t)((X * TILE) >> 4);
#pragma unroll
                for (int ks = 0; ks < D / 16; ks++) {
                    const uint64_t qoff = (uint64_t)(((ks >> 2) * BLK + (ks & 3) * 32) >> 4);
                    const uint64_t koff = (uint64_t)(((ks >> 2) * KBLK + (ks & 3) * 32) >> 4);
                    umma(tmem + X * 128, dq + qst + qoff, dk + kst + koff, id_qk, ks > 0);
                }
                umma_commit(b_s_full + X * 8);
                if (Q8 && X == 1) umma_commit(b_kv_empty + (j & 1) * 8);  // both tiles' scores of this K buffer have been issued
            };
            auto issue_pv = [&](int X, int j) {
                const uint64_t vst = Q8 ? 0ull : (uint64_t)(((j & 1) * STAGE) >> 4);
#pragma unroll
                for (int ks = 0; ks < 8; ks++)  // 16 keys = one page per step; P: 8 packed columns per step
                    umma_ts(tmem + 256 + X * 128, tmem + X * 128 + ks * 8, dv + vst + (uint64_t)((ks * VPAGE) >> 4), id_pv, (j > 0 || ks > 0));
                umma_commit(b_o_done + X * 8);
            };
            long long tprev = TC_NOW(), c_wkv = 0, c_wp = 0, c_iss = 0, c_pv = 0;
            bool ok = n_tiles == 0 || mbar_wait_bounded(b_kv_full, 0);  // an empty slice of a cut item: nothing to issue
            if (ok && n_tiles > 0) { tc_fence_after(); issue_qk(0, 0); issue_qk(1, 0); }
            for (int j = 0; ok && j < n_tiles; j++) {
                TC_ACC(c_iss);
                ok = mbar_wait_bounded(b_p_full, j & 1) && !*failed;
                TC_ACC(c_wp);
                if (Q8 && ok) { ok = mbar_wait_bounded(b_v_full, j & 1); TC_ACC(c_wkv); }
                if (!ok) break;
                tc_fence_after();
                issue_pv(0, j);
                TC_ACC(c_pv);
                if (j + 1 < n_tiles) {
                    ok = mbar_wait_bounded(b_kv_full + ((j + 1) & 1) * 8, ((j + 1) >> 1) & 1);
                    TC_ACC(c_wkv);
                    if (!ok) break;
                    tc_fence_after();
                    issue_qk(0, j + 1);
                }
                TC_ACC(c_iss);
                ok = mbar_wait_bounded(b_p_full + 8, j & 1) && !*failed;
                TC_ACC(c_wp);
                if (!ok) break;
                tc_fence_after();
                issue_pv(1, j);
                TC_ACC(c_pv);
                // every read of this stage (int8 layer: of the V buffer) has been issued before
                umma_commit(Q8 ? b_v_empty : b_kv_empty + (j & 1) * 8);
                if (j + 1 < n_tiles) issue_qk(1, j + 1);
            }
            if (!ok) { *failed = 1; atomicOr(a.status, ST_WAIT_TIMEOUT); }
            (void)c_pv;
            TC_DUMP(a.dbg_buf[(size_t)blockIdx.x * 16 + 2] = c_wkv; a.dbg_buf[(size_t)blockIdx.x * 16 + 3] = c_wp; a.dbg_buf[(size_t)blockIdx.x * 16 + 4] = c_iss;
                    a.dbg_buf[(size_t)blockIdx.x * 16 + 11] = c_pv;);
        }
    } else if (warp >= 2 && warp < 18) {
        // ------------------------------------------------------------ softmax + epilogue of tile X, half H of the keys
        const int X = (warp - 2) >> 3, H = ((warp - 2) >> 2) & 1;
        const int lane_base = (warp & 3) * 32;  // the quarter of the tensor-memory lanes this warp may touch
        const int m = lane_base + lane;
        const int rep = m / TPT, r = r0 + X * TPT + (m - rep * TPT);
        const bool row_ok = rep < n_rep && r < sm.snew;
        const int q_pos = sm.pos + min(r, sm.snew - 1);
        const int qx_min = sm.pos + min(r0 + X * TPT, sm.snew - 1), qx_max = sm.pos + min(r0 + (X + 1) * TPT, sm.snew) - 1;
        const uint32_t lane_addr = (uint32_t)lane_base << 16;
        const uint32_t tS = tmem + X * 128 + lane_addr, tO = tmem + 256 + X * 128 + lane_addr;
        const int pair_bar = 1 + X * 4 + (warp & 3);  // named barrier of the two warps that share this quarter of tile X
        auto pair_sync = [&]() { asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory"); };
        // A named barrier has no time limit, so the two warps of a pair must leave the loop in the same
        // iteration: whichever sees a wait run out says so here before the pair's barrier, both read it after.
        volatile int* pair_failed = reinterpret_cast<volatile int*>(s_xch + 2 * 2 * 128 * 2) + X * 4 + (warp & 3);
        float m_ref = -INFINITY, l_run = 0.f;  // l_run: this half's share of the row sum
        bool ok = true;
        long long tprev = TC_NOW(), c_ws = 0, c_ld = 0, c_exp = 0, c_wo = 0, c_st = 0;
        const long long tstart = tprev;
#pragma unroll 1
        for (int j = 0; j < n_tiles; j++) {
            ok = mbar_wait_bounded(b_s_full + X * 8, j & 1) && !*failed;
            ok = __all_sync(0xffffffffu, ok);
            TC_ACC(c_ws);
            if (!ok && lane == 0) *pair_failed = 1;  // the loads below then read stale columns: harmless, nothing is kept
            tc_fence_after();
            const int kbase = k0 + j * 128 + H * 64;
            const bool need_mask = (kbase + 63 > qx_min) || (a.window > 0 && kbase + a.window <= max(qx_max, qx_min));
            // this half of the row of S in registers: maximum, exponentials, packed P back over the S columns
            uint32_t sv[64];
            tmem_ld_row<64>(tS + H * 64, sv);
            if (need_mask) {
#pragma unroll
                for (int e = 0; e < 64; e++) {
                    const int kp = kbase + e;
                    if (!(kp <= q_pos && (a.window <= 0 || kp + a.window > q_pos))) sv[e] = 0xff800000u;  // -inf
                }
            }
            float mx;
            {
                float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
                for (int e = 0; e < 64; e += 4) {
                    m0 = fmaxf(m0, __uint_as_float(sv[e])); m1 = fmaxf(m1, __uint_as_float(sv[e + 1]));
                    m2 = fmaxf(m2, __uint_as_float(sv[e + 2])); m3 = fmaxf(m3, __uint_as_float(sv[e + 3]));
                }
                mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
            }
            // the other half's maximum (double-buffered by tile parity: the partner may still be reading the
            // previous tile's entry when this one is written only if it were two tiles behind, which the
            // barrier of the tile in between rules out)
            float* xrow = s_xch + (((j & 1) * 2 + X) * 128 + m) * 2;
            xrow[H] = mx;
            pair_sync();  // also: both warps have their S columns in registers, so P may overwrite them
            mx = fmaxf(mx, xrow[H ^ 1]) * a.scale_log2;
            if (*pair_failed) { ok = false; break; }  // both warps of the pair, in the same iteration
            TC_ACC(c_ld);
            float alpha = 1.f;
            if (mx > m_ref + 8.f || m_ref == -INFINITY) {  // both halves see the same mx: the same decision
                alpha = (m_ref == -INFINITY) ? 0.f : exp2f(m_ref - mx);
                m_ref = mx;
            }
            const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
            float sum = 0.f, sum2 = 0.f;
#pragma unroll
            for (int e = 0; e < 64; e += 2) {
                const float p0 = ex2_approx(fmaf(__uint_as_float(sv[e]), a.scale_log2, -m_use));
                const float p1 = ex2_approx(fmaf(__uint_as_float(sv[e + 1]), a.scale_log2, -m_use));
                if (e & 2) sum2 += p0 + p1; else sum += p0 + p1;
                sv[e >> 1] = pack2<BF16>(p0, p1);  // P pair e/2 reuses a register whose score is already consumed
            }
#pragma unroll
            for (int c = 0; c < 2; c++) {  // keys 64 H .. 64 H + 63 are packed columns 32 H .. 32 H + 31 of P
                asm volatile(
                    "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                    ::"r"(tS + H * 32 + c * 16), "r"(sv[c * 16 + 0]), "r"(sv[c * 16 + 1]), "r"(sv[c * 16 + 2]), "r"(sv[c * 16 + 3]), "r"(sv[c * 16 + 4]),
                      "r"(sv[c * 16 + 5]), "r"(sv[c * 16 + 6]), "r"(sv[c * 16 + 7]), "r"(sv[c * 16 + 8]), "r"(sv[c * 16 + 9]), "r"(sv[c * 16 + 10]),
                      "r"(sv[c * 16 + 11]), "r"(sv[c * 16 + 12]), "r"(sv[c * 16 + 13]), "r"(sv[c * 16 + 14]), "r"(sv[c * 16 + 15]) : "memory");
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            l_run = l_run * alpha + (sum + sum2);
            TC_ACC(c_exp);
            // S_X being full means P V_X of the previous tile has completed (the tensor pipe runs in
            // order), so O_X may be rescaled now: this warp takes the O columns 64 H .. 64 H + 63
            if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll 1
                for (int c = 0; c < 2; c++) {
                    uint32_t ov[32];
                    tmem_ld32(tO + H * 64 + c * 32, ov);
#pragma unroll
                    for (int e = 0; e < 32; e++) ov[e] = __float_as_uint(__uint_as_float(ov[e]) * alpha);
                    tmem_st32(tO + H * 64 + c * 32, ov);
                }
            }
            tc_fence_before();
            mbar_arrive(b_p_full + X * 8);
            TC_ACC(c_st);
        }
        TC_DUMP(if (tid == 64) {
            unsigned long long* b = a.dbg_buf + (size_t)blockIdx.x * 16;
            b[5] = c_ws; b[6] = c_ld; b[7] = c_exp; b[8] = c_wo; b[9] = c_st; b[10] = TC_NOW() - tstart;
            if (!Q8) { b[12] = 0x7c2; b[13] = tstart - t_entry; }  // float layer: cycles in front of the softmax loop
        });
        const long long t_loop_end = TC_NOW();
        (void)tstart; (void)c_wo; (void)t_loop_end;
        if (ok && n_tiles > 0) ok = mbar_wait_bounded(b_o_done + X * 8, (n_tiles - 1) & 1) && !*failed;
        ok = __all_sync(0xffffffffu, ok);
        // the row sum is the two halves' sums (exchanged whether or not the wait succeeded: the pair must
        // meet at its barrier the same number of times)
        float* xrow = s_xch + ((n_tiles & 1) * 2 + X) * 256 + m * 2;
        xrow[H] = l_run;
        pair_sync();
        const float l_row = l_run + xrow[H ^ 1];
        if (!ok && lane == 0) {
            *failed = 1;
            atomicOr(a.status, ST_WAIT_TIMEOUT);
        }
        uint16_t* orow = reinterpret_cast<uint16_t*>(a.out) +
                         ((size_t)sm.tok_off * a.geo.n_q + (size_t)(h * n_rep + (row_ok ? rep : 0)) * sm.snew + (row_ok ? r : 0)) * D;
        auto store_row = [&](int c, const float (&v)[32], float inv) {  // 32 output columns from c * 32
#pragma unroll
            for (int u = 0; u < 4; u++) {
                uint4 w;
                w.x = pack2<BF16>(v[u * 8 + 0] * inv, v[u * 8 + 1] * inv);
                w.y = pack2<BF16>(v[u * 8 + 2] * inv, v[u * 8 + 3] * inv);
                w.z = pack2<BF16>(v[u * 8 + 4] * inv, v[u * 8 + 5] * inv);
                w.w = pack2<BF16>(v[u * 8 + 6] * inv, v[u * 8 + 7] * inv);
                *reinterpret_cast<uint4*>(orow + c * 32 + u * 8) = w;
            }
        };
        if (parts == 1) {
            if (ok) {
                tc_fence_after();
                const float inv = 1.f / l_row;
#pragma unroll 1
                for (int c = 2 * H; c < 2 * H + 2; c++) {  // this warp writes the output columns 64 H .. 64 H + 63
                    uint32_t v[32];
                    tmem_ld32(tO + c * 32, v);
                    float f[32];
#pragma unroll
                    for (int e = 0; e < 32; e++) f[e] = __uint_as_float(v[e]);
                    if (row_ok) store_row(c, f, inv);
                }
            }
        } else {
            // ---- a slice of a cut item: un-normalised rows and their (reference exponent, sum) go to memory, the
            // CTA draws a ticket, and the CTA that draws the item's last one adds the slices up.  No CTA waits
            // for another; every softmax warp passes both barriers whatever happened to its waits.
            const int cut = item - a.split_first;
            // rows are the fast index of the partial rows in memory (split_o as float4 [slice][tile][32 column
            // groups][128 rows]): a warp's 32 rows make one contiguous 512-byte access
            const size_t mine = ((size_t)(cut * parts + part) * 2 + X) * 128 + m;
            float4* my_o = reinterpret_cast<float4*>(a.split_o) + ((size_t)(cut * parts + part) * 2 + X) * 32 * 128 + m;
            if (ok) {
                if (n_tiles > 0) {
                    tc_fence_after();
#pragma unroll 1
                    for (int c = 2 * H; c < 2 * H + 2; c++) {
                        uint32_t v[32];
                        tmem_ld32(tO + c * 32, v);
#pragma unroll
                        for (int u = 0; u < 8; u++)
                            my_o[(size_t)(c * 8 + u) * 128] = make_float4(__uint_as_float(v[u * 4]), __uint_as_float(v[u * 4 + 1]),
                                                                          __uint_as_float(v[u * 4 + 2]), __uint_as_float(v[u * 4 + 3]));
                    }
                }
                if (H == 0) a.split_ml[mine] = make_float2(n_tiles > 0 ? m_ref : -INFINITY, n_tiles > 0 ? l_row : 0.f);
            }
            __threadfence();
            asm volatile("bar.sync 9, 512;" ::: "memory");
            int* s_ticket = reinterpret_cast<int*>(const_cast<int*>(failed)) + 1;
            if (tid == 64) {
                const int tk = atomicAdd(a.split_counter + cut, 1);
                if (tk == parts - 1) a.split_counter[cut] = 0;  // ready for the next launch
                *s_ticket = tk;
            }
            asm volatile("bar.sync 9, 512;" ::: "memory");
            if (*s_ticket == parts - 1 && ok && !*failed && row_ok) {
                __threadfence();
                const size_t base = ((size_t)cut * parts * 2 + X) * 128 + m;  // slice p: + p * 256
                float mx = -INFINITY;
                for (int p = 0; p < parts; p++) mx = fmaxf(mx, __ldcg(&a.split_ml[base + (size_t)p * 256].x));
                float wsum = 0.f;
                for (int p = 0; p < parts; p++) {
                    const float2 ml = __ldcg(&a.split_ml[base + (size_t)p * 256]);
                    if (ml.x != -INFINITY) wsum += ml.y * exp2f(ml.x - mx);
                }
                const float inv = 1.f / wsum;
#pragma unroll 1
                for (int c = 2 * H; c < 2 * H + 2; c++) {
                    float acc[32];
#pragma unroll
                    for (int e = 0; e < 32; e++) acc[e] = 0.f;
                    for (int p = 0; p < parts; p++) {
                        const float mp = __ldcg(&a.split_ml[base + (size_t)p * 256].x);
                        if (mp == -INFINITY) continue;  // an empty slice, or rows it never saw: its rows were not written
                        const float w = exp2f(mp - mx);
                        const float4* src = reinterpret_cast<const float4*>(a.split_o) + ((size_t)(cut * parts + p) * 2 + X) * 32 * 128 + m;
#pragma unroll
                        for (int u = 0; u < 8; u++) {
                            const float4 t = __ldcg(src + (size_t)(c * 8 + u) * 128);
                            acc[u * 4] += w * t.x; acc[u * 4 + 1] += w * t.y; acc[u * 4 + 2] += w * t.z; acc[u * 4 + 3] += w * t.w;
                        }
                    }
                    store_row(c, acc, inv);
                }
            }
        }
        TC_DUMP(if (tid == 64 && !Q8) { a.dbg_buf[(size_t)blockIdx.x * 16 + 14] = TC_NOW() - t_loop_end; });
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
}

template <bool BF16>
static cudaError_t launch_tc2(const CUtensorMap& map32, const CUtensorMap& map_sc, const ChunkArgs& a, cudaStream_t st) {
    if (a.n_items <= 0) return cudaSuccess;
    const int grid = a.split_parts > 1 ? a.split_first + (a.n_items - a.split_first) * a.split_parts : a.n_items;
    if (a.q8_arena) chunk_tc2_kernel<128, BF16, true><<<grid, kThreads2Q8, tc2_smem_bytes_q8<128>(), st>>>(map32, map_sc, a);
    else chunk_tc2_kernel<128, BF16, false><<<grid, kThreads2, tc2_smem_bytes<128>(), st>>>(map32, map_sc, a);
    return cudaGetLastError();
}

bool chunk_tc2_supported(int d) { return d == 128; }

// Two query tiles per CTA (head_dim 128): the work list has one item per pair of tiles.
cudaError_t launch_chunk_tc2(const CUtensorMap& map32, const CUtensorMap& map_sc, const ChunkArgs& a, bool bf16, cudaStream_t st) {
    if (a.geo.d != 128) return cudaErrorInvalidValue;
    return bf16 ? launch_tc2<true>(map32, map_sc, a, st) : launch_tc2<false>(map32, map_sc, a, st);
}

bool chunk_tc_supported(int d) { return d == 64 || d == 128 || d == 256; }

cudaError_t chunk_tc_init() {
    cudaError_t e;
    if ((e = cudaFuncSetAttribute(chunk_tc_kernel<64, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc_smem_bytes<64>())) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(chunk_tc_kernel<64, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc_smem_bytes<64>())) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(chunk_tc_kernel<128, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc_smem_bytes<128>())) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(chunk_tc_kernel<128, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc_smem_bytes<128>())) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(chunk_tc_kernel<256, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc_smem_bytes<256>())) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(chunk_tc_kernel<256, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc_smem_bytes<256>())) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(chunk_tc2_kernel<128, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc2_smem_bytes<128>())) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(chunk_tc2_kernel<128, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc2_smem_bytes<128>())) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(chunk_tc2_kernel<128, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc2_smem_bytes_q8<128>())) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(chunk_tc2_kernel<128, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc2_smem_bytes_q8<128>())) != cudaSuccess) return e;
    return cudaSuccess;
}

// `map` must be the 16-row box view of the layer (one K or V tile of a page per box).
cudaError_t launch_chunk_tc(const CUtensorMap& map, const CUtensorMap& map32, const ChunkArgs& a, bool bf16, cudaStream_t st) {
    switch (a.geo.d) {
        case 64: return bf16 ? launch_tc<64, true>(map, map32, a, st) : launch_tc<64, false>(map, map32, a, st);
        case 128: return bf16 ? launch_tc<128, true>(map, map32, a, st) : launch_tc<128, false>(map, map32, a, st);
        case 256: return bf16 ? launch_tc<256, true>(map, map32, a, st) : launch_tc<256, false>(map, map32, a, st);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace cbkv
