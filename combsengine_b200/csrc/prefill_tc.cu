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
//   warp 0        TMA producer: K and V boxes of 8 pages per tile, two stages
//   warp 1        one thread issues tcgen05.mma: S = Q K^T (two S buffers), O += P V
//   warps 2..5    softmax: one TMEM lane (row) per thread, P written to shared memory
//                 in the K-major swizzled layout, O rescaled in TMEM when a row max moves
//
// Tensor memory: S0 [0,128), S1 [128,256), O [256, 256 + D) -> 512 columns allocated.
// Shared memory: Q, 2 x K, 2 x V, P tiles of 128 rows x D (or 128 keys), each stored as
// D/64 blocks of 128 rows x 128 bytes with the 128-byte swizzle TMA produces.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>

#include "kernels.hpp"

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
    const uint64_t t0 = global_ns();
    while (!mbar_try_wait(bar, parity))
        if (global_ns() - t0 > limit_ns) return false;
    return true;
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

constexpr int kThreads = 192;
constexpr int kTmemCols = 512;

template <int D>
constexpr int tc_smem_bytes() {
    // Q + 2 K + 2 V tiles of 128 rows x D, P tile of 128 rows x 128 keys, barriers and flags; at least
    // 120 KB so that two CTAs never share an SM (each allocates all 512 tensor-memory columns)
    return (5 * 128 * D * 2 + 128 * 128 * 2 + 256) < 120 * 1024 ? 120 * 1024 : (5 * 128 * D * 2 + 128 * 128 * 2 + 256);
}

}  // namespace

template <int D, bool BF16>
__global__ void __launch_bounds__(kThreads) chunk_tc_kernel(const __grid_constant__ CUtensorMap tmap, const ChunkArgs a) {
    constexpr uint32_t TILE = 128u * D * 2u;   // one operand tile (Q, K or V)
    constexpr uint32_t BLK = 128u * 128u;      // one 64-element column block of a tile: 128 rows x 128 bytes
    constexpr int XB = D / 64;                 // column blocks per row
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sQ = smem;
    uint8_t* sK = sQ + TILE;            // 2 stages
    uint8_t* sV = sK + 2 * TILE;        // 2 stages
    uint8_t* sP = sV + 2 * TILE;        // 128 x 128 keys
    uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 128 * 128 * 2);
    // barriers: kv_full[2], kv_empty[2], s_full[2], p_full, o_done
    const uint32_t b_kv_full = smem_u32(bars + 0), b_kv_empty = smem_u32(bars + 2), b_s_full = smem_u32(bars + 4);
    const uint32_t b_p_full = smem_u32(bars + 6), b_o_done = smem_u32(bars + 7);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
    volatile int* failed = reinterpret_cast<volatile int*>(bars + 9);

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
    const int n_tiles = (p_hi - p_lo + 1 + 7) >> 3;
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
        if (lane == 0) {
            for (int j = 0; j < n_tiles; j++) {
                const int st = j & 1;
                if (j >= 2 && !mbar_wait_bounded(b_kv_empty + st * 8, ((j >> 1) - 1) & 1)) { *failed = 1; atomicOr(a.status, ST_WAIT_TIMEOUT); break; }
                if (*failed) break;
                mbar_expect_tx(b_kv_full + st * 8, 2 * TILE);
                for (int pg = 0; pg < 8; pg++) {
                    // pages past the last visible one repeat it: finite data that the causal mask hides
                    const int lp = min(p_lo + j * 8 + pg, p_hi);
                    int phys = a.step.tables[sm.tbl_off + lp];
                    if (phys < 0 || phys >= a.geo.num_pages) { atomicOr(a.status, ST_BAD_PAGE); phys = 0; }
                    const int row = (phys * Hkv + h) * 32;
#pragma unroll
                    for (int x = 0; x < XB; x++) {
                        tma_load_2d(smem_u32(sK + st * TILE + x * BLK + pg * 2048), &tmap, x * 64, row, b_kv_full + st * 8);
                        tma_load_2d(smem_u32(sV + st * TILE + x * BLK + pg * 2048), &tmap, x * 64, row + 16, b_kv_full + st * 8);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t id_qk = instr_desc(BF16, 128, 128, false);
            const uint32_t id_pv = instr_desc(BF16, 128, D, true);
            auto issue_qk = [&](int j) {
                const int st = j & 1;
                const uint32_t ka = smem_u32(sK + st * TILE), qa = smem_u32(sQ);
#pragma unroll
                for (int ks = 0; ks < D / 16; ks++) {
                    const uint32_t off = (ks >> 2) * BLK + (ks & 3) * 32;  // 16 elements = 32 bytes inside the swizzled row
                    umma(tS0 + (j & 1) * 128, smem_desc(qa + off, 16, 1024), smem_desc(ka + off, 16, 1024), id_qk, ks > 0);
                }
                umma_commit(b_s_full + (j & 1) * 8);
            };
            bool ok = mbar_wait_bounded(b_kv_full, 0);
            if (ok) { tc_fence_after(); issue_qk(0); }
            for (int j = 0; ok && j < n_tiles; j++) {
                if (j + 1 < n_tiles) {
                    ok = mbar_wait_bounded(b_kv_full + ((j + 1) & 1) * 8, ((j + 1) >> 1) & 1);
                    if (!ok) break;
                    tc_fence_after();
                    issue_qk(j + 1);
                }
                ok = mbar_wait_bounded(b_p_full, j & 1) && !*failed;
                if (!ok) break;
                tc_fence_after();
                const int st = j & 1;
                const uint32_t pa = smem_u32(sP), va = smem_u32(sV + st * TILE);
#pragma unroll
                for (int ks = 0; ks < 8; ks++) {  // 16 keys per step
                    // P: K-major, keys 16 ks.. inside key block ks / 4; V: MN-major, 64-wide d blocks BLK apart,
                    // groups of 8 keys 1024 bytes apart, 16 keys = 2048 bytes per step
                    umma(tO, smem_desc(pa + (ks >> 2) * BLK + (ks & 3) * 32, 16, 1024), smem_desc(va + ks * 2048, BLK, 1024), id_pv,
                         (j > 0 || ks > 0));
                }
                umma_commit(b_kv_empty + st * 8);
                umma_commit(b_o_done);
            }
            if (!ok) { *failed = 1; atomicOr(a.status, ST_WAIT_TIMEOUT); }
        }
    } else {
        // ------------------------------------------------------------ softmax + epilogue, one row per thread
        const int lane_base = (warp & 3) * 32;             // the TMEM lanes this warp may touch
        const int m = lane_base + lane;                    // row of the tile
        const int rep = m / TPT, r = r0 + (m - rep * TPT);
        const bool row_ok = rep < n_rep && r < sm.snew;
        const int q_pos = sm.pos + min(r, sm.snew - 1);    // rows past the data mimic the last token
        const uint32_t lane_addr = (uint32_t)lane_base << 16;
        float m_run = -INFINITY, l_run = 0.f;
        bool ok = true;
        for (int j = 0; j < n_tiles; j++) {
            ok = mbar_wait_bounded(b_s_full + (j & 1) * 8, (j >> 1) & 1) && !*failed;
            ok = __all_sync(0xffffffffu, ok);  // the tensor-memory accesses below need the whole warp
            if (!ok) break;
            tc_fence_after();
            const uint32_t tS = tS0 + (j & 1) * 128 + lane_addr;
            const int kbase = k0 + j * 128;
            const bool need_mask = (kbase + 127 > q_min) || (a.window > 0 && kbase + a.window <= q_max);
            // pass 1: row maximum
            float mx = -INFINITY;
#pragma unroll 1
            for (int c = 0; c < 4; c++) {
                uint32_t v[32];
                tmem_ld32(tS + c * 32, v);
#pragma unroll
                for (int e = 0; e < 32; e++) {
                    float s = __uint_as_float(v[e]) * a.scale_log2;
                    if (need_mask) {
                        const int kp = kbase + c * 32 + e;
                        if (!(kp <= q_pos && (a.window <= 0 || kp + a.window > q_pos))) s = -INFINITY;
                    }
                    mx = fmaxf(mx, s);
                }
            }
            const float m_new = fmaxf(m_run, mx);
            const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
            const float alpha = exp2f(m_run - m_use);
            // the previous P V must be finished before P is overwritten and O rescaled
            if (j > 0) {
                ok = mbar_wait_bounded(b_o_done, (j - 1) & 1) && !*failed;
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
            }
            // pass 2: probabilities -> P (keys along the row, K-major swizzled), row sum
            float sum = 0.f;
#pragma unroll 1
            for (int c = 0; c < 4; c++) {
                uint32_t v[32];
                tmem_ld32(tS + c * 32, v);
                uint32_t pk[16];
#pragma unroll
                for (int e = 0; e < 32; e += 2) {
                    float s0 = __uint_as_float(v[e]) * a.scale_log2, s1 = __uint_as_float(v[e + 1]) * a.scale_log2;
                    if (need_mask) {
                        const int kp = kbase + c * 32 + e;
                        if (!(kp <= q_pos && (a.window <= 0 || kp + a.window > q_pos))) s0 = -INFINITY;
                        if (!(kp + 1 <= q_pos && (a.window <= 0 || kp + 1 + a.window > q_pos))) s1 = -INFINITY;
                    }
                    const float p0 = exp2f(s0 - m_use), p1 = exp2f(s1 - m_use);
                    sum += p0 + p1;
                    pk[e >> 1] = pack2<BF16>(p0, p1);
                }
#pragma unroll
                for (int u = 0; u < 4; u++) {  // four 16-byte pieces = 32 keys
                    const int jj = (c & 1) * 4 + u;
                    const uint32_t off = (c >> 1) * BLK + m * 128u + ((jj ^ (m & 7)) << 4);
                    *reinterpret_cast<uint4*>(sP + off) = make_uint4(pk[u * 4], pk[u * 4 + 1], pk[u * 4 + 2], pk[u * 4 + 3]);
                }
            }
            l_run = l_run * alpha + sum;
            m_run = m_new;
            // rescale O when some row of this warp moved its maximum
            if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll 1
                for (int c = 0; c < D / 32; c++) {
                    uint32_t v[32];
                    tmem_ld32(tO + lane_addr + c * 32, v);
#pragma unroll
                    for (int e = 0; e < 32; e++) v[e] = __float_as_uint(__uint_as_float(v[e]) * alpha);
                    tmem_st32(tO + lane_addr + c * 32, v);
                }
            }
            fence_proxy_async();   // P for the async proxy
            tc_fence_before();     // the tensor-memory traffic above is ordered before the hand-over
            mbar_arrive(b_p_full);
        }
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
static cudaError_t launch_tc(const CUtensorMap& map, const ChunkArgs& a, cudaStream_t st) {
    if (a.n_items <= 0) return cudaSuccess;
    chunk_tc_kernel<D, BF16><<<a.n_items, kThreads, tc_smem_bytes<D>(), st>>>(map, a);
    return cudaGetLastError();
}

bool chunk_tc_supported(int d) { return d == 64 || d == 128; }

cudaError_t chunk_tc_init() {
    cudaError_t e;
    if ((e = cudaFuncSetAttribute(chunk_tc_kernel<64, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc_smem_bytes<64>())) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(chunk_tc_kernel<64, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc_smem_bytes<64>())) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(chunk_tc_kernel<128, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc_smem_bytes<128>())) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(chunk_tc_kernel<128, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc_smem_bytes<128>())) != cudaSuccess) return e;
    return cudaSuccess;
}

// `map` must be the 16-row box view of the layer (one K or V tile of a page per box).
cudaError_t launch_chunk_tc(const CUtensorMap& map, const ChunkArgs& a, bool bf16, cudaStream_t st) {
    switch (a.geo.d) {
        case 64: return bf16 ? launch_tc<64, true>(map, a, st) : launch_tc<64, false>(map, a, st);
        case 128: return bf16 ? launch_tc<128, true>(map, a, st) : launch_tc<128, false>(map, a, st);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace cbkv
