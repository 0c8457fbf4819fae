// CUDA kernels of the paged KV path, written for sm_100a.
//
//   append_kernel   scatter of a step's new K/V rows into page slots
//                   (reference: the slice_assign loop, kv.rs:721-734)
//   decode_kernel   GQA decode attention read in place from the pages, with the
//                   append fused in: no gather copy (kv.rs:611-636), no repeat_kv
//                   (kv.rs:177-187), no f32 upcast pass (kv.rs:213-215)
//   chunk_kernel    attention of a chunk of new tokens over paged prefix + chunk
//                   (causal, bottom-right aligned, optional window; kv.rs:243-268)
//   generic_kernel  any page size / head_dim; one warp per query row
//
// Layout of one layer in HBM: pages [num_pages][n_kv][32 rows][d] (f16/bf16).  The 32
// rows of one (page, kv head) are [K slots 0-7][V slots 0-7][K slots 8-15][V slots 8-15]
// (page_row() in kernels.hpp).
// A tile reaches shared memory through one TMA box per 64-element column block
// (32 rows x 128 B, 128-byte swizzle), so ldmatrix reads are bank-conflict free.
//
// Math per tile (16 tokens) in a warp, all in registers:
//   S^T[16 tok x 8 col] = K[16 x d] . Q^T[d x 8 col]      mma.m16n8k16, f32 accumulate
//   online softmax over tokens: warp shuffles across the 8 row groups
//   O^T[d x 8 col]     += V^T[d x 16 tok] . P^T[16 tok x 8 col]
// A "column" is one (query token, q head of the kv group): for decode the 8 columns
// are the q heads that share the kv head, so K/V are read once for the whole group.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>

#include "kernels.hpp"
#include "q8_unpack.cuh"

namespace cbkv {

// ------------------------------------------------------------------ PTX helpers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
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
// Non-blocking look at a barrier phase (try_wait may suspend the thread for a while).
__device__ __forceinline__ uint32_t mbar_test_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}
// Bounded wait: gives up after `limit_ns` of wall time and returns false (the caller
// records it in the status word and stops consuming; nothing spins forever).
__device__ __forceinline__ uint64_t global_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, uint64_t limit_ns = 100000000ull) {
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
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
    uint32_t y;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
    return y;
}
template <bool BF16>
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    if constexpr (BF16) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    } else {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
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
template <bool BF16>
__device__ __forceinline__ uint16_t to_elem(float x) {
    if constexpr (BF16) { __nv_bfloat16 v = __float2bfloat16_rn(x); return *reinterpret_cast<uint16_t*>(&v); }
    else { __half v = __float2half_rn(x); return *reinterpret_cast<uint16_t*>(&v); }
}
template <bool BF16>
__device__ __forceinline__ float from_elem(uint16_t x) {
    if constexpr (BF16) { return __bfloat162float(*reinterpret_cast<__nv_bfloat16*>(&x)); }
    else { return __half2float(*reinterpret_cast<__half*>(&x)); }
}

// Byte offset of (row, 16-byte chunk j) inside one swizzled 32-row x 128-byte block.
__device__ __forceinline__ uint32_t swz(uint32_t row, uint32_t j) { return row * 128u + ((j ^ (row & 7u)) << 4); }

// One 16-token tile against NT blocks of 8 query columns.
//   stage        shared address of the K|V tile ([D/64] blocks of 32 rows x 128 B)
//   qf           Q^T fragments (B operand), loaded once per work item
//   kpos0        absolute position of the tile's first token
//   qpos         absolute query position of this thread's two columns per block
template <int D, int NT, bool BF16>
__device__ __forceinline__ void attend_tile(uint32_t stage, const uint32_t (&qf)[NT][D / 16][2],
                                            float (&o)[NT][D / 16][4], float (&m)[NT][2], float (&l)[NT][2],
                                            int kpos0, const int (&qpos)[NT][2], int window, float scale_log2,
                                            bool need_mask, int lane) {
    const int g = lane >> 2;
    float s[NT][4], s2[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
        s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
        s2[nt][0] = s2[nt][1] = s2[nt][2] = s2[nt][3] = 0.f;
    }
    // ---- S^T = K . Q^T  (two accumulator chains, summed at the end)
    {
        const uint32_t row = (lane & 7) + ((lane >> 3) & 1) * 16;  // K slot (lane&7) + 8*((lane>>3)&1) -> its row
        const uint32_t jsel = lane >> 4;                           // which of the two 16-byte chunks
#pragma unroll
        for (int ks = 0; ks < D / 16; ks++) {
            uint32_t a[4];
            ldsm_x4(stage + (ks >> 2) * 4096u + swz(row, (ks & 3) * 2 + jsel), a);
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                if (ks & 1) mma_16816<BF16>(s2[nt], a, qf[nt][ks][0], qf[nt][ks][1]);
                else mma_16816<BF16>(s[nt], a, qf[nt][ks][0], qf[nt][ks][1]);
            }
        }
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
#pragma unroll
            for (int i = 0; i < 4; i++) s[nt][i] += s2[nt][i];
        }
    }
    // ---- online softmax over the tile's 16 tokens (rows g and g+8 of the fragment)
    uint32_t pb[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
#pragma unroll
        for (int i = 0; i < 4; i++) s[nt][i] *= scale_log2;
        if (need_mask) {
#pragma unroll
            for (int i = 0; i < 4; i++) {
                int kp = kpos0 + g + (i >> 1) * 8;
                int qp = qpos[nt][i & 1];
                bool ok = kp <= qp && (window <= 0 || kp + window > qp);  // keys in (p - w, p], kv.rs:252-257
                if (!ok) s[nt][i] = -INFINITY;
            }
        }
        float alpha[2];
#pragma unroll
        for (int j = 0; j < 2; j++) {
            float mx = fmaxf(s[nt][j], s[nt][j + 2]);
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
            float m_new = fmaxf(m[nt][j], mx);
            float m_use = (m_new == -INFINITY) ? 0.f : m_new;
            alpha[j] = exp2f(m[nt][j] - m_use);
            m[nt][j] = m_new;
            float p0 = exp2f(s[nt][j] - m_use);
            float p1 = exp2f(s[nt][j + 2] - m_use);
            s[nt][j] = p0;
            s[nt][j + 2] = p1;
            l[nt][j] = l[nt][j] * alpha[j] + p0 + p1;  // this thread's share; reduced over row groups at the end
        }
#pragma unroll
        for (int mt = 0; mt < D / 16; mt++) {
            o[nt][mt][0] *= alpha[0]; o[nt][mt][1] *= alpha[1];
            o[nt][mt][2] *= alpha[0]; o[nt][mt][3] *= alpha[1];
        }
        // P^T as the B operand: transpose the two 8x8 blocks across the warp
        pb[nt][0] = movmatrix_trans(pack2<BF16>(s[nt][0], s[nt][1]));
        pb[nt][1] = movmatrix_trans(pack2<BF16>(s[nt][2], s[nt][3]));
    }
    // ---- O^T += V^T . P^T   (V slots 0-7 are rows 8-15 of the block, slots 8-15 rows 24-31)
    {
        const uint32_t row = 8 + (lane & 7) + (lane >> 4) * 16;  // V slot (lane&7) + 8*(lane>>4) -> its row
        const uint32_t jsel = (lane >> 3) & 1;                   // d chunk
#pragma unroll
        for (int mt = 0; mt < D / 16; mt++) {
            uint32_t a[4];
            ldsm_x4_trans(stage + (mt >> 2) * 4096u + swz(row, (mt & 3) * 2 + jsel), a);
#pragma unroll
            for (int nt = 0; nt < NT; nt++) mma_16816<BF16>(o[nt][mt], a, pb[nt][0], pb[nt][1]);
        }
    }
}

// ------------------------------------------------------------------ int8 pages (kv.rs:271-358)
// A quantised record (kernels.hpp, qrec_*) reaches shared memory as it lies in HBM, by one TMA box.  Values are
// converted in registers by a byte permute that puts a constant exponent byte over each value byte
// and one exact subtraction (q8_pair).  The group scales never touch the values: K's multiply the f32 score partial sums of their 32-wide group, V's multiply the
// probabilities of their token before the P.V product of that group's rows.
//
// The contraction index of an MMA may be permuted freely if both operands agree, and so may the
// output rows of O^T if the store undoes it; that is how a thread gets whole 4- and 8-byte words:
//   K (A operand, row = token): per group a thread takes bytes 8t..8t+7 of rows g and g+8; k-step s
//     contracts d = 32*grp + 8t + 4s + {0,1,2,3} against the Q fragment loaded in the same order.
//   V (A operand of O^T, row = d): per group a thread takes d = 4g..4g+3 of token pairs (2t, 2t+1)
//     and (2t+8, 2t+9), stored pair-interleaved so that one register is one 16-bit pick; m-tile
//     2*grp has rows d = 32*grp + 4g + {0 (row g), 1 (row g+8)}, m-tile 2*grp+1 the other two.
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.b32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t addr) {
    uint16_t v;
    asm volatile("ld.shared.b16 %0, [%1];" : "=h"(v) : "r"(addr));
    return v;
}
// Byte -> number conversions (q8_fix, q8_pair, mul2): q8_unpack.cuh.
template <bool BF16>
__device__ __forceinline__ float2 up2(uint32_t v) {
    if constexpr (BF16) return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&v));
    else return __half22float2(*reinterpret_cast<__half2*>(&v));
}
__device__ __forceinline__ float fast_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// One 16-token quantised tile against the 8 query columns of the kv group (decode), in two steps:
// q8_load copies this thread's share of the record from shared memory to registers, after which the
// ring stage can go back to the producer; q8_attend does the math from registers.  The running
// maximum of a column moves only when the new one exceeds it by 2^8 (the exponentials stay far inside
// the f16 range), so most tiles skip the rescaling of the output accumulators.
template <int D>
struct Q8Tile {
    static constexpr int G = D / 32;
    uint2 kx[G], ky[G], va[G], vb[G];            // K bytes of rows g, g+8; V bytes of token pairs t, t+4
    uint32_t ks0[G / 2], ks1[G / 2], vs0[G], vs1[G];  // their scales
};

template <int D>
__device__ __forceinline__ void q8_load(uint32_t stage, int lane, Q8Tile<D>& r) {
    constexpr int G = D / 32;
    static_assert(G % 2 == 0, "scales are read two at a time");
    const int g = lane >> 2, t = lane & 3;
    const uint32_t kbase = stage, vbase = stage + 16u * D, ksc = stage + 32u * D, vsc = ksc + 16u * G * 2u;
    const int swz = qrec_swz(g, D);  // rows g and g+8 share it
    const uint32_t r0 = kbase + (uint32_t)g * D + 8u * t, r1 = r0 + 8u * D;
#pragma unroll
    for (int grp = 0; grp < G; grp++) {
        const uint32_t off = (uint32_t)((grp ^ swz) << 5);
        r.kx[grp] = lds64(r0 + off);
        r.ky[grp] = lds64(r1 + off);
    }
#pragma unroll
    for (int i = 0; i < G / 2; i++) {
        r.ks0[i] = lds32(ksc + (uint32_t)(g * G + 2 * i) * 2u);
        r.ks1[i] = lds32(ksc + (uint32_t)((g + 8) * G + 2 * i) * 2u);
    }
    // pair t and pair t+4 share the unit and chunk permutation (qrec_value_off)
    const uint32_t c0 = vbase + (uint32_t)t * 2u * D + (uint32_t)((g ^ (4 * ((t >> 1) & 1))) * 8);
#pragma unroll
    for (int grp = 0; grp < G; grp++) {
        const uint32_t off = (uint32_t)((grp ^ (t & 1)) * 64);
        r.va[grp] = lds64(c0 + off);
        r.vb[grp] = lds64(c0 + 8u * D + off);
        r.vs0[grp] = lds32(vsc + (uint32_t)(grp * 16 + 2 * t) * 2u);
        r.vs1[grp] = lds32(vsc + (uint32_t)(grp * 16 + 2 * t + 8) * 2u);
    }
}

template <int D, bool BF16>
__device__ __forceinline__ void q8_attend(const Q8Tile<D>& r, const uint32_t (&qf)[1][D / 16][2], float (&o)[1][D / 16][4],
                                          float (&m)[1][2], float (&l)[1][2], int kpos0, const int (&qpos)[1][2],
                                          int window, float scale_log2, bool need_mask, int lane, int dbg = 0) {
    (void)dbg;  // phase switches exist in the measurement build only
    constexpr int G = D / 32;
    const int g = lane >> 2;
    const uint2 (&kx)[G] = r.kx; const uint2 (&ky)[G] = r.ky; const uint2 (&va)[G] = r.va; const uint2 (&vb)[G] = r.vb;
    const uint32_t (&ks0)[G / 2] = r.ks0; const uint32_t (&ks1)[G / 2] = r.ks1;
    const uint32_t (&vs0)[G] = r.vs0; const uint32_t (&vs1)[G] = r.vs1;
    // ---- S^T = sum over groups of scale_K[token][grp] * (Kq . Q^T)
    float s[4] = {0.f, 0.f, 0.f, 0.f};
#ifdef CBKV_MEASURE
    if (!(dbg & 32))  // skip the score phase
#endif
#pragma unroll
    for (int grp = 0; grp < G; grp++) {
        const uint32_t x0 = q8_fix<BF16>(kx[grp].x), x1 = q8_fix<BF16>(kx[grp].y);
        const uint32_t y0 = q8_fix<BF16>(ky[grp].x), y1 = q8_fix<BF16>(ky[grp].y);
        float sg[4] = {0.f, 0.f, 0.f, 0.f};
        uint32_t a[4];
        a[0] = q8_pair<BF16>(x0, SEL_LO); a[1] = q8_pair<BF16>(y0, SEL_LO);
        a[2] = q8_pair<BF16>(x0, SEL_HI); a[3] = q8_pair<BF16>(y0, SEL_HI);
        mma_16816<BF16>(sg, a, qf[0][2 * grp][0], qf[0][2 * grp][1]);
        a[0] = q8_pair<BF16>(x1, SEL_LO); a[1] = q8_pair<BF16>(y1, SEL_LO);
        a[2] = q8_pair<BF16>(x1, SEL_HI); a[3] = q8_pair<BF16>(y1, SEL_HI);
        mma_16816<BF16>(sg, a, qf[0][2 * grp + 1][0], qf[0][2 * grp + 1][1]);
        const float2 f0 = up2<BF16>(ks0[grp >> 1]), f1 = up2<BF16>(ks1[grp >> 1]);
        const float k0 = (grp & 1) ? f0.y : f0.x, k1 = (grp & 1) ? f1.y : f1.x;
        s[0] += sg[0] * k0; s[1] += sg[1] * k0; s[2] += sg[2] * k1; s[3] += sg[3] * k1;
    }
    // ---- online softmax over the tile's 16 tokens (rows g and g+8 of the fragment)
#pragma unroll
    for (int i = 0; i < 4; i++) s[i] *= scale_log2;
    if (need_mask) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int kp = kpos0 + g + (i >> 1) * 8, qp = qpos[0][i & 1];
            const bool ok = kp <= qp && (window <= 0 || kp + window > qp);
            if (!ok) s[i] = -INFINITY;
        }
    }
    float alpha[2] = {1.f, 1.f};
    bool moved = false;
#ifdef CBKV_MEASURE
    if (!(dbg & 64))  // skip the softmax
#endif
#pragma unroll
    for (int j = 0; j < 2; j++) {
        float mx = fmaxf(s[j], s[j + 2]);
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
        if (mx > m[0][j] + 8.f) {  // also the first finite maximum (m starts at -inf)
            alpha[j] = fast_ex2(m[0][j] - mx);
            m[0][j] = mx;
            moved = true;
        }
        const float m_use = (m[0][j] == -INFINITY) ? 0.f : m[0][j];
        const float p0 = fast_ex2(s[j] - m_use), p1 = fast_ex2(s[j + 2] - m_use);
        s[j] = p0; s[j + 2] = p1;
        l[0][j] = l[0][j] * alpha[j] + p0 + p1;
    }
    if (__any_sync(0xffffffffu, moved)) {
#pragma unroll
        for (int mt = 0; mt < D / 16; mt++) {
            o[0][mt][0] *= alpha[0]; o[0][mt][1] *= alpha[1];
            o[0][mt][2] *= alpha[0]; o[0][mt][3] *= alpha[1];
        }
    }
    uint32_t pb0 = pack2<BF16>(s[0], s[1]), pb1 = pack2<BF16>(s[2], s[3]);
    pb0 = movmatrix_trans(pb0);  // tokens 2t, 2t+1 of column g
    pb1 = movmatrix_trans(pb1);  // tokens 2t+8, 2t+9
    // ---- O^T += sum over groups of Vq^T . (P^T * scale_V[token][grp])
#ifdef CBKV_MEASURE
    if (!(dbg & 128))  // skip the output phase
#endif
#pragma unroll
    for (int grp = 0; grp < G; grp++) {
        const uint32_t a0 = q8_fix<BF16>(va[grp].x), a1 = q8_fix<BF16>(va[grp].y);  // d 4g, 4g+1 | 4g+2, 4g+3 of tokens 2t, 2t+1
        const uint32_t c0 = q8_fix<BF16>(vb[grp].x), c1 = q8_fix<BF16>(vb[grp].y);  // the same of tokens 2t+8, 2t+9
        const uint32_t b0 = mul2<BF16>(pb0, vs0[grp]), b1 = mul2<BF16>(pb1, vs1[grp]);
        uint32_t a[4];
        a[0] = q8_pair<BF16>(a0, SEL_LO); a[1] = q8_pair<BF16>(a0, SEL_HI);
        a[2] = q8_pair<BF16>(c0, SEL_LO); a[3] = q8_pair<BF16>(c0, SEL_HI);
        mma_16816<BF16>(o[0][2 * grp], a, b0, b1);
        a[0] = q8_pair<BF16>(a1, SEL_LO); a[1] = q8_pair<BF16>(a1, SEL_HI);
        a[2] = q8_pair<BF16>(c1, SEL_LO); a[3] = q8_pair<BF16>(c1, SEL_HI);
        mma_16816<BF16>(o[0][2 * grp + 1], a, b0, b1);
    }
}

// Fused append for int8 pages: kv_quantize (kv.rs:284-313) of the step's new K and V rows of one
// (sequence, kv head), written into the tile that was just fetched and into its record in HBM.
// Lane c owns values 4c..4c+3 (a 32-value group = 8 lanes); head_dim <= 128 per round.
template <int D, bool BF16>
__device__ __forceinline__ void q8_append_row(uint32_t stage, uint8_t* recp, const uint16_t* krow, const uint16_t* vrow,
                                              int slot, int lane) {
#pragma unroll
    for (int is_v = 0; is_v < 2; is_v++) {
        const uint2* src = reinterpret_cast<const uint2*>(is_v ? vrow : krow);
#pragma unroll
        for (int c0 = 0; c0 < D / 4; c0 += 32) {
            const int c = c0 + lane;
            const bool live = c < D / 4;
            float x[4] = {0.f, 0.f, 0.f, 0.f};
            if (live) {
                const uint2 raw = src[c];
                x[0] = from_elem<BF16>((uint16_t)(raw.x & 0xffff)); x[1] = from_elem<BF16>((uint16_t)(raw.x >> 16));
                x[2] = from_elem<BF16>((uint16_t)(raw.y & 0xffff)); x[3] = from_elem<BF16>((uint16_t)(raw.y >> 16));
            }
            float amax = fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3])));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
            const float scale = fmaxf(__fdiv_rn(amax, 127.0f), 1e-8f);
            if (live) {
                uint32_t word = 0;
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    float q = roundf(__fdiv_rn(x[i], scale));
                    q = fminf(fmaxf(q, -127.f), 127.f);
                    word |= (uint32_t)((int)q + 128) << (8 * i);
                }
                if (!is_v) {
                    const uint32_t off = (uint32_t)qrec_value_off(0, slot, 4 * c, 16, D);
                    asm volatile("st.shared.b32 [%0], %1;" ::"r"(stage + off), "r"(word) : "memory");
                    *reinterpret_cast<uint32_t*>(recp + off) = word;
                } else {
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const uint32_t off = (uint32_t)qrec_value_off(1, slot, 4 * c + i, 16, D);
                        const uint32_t b = (word >> (8 * i)) & 0xffu;
                        asm volatile("st.shared.u8 [%0], %1;" ::"r"(stage + off), "r"(b) : "memory");
                        recp[off] = (uint8_t)b;
                    }
                }
                if ((c & 7) == 0) {
                    const uint32_t off = (uint32_t)qrec_scale_off(is_v, slot, c >> 3, 16, D);
                    const uint32_t sv = to_elem<BF16>(scale);
                    asm volatile("st.shared.u16 [%0], %1;" ::"r"(stage + off), "h"((uint16_t)sv) : "memory");
                    *reinterpret_cast<uint16_t*>(recp + off) = (uint16_t)sv;
                }
            }
        }
    }
}

// Issue the TMA copies for one (page, kv head) tile: D/64 boxes of 32 rows x 64 elems.
template <int D>
__device__ __forceinline__ void issue_tile(const CUtensorMap* map, uint32_t stage, uint32_t bar, int row0) {
    mbar_expect_tx(bar, 32u * D * 2u);
#pragma unroll
    for (int x = 0; x < D / 64; x++) tma_load_2d(stage + x * 4096u, map, x * 64, row0, bar);
}

// ------------------------------------------------------------------ append
template <typename T>
__global__ void append_kernel(const AppendArgs a) {
    const int D8 = a.geo.d / 8;
    const int64_t total = (int64_t)a.step.n_tokens * a.geo.n_kv * 2 * D8;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        int c = (int)(idx % D8);
        int64_t rem = idx / D8;
        int kv = (int)(rem & 1);
        int64_t row = rem >> 1;  // packed row: sequence blocks of [n_kv][snew] rows
        int lo = 0, hi = a.step.n_seqs - 1;  // last sequence whose first row is <= row
        while (lo < hi) {
            int mid = (lo + hi + 1) >> 1;
            if ((int64_t)a.step.seq_meta[mid].tok_off * a.geo.n_kv <= row) lo = mid; else hi = mid - 1;
        }
        const SeqMeta sm = a.step.seq_meta[lo];
        int64_t local = row - (int64_t)sm.tok_off * a.geo.n_kv;
        int h = (int)(local / sm.snew), r = (int)(local % sm.snew);
        int gpos = sm.pos + r;                         // global = pos + written, kv.rs:725
        int phys = a.step.tables[sm.tbl_off + gpos / a.geo.page_size];  // kv.rs:728
        int slot = gpos % a.geo.page_size;             // kv.rs:726
        if (phys < 0 || phys >= a.geo.num_pages) { atomicOr(a.status, ST_BAD_PAGE); continue; }
        const uint4* src = reinterpret_cast<const uint4*>(kv ? a.v : a.k) + row * D8 + c;
        int64_t drow = ((int64_t)phys * a.geo.n_kv + h) * 2 * a.geo.page_size + page_row(kv, slot, a.geo.page_size, a.geo.tiled != 0);
        reinterpret_cast<uint4*>(a.arena)[drow * D8 + c] = *src;
    }
}

// ------------------------------------------------------------------ decode
// The launch's (sequence, kv head, page) units are cut into work items (manager.hpp): CTA c
// starts with item c and then claims further items from a device counter, larger ones first,
// so CTAs on SMs that stream more slowly take fewer of them and all finish together.  An item
// may cover the tail of one segment, whole segments and the head of another ("pieces").
//
// Warp 0 is the producer: it claims items two ahead, publishes them to the other warps
// through a small queue in shared memory, reads each tile's record index from the per-step
// unit_row array (one coalesced load per 32 tiles) and issues the TMA copies into a CTA-wide
// ring of NS stages.  The next C warps consume: tile n of the CTA (counted across items)
// lives in stage n % NS and belongs to consumer warp n % C, and NS is a multiple of C, so
// every stage has one producer and one consumer that visit it in order (an mbarrier parity
// wait is only unambiguous for a waiter at most one phase ahead).  Each consumer keeps a
// running (max, sum, numerator) state in registers; when a piece ends the states go to
// shared memory and the last warp (merger) combines them off the consumers' path.  A segment
// cut across items leaves partials in global scratch; whoever draws the segment's last ticket
// merges them (nobody waits for another CTA).
//
// Every wait is bounded; a warp that gives up records it in the status word, raises the CTA's
// failure flag and falls through the remaining barriers without computing.  The producer
// leaves last, after every copy it issued has landed.
constexpr int QN = 8;          // slots of the item queue (a power of two)
constexpr int DEFER_CAP = 20;  // segments a CTA can leave to its cooperative merge at the end

struct Piece {
    int sb, se;  // unit range of the segment
    int h;
    int q_pos, page_lo, page_last, tok_off, nparts, part_base;
};

__device__ __forceinline__ Piece load_piece(const DecodeArgs& a, int seg) {
    // this segment's record and the first word of the next one (the array has n_segs + 1 entries)
    const int4* p = reinterpret_cast<const int4*>(a.segs + seg);
    const int4 x = __ldg(p), y = __ldg(p + 1), z = __ldg(p + 2);
    Piece pc;
    pc.sb = x.x; pc.page_lo = x.y; pc.q_pos = x.z; pc.tok_off = x.w;
    pc.nparts = y.x; pc.part_base = y.y;
    pc.se = z.x;
    pc.h = seg % a.geo.n_kv;
    pc.page_last = pc.q_pos >> 4;  // decode: the one new token, at the end of the window
    return pc;
}

template <int D>
__device__ __forceinline__ void load_q_frags(const DecodeArgs& a, const Piece& p, int g, int t, uint32_t (&qf)[1][D / 16][2]) {
    // Q^T fragments of the kv group's q heads (columns >= n_rep are zero)
    const int n_rep = a.geo.n_rep;
    const uint32_t* qrow = reinterpret_cast<const uint32_t*>(
        reinterpret_cast<const uint16_t*>(a.q) + ((size_t)p.tok_off * a.geo.n_q + (size_t)p.h * n_rep + (g < n_rep ? g : 0)) * D);
#pragma unroll
    for (int ks = 0; ks < D / 16; ks++) {
        qf[0][ks][0] = g < n_rep ? __ldg(qrow + ks * 8 + t) : 0u;
        qf[0][ks][1] = g < n_rep ? __ldg(qrow + ks * 8 + 4 + t) : 0u;
    }
}

// The same fragments in the contraction order of the quantised K tiles (see q8_attend).
template <int D>
__device__ __forceinline__ void load_q_frags_q8(const DecodeArgs& a, const Piece& p, int g, int t, uint32_t (&qf)[1][D / 16][2]) {
    const int n_rep = a.geo.n_rep;
    const uint2* qrow = reinterpret_cast<const uint2*>(
        reinterpret_cast<const uint16_t*>(a.q) + ((size_t)p.tok_off * a.geo.n_q + (size_t)p.h * n_rep + (g < n_rep ? g : 0)) * D);
#pragma unroll
    for (int ks = 0; ks < D / 16; ks++) {
        // k-step ks = 2*grp + s contracts d = 32*grp + 8t + 4s + {0..3}: one 8-byte word
        const uint2 v = g < n_rep ? __ldg(qrow + (ks >> 1) * 8 + 2 * t + (ks & 1)) : make_uint2(0u, 0u);
        qf[0][ks][0] = v.x;
        qf[0][ks][1] = v.y;
    }
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void consumer_sync(int nthreads) {
    asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
}
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ int4 lds128(uint32_t addr) {
    int4 v;
    asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, int4 v) {
    asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

#ifdef CBKV_MEASURE
// per-CTA timestamps, 16 slots each
#define CBKV_STAMP(slot) do { if ((a.debug & 4) && a.dbg_buf) a.dbg_buf[(size_t)blockIdx.x * 16 + (slot)] = global_ns(); } while (0)
#define CBKV_DBG(bit) (a.debug & (bit))
#else
#define CBKV_STAMP(slot) do { } while (0)
#define CBKV_DBG(bit) 0
#endif

// Merge the partial results of one segment (log-sum-exp combine) and store its output.
// Thread r of T takes every T-th (column, 4 d-values) item; the loads of up to eight
// parts are issued together, so an item costs one round trip to memory.
template <int D, bool BF16>
__device__ __forceinline__ void merge_parts(const DecodeArgs& a, int base, int nparts, uint16_t* out_row, int n_rep, int r, int T) {
    constexpr int PER_COL = D / 4;
    for (int idx = r; idx < n_rep * PER_COL; idx += T) {
        const int col = idx / PER_COL, j4 = idx - col * PER_COL;
        float M = -INFINITY, L = 0.f;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
        for (int p0 = 0; p0 < nparts; p0 += 8) {
            float2 ml[8];
            float4 v[8];
#pragma unroll
            for (int q = 0; q < 8; q++) {
                const bool ok = p0 + q < nparts;
                const size_t rec = (size_t)(base + p0 + (ok ? q : 0)) * 8 + col;
                ml[q] = __ldcg(reinterpret_cast<const float2*>(a.part_ml) + rec);
                v[q] = __ldcg(reinterpret_cast<const float4*>(a.part_o + rec * D) + j4);
                if (!ok) ml[q] = make_float2(-INFINITY, 0.f);
            }
            float Mnew = M;
#pragma unroll
            for (int q = 0; q < 8; q++) Mnew = fmaxf(Mnew, ml[q].x);
            const float so = (M == -INFINITY) ? 0.f : exp2f(M - Mnew);
            acc.x *= so; acc.y *= so; acc.z *= so; acc.w *= so;
            L *= so;
#pragma unroll
            for (int q = 0; q < 8; q++) {
                const float f = (ml[q].x == -INFINITY) ? 0.f : exp2f(ml[q].x - Mnew);
                acc.x += f * v[q].x; acc.y += f * v[q].y; acc.z += f * v[q].z; acc.w += f * v[q].w;
                L += f * ml[q].y;
            }
            M = Mnew;
        }
        const float inv = 1.f / L;
        uint2 pk;
        pk.x = pack2<BF16>(acc.x * inv, acc.y * inv);
        pk.y = pack2<BF16>(acc.z * inv, acc.w * inv);
        *reinterpret_cast<uint2*>(out_row + col * D + j4 * 4) = pk;
    }
}

// Record index (page * n_kv + kv head) of every unit of a decode plan, once per step and
// window: the decode launches of all layers read it instead of chasing the block tables.
__global__ void resolve_units_kernel(const SegInfo* segs, int n_segs, const int32_t* tables, int n_kv, int num_pages,
                                     int32_t* unit_row, int n_units, int32_t* status,
                                     int32_t* zero_a, int n_a, int32_t* zero_b, int n_b) {
    // the step's first launch of this kernel also puts the tickets and claim counters back to zero (whatever a
    // launch that gave up left behind): one stream operation per step instead of three
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_a; i += gridDim.x * blockDim.x) zero_a[i] = 0;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_b; i += gridDim.x * blockDim.x) zero_b[i] = 0;
    for (int u = blockIdx.x * blockDim.x + threadIdx.x; u < n_units; u += gridDim.x * blockDim.x) {
        int lo = 0, hi = n_segs - 1;  // last segment whose first unit is <= u (an empty segment shares its successor's)
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (segs[mid].unit_begin <= u) lo = mid; else hi = mid - 1;
        }
        const SegInfo sg = segs[lo];
        const int phys = tables[sg.tbl_off + sg.page_lo + (u - sg.unit_begin)];
        if (phys < 0 || phys >= num_pages) {
            atomicOr(status, ST_BAD_PAGE);
            unit_row[u] = -1;  // the decode kernel reads page 0 instead and writes nothing
        } else {
            unit_row[u] = phys * n_kv + lo % n_kv;
        }
    }
}

// Warp roles: 0 = producer, 1..C = consumers, C+1 = merger.
// Q8: the layer holds int8 records; a tile is one record fetched as one box of a byte tensor map.
template <int D, int C, bool BF16, bool Q8>
__global__ void __launch_bounds__((C + 2) * 32) decode_kernel(const __grid_constant__ CUtensorMap tmap, const DecodeArgs a) {
    constexpr uint32_t UNIT = Q8 ? (uint32_t)(2 * 16 * D + 2 * 16 * (D / 32) * 2) : 32u * D * 2u;
    constexpr int DP = D + 4;  // row pitch of the merge buffers: the four lanes of a quad land in different banks
    extern __shared__ __align__(1024) uint8_t smem[];
    const int NS = a.n_stages;            // multiple of C (checked by the host)
    const int ccols = a.comb_cols;
    const int NB = a.comb_bufs;           // 1 or 2 state buffers between consumers and merger
    float* comb_o = reinterpret_cast<float*>(smem + (size_t)NS * UNIT);      // [NB][C][ccols][DP]
    float* comb_ml = comb_o + (size_t)NB * C * ccols * DP;                    // [NB][C][8][2]
    int4* qitems = reinterpret_cast<int4*>(comb_ml + NB * C * 16);            // [QN] published items
    uint64_t* bar_full = reinterpret_cast<uint64_t*>(qitems + QN);           // [NS] tile landed
    uint64_t* bar_empty = bar_full + NS;                                      // [NS] tile consumed
    uint64_t* bar_cfull = bar_empty + NS;                                     // [2] all consumers stored their states
    uint64_t* bar_cempty = bar_cfull + 2;                                     // [2] merger is done with the buffer
    uint64_t* bar_qfull = bar_cempty + 2;                                     // [QN] item published
    uint64_t* bar_qempty = bar_qfull + QN;                                    // [QN] item read by consumers and merger
    int* flag = reinterpret_cast<int*>(bar_qempty + QN);                      // [1] a warp gave up, [2] merges left to the end, [4..4+DEFER_CAP) their segments

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cta = blockIdx.x;
    if ((smem_u32(smem) & 1023u) != 0) {
        if (tid == 0) atomicOr(a.status, ST_SMEM_ALIGN);
        return;
    }
    if (tid == 0) CBKV_STAMP(0);
    const uint32_t ring = smem_u32(smem);
    const uint32_t full0 = smem_u32(bar_full), empty0 = smem_u32(bar_empty);
    const uint32_t cfull0 = smem_u32(bar_cfull), cempty0 = smem_u32(bar_cempty);
    const uint32_t qfull0 = smem_u32(bar_qfull), qempty0 = smem_u32(bar_qempty), qitems0 = smem_u32(qitems);
    const int Hkv = a.geo.n_kv;
    const uint64_t lim = (uint64_t)a.wait_us * 1000ull;
    if (tid == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap) : "memory");
        for (int i = 0; i < NS; i++) { mbar_init(full0 + i * 8, 1); mbar_init(empty0 + i * 8, 1); }
        for (int i = 0; i < 2; i++) { mbar_init(cfull0 + i * 8, C); mbar_init(cempty0 + i * 8, 1); }
        for (int i = 0; i < QN; i++) { mbar_init(qfull0 + i * 8, 1); mbar_init(qempty0 + i * 8, C + 1); }
        flag[0] = 0; flag[1] = 0; flag[2] = 0;
        fence_mbar_init();
        fence_proxy_async();
    }
    __syncthreads();
    volatile int* vflag = flag;

    if (warp == 0) {
        // ------------------------------------------------------------ producer
        // The pages read here were written by earlier steps; only when earlier work in the
        // stream wrote this layer's pages or the unit_row array must it be waited for.
        if (a.kv_dep) pdl_wait();
        bool failed = false;
        const int rshift = NS < 8 ? 2 : 3;  // lanes per issue round (4 or 8): never more than the ring has stages
        auto fetch = [&](int id) -> int4 {
            return id < a.n_items ? __ldg(reinterpret_cast<const int4*>(a.items) + id) : make_int4(-1, -1, 0, 0);
        };
        // A claim is issued (one atomic by lane 0) when an item starts and picked up after the item's
        // first round of copies is out, so the counter's round trip never holds up a copy.
        auto claim_issue = [&]() -> int {
            int v = 0;
            if (lane == 0) v = a.n_ctas + atomicAdd(a.work_counters + a.work_slot, 1);
            return v;
        };
        auto publish = [&](int j, int4 info) {
            if (lane == 0) {
                const int s = j & (QN - 1);
                if (j >= QN && !mbar_wait_bounded(qempty0 + s * 8, ((j / QN) - 1) & 1, 4 * lim)) {
                    failed = true;
                } else {
                    sts128(qitems0 + s * 16, info);
                    mbar_arrive(qfull0 + s * 8);
                }
            }
            failed = __any_sync(0xffffffffu, failed);
        };
        int raw = claim_issue();  // this CTA's second item
        // The unit range of this CTA's first item follows from the launch's totals (the host cuts the
        // same way, build_decode_plan), so the first copies leave without waiting for its record; the
        // record itself (first segment, part index) is fetched meanwhile for the other warps.
        int4 cur;
        {
            const long long rb = (long long)a.n_units * cta / a.n_ctas, re = (long long)a.n_units * (cta + 1) / a.n_ctas;
            const long long len = re - rb;
            cur = make_int4((int)rb, (int)(re - len * a.tail_pct / 100), 0, 0);
        }
        // the record and the first rows travel together; the other warps get the record the moment it is there
        const int4 rec0 = fetch(cta);
        int row_first = lane < cur.y - cur.x ? __ldcg(a.unit_row + cur.x + lane) : 0;
        publish(0, rec0);
        int4 nxt = make_int4(-1, -1, 0, 0);
        int j = 0, T = 0;  // items started, tile slots used (copies and the fillers between items)
#pragma unroll 1
        while (!failed) {
            const int ub = cur.x, ntl = cur.y - cur.x;
            bool to_publish = true;
            int row_next = j == 0 ? row_first : (lane < ntl ? __ldcg(a.unit_row + ub + lane) : 0);
#pragma unroll 1
            for (int base = 0; base < ntl && !failed; base += 32) {
                const int row = row_next;
                if (base + 32 + lane < ntl) row_next = __ldcg(a.unit_row + ub + base + 32 + lane);
                const int nb = min(32, ntl - base);
                const int Tl = T + base + lane;
                const int st = Tl % NS, rev = Tl / NS;
                for (int r = 0; (r << rshift) < nb; r++) {
                    if ((lane >> rshift) == r && lane < nb) {
                        if (Tl >= NS && !mbar_wait_bounded(empty0 + st * 8, (rev - 1) & 1, lim)) {
                            failed = true;
                        } else if (!(cta == 0 && Tl == a.fault_tile)) {
                            const int rec = row < 0 ? 0 : row;
                            if constexpr (Q8) {
                                mbar_expect_tx(full0 + st * 8, UNIT);  // one box of UNIT/128 rows x 128 bytes = one record
                                tma_load_2d(ring + st * UNIT, &tmap, 0, rec * (int)(UNIT / 128u), full0 + st * 8);
                            } else {
                                issue_tile<D>(&tmap, ring + st * UNIT, full0 + st * 8, rec * 32);
                            }
                        }
                    }
                    __syncwarp();
                    // The item after this one is published once the first round is out: that round only
                    // needs stages of earlier items, whereas later rounds may need this item's own tiles
                    // consumed, and its consumers may already be waiting for the queue entry.
                    if (to_publish) {
                        nxt = fetch(__shfl_sync(0xffffffffu, raw, 0));
                        publish(j + 1, nxt);
                        to_publish = false;
                    }
                }
                failed = __any_sync(0xffffffffu, failed) || vflag[1] != 0;
                if (j == 0 && base == 0 && lane == 0) CBKV_STAMP(2);
            }
            if (to_publish && !failed) {  // an item without tiles (the host never makes one)
                nxt = fetch(__shfl_sync(0xffffffffu, raw, 0));
                publish(j + 1, nxt);
            }
            T += ntl;
            if (nxt.x < 0 || failed) break;  // the end marker is already in the queue
            // Fillers: every item starts on a tile slot that is a multiple of C, so that a tile's consumer
            // warp depends on its place in the item only and results do not depend on which CTA ran which
            // item.  A filler slot carries no copy: its barrier is completed by a plain arrival.
            const int pad = (C - T % C) % C;
            if (pad) {
                const int Tl = T + lane;
                if (lane < pad) {
                    const int st = Tl % NS, rev = Tl / NS;
                    if (Tl >= NS && !mbar_wait_bounded(empty0 + st * 8, (rev - 1) & 1, lim)) failed = true;
                    else mbar_arrive(full0 + st * 8);
                }
                failed = __any_sync(0xffffffffu, failed);
                T += pad;
            }
            cur = nxt;
            j++;
            raw = claim_issue();
        }
        if (lane == 0) CBKV_STAMP(7);
        // Leave last: the stages of the final tiles are released by their consumers, which means the
        // copies have landed.  After a failure nobody may be consuming, so the copies themselves are awaited.
        {
            const int from = max(0, T - NS);
            bool bad = failed || vflag[1] != 0;
            for (int n = from + lane; n < T && !bad; n += 32)
                if (!mbar_wait_bounded(empty0 + (n % NS) * 8, (n / NS) & 1, 4 * lim)) bad = true;
            bad = __any_sync(0xffffffffu, bad) || vflag[1] != 0;
            if (bad) {
                if (lane == 0) { atomicOr(a.status, ST_WAIT_TIMEOUT); atomicExch(flag + 1, 1); }
                for (int n = from + lane; n < T; n += 32)
                    if (!(cta == 0 && n == a.fault_tile)) mbar_wait_bounded(full0 + (n % NS) * 8, (n / NS) & 1, 20000000ull);
            }
        }
        return;
    }

    // consumers and merger: read entry j of the item queue (false: no more items, or a wait ran out)
    bool failed = false;
    auto get_item = [&](int j, int4& out) -> bool {
        if (failed) return false;
        const int s = j & (QN - 1);
        if (!mbar_wait_bounded(qfull0 + s * 8, (j / QN) & 1, 4 * lim)) {
            failed = true;
            if (lane == 0) { atomicOr(a.status, ST_WAIT_TIMEOUT); atomicExch(flag + 1, 1); }
            return false;
        }
        out = lds128(qitems0 + s * 16);
        __syncwarp();
        if (lane == 0) mbar_arrive(qempty0 + s * 8);
        return out.x >= 0;
    };

    // the same without waiting: 1 = entry read (out valid, possibly the end marker), 0 = not published yet
    auto peek_item = [&](int j, int4& out) -> bool {
        const int s = j & (QN - 1);
        int ok = 0;
        if (lane == 0) ok = (int)mbar_test_wait(qfull0 + s * 8, (j / QN) & 1);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) return false;
        out = lds128(qitems0 + s * 16);
        __syncwarp();
        if (lane == 0) mbar_arrive(qempty0 + s * 8);
        return true;
    };

    const int n_rep = a.geo.n_rep;
    if (warp == C + 1) {
        // -------------------------------------------------------------- merger
        // Combines the consumers' states of each piece, writes the output (or a partial
        // plus a ticket; the last ticket holder merges the segment's partials), and hands
        // the buffer back.  The consumers never wait on global memory.
        pdl_wait();  // out and the scratch are shared with earlier launches
        if (cta == 0 && lane == 0) a.work_counters[(a.work_slot + 2) & 3] = 0;  // for the launch after the next one
        // Only now may the next launch start: at most two launches are alive at a time, which is
        // what lets four claim counters rotate.
        pdl_launch_dependents();
        int k = 0, kk = 0, n_deferred = 0;
        // The ticket of a cut piece is drawn right after its partial is stored but looked at one piece
        // later, so the counter's round trip overlaps the wait for the next piece.  A segment whose
        // last ticket this CTA drew is merged at the end of the CTA by all its warps (the consumers
        // are idle by then); only when the list is full does this warp merge alone.
        int pend_seg = -1, pend_np = 0, pend_raw = 0;
        auto settle = [&]() {
            if (pend_seg < 0) return;
            int last = 0;
            if (lane == 0 && pend_raw == pend_np - 1) {
                last = 1;
                a.seg_counter[pend_seg] = 0;  // ready for the next launch
            }
            last = __shfl_sync(0xffffffffu, last, 0);
            if (last) {
                if (n_deferred < DEFER_CAP) {
                    if (lane == 0) flag[4 + n_deferred] = pend_seg;
                    n_deferred++;
                } else {
                    const int4* sp = reinterpret_cast<const int4*>(a.segs + pend_seg);
                    const int4 x = __ldg(sp), y = __ldg(sp + 1);
                    uint16_t* orow = reinterpret_cast<uint16_t*>(a.out) + ((size_t)x.w * a.geo.n_q + (size_t)(pend_seg % Hkv) * n_rep) * D;
                    merge_parts<D, BF16>(a, y.y, y.x, orow, n_rep, lane, 32);
                }
            }
            pend_seg = -1;
        };
#ifdef CBKV_MEASURE
        int dbg_tiles = 0, dbg_cut = 0;
#endif
        int4 it;
        bool have = get_item(0, it);
#pragma unroll 1
        while (have) {
            int seg = it.z, pb = it.x;
#pragma unroll 1
            while (pb < it.y) {
                const int4* sp = reinterpret_cast<const int4*>(a.segs + seg);
                const int4 x = __ldg(sp), y = __ldg(sp + 1), z = __ldg(sp + 2);
                const int pe = min(it.y, z.x);
                const int h = seg % Hkv;
                const int tok_off = x.w, nparts = y.x;
                const int slot = nparts > 1 ? y.y + (seg == it.z ? it.w : 0) : 0;
                const int buf = NB == 2 ? (kk & 1) : 0, use = NB == 2 ? (kk >> 1) : kk;
                if (!mbar_wait_bounded(cfull0 + buf * 8, use & 1, 4 * lim)) {
                    failed = true;
                    if (lane == 0) { atomicOr(a.status, ST_WAIT_TIMEOUT); atomicExch(flag + 1, 1); }
                    break;
                }
                if (lane == 0) CBKV_STAMP(5);
                const float* co = comb_o + (size_t)buf * C * ccols * DP;
                const float* cml = comb_ml + buf * C * 16;
                uint16_t* out_row = reinterpret_cast<uint16_t*>(a.out) + ((size_t)tok_off * a.geo.n_q + (size_t)h * n_rep) * D;
                // lane owns 4 consecutive d-values (per pass of 128) of every query column
                constexpr int PASSES = (D + 127) / 128;
#pragma unroll
                for (int ps = 0; ps < PASSES; ps++) {
                    const int j4 = ps * 32 + lane;  // float4 index within a row of D
                    if (j4 * 4 < D) {
#pragma unroll
                        for (int col = 0; col < 8; col++) {
                            if (col < n_rep) {
                                float M = -INFINITY;
#pragma unroll
                                for (int ww = 0; ww < C; ww++) M = fmaxf(M, cml[(ww * 8 + col) * 2]);
                                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                                float ls = 0.f;
#pragma unroll
                                for (int ww = 0; ww < C; ww++) {
                                    const float mw = cml[(ww * 8 + col) * 2];
                                    const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
                                    const float4 v = *reinterpret_cast<const float4*>(co + ((size_t)ww * ccols + col) * DP + j4 * 4);
                                    acc.x += f * v.x; acc.y += f * v.y; acc.z += f * v.z; acc.w += f * v.w;
                                    ls += f * cml[(ww * 8 + col) * 2 + 1];
                                }
                                if (nparts == 1) {
                                    const float inv = 1.f / ls;
                                    uint2 pk;
                                    pk.x = pack2<BF16>(acc.x * inv, acc.y * inv);
                                    pk.y = pack2<BF16>(acc.z * inv, acc.w * inv);
                                    *reinterpret_cast<uint2*>(out_row + col * D + j4 * 4) = pk;
                                } else {
                                    *reinterpret_cast<float4*>(a.part_o + ((size_t)slot * 8 + col) * D + j4 * 4) = acc;
                                    if (j4 == 0) *reinterpret_cast<float2*>(a.part_ml + ((size_t)slot * 8 + col) * 2) = make_float2(M, ls);
                                }
                            }
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(cempty0 + buf * 8);  // the consumers may store the next piece here
                settle();  // the previous cut piece's ticket has had a whole piece to come back
                if (nparts > 1) {
                    if (lane == 0) {
                        // release: the warp's partial (ordered before by __syncwarp) is visible before the ticket;
                        // acquire: whoever draws the last ticket sees every other part's partial
                        asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(pend_raw) : "l"(a.seg_counter + seg) : "memory");
                    }
                    pend_seg = seg;
                    pend_np = nparts;
#ifdef CBKV_MEASURE
                    dbg_cut++;
#endif
                }
#ifdef CBKV_MEASURE
                dbg_tiles += pe - pb;
#endif
                kk++;
                seg++;
                pb = pe;
            }
            if (failed) break;
            k++;
            have = get_item(k, it);
        }
        settle();
        // hand the segments to merge to the whole CTA
        if (lane == 0) flag[2] = n_deferred;
        __syncwarp();
        consumer_sync((C + 1) * 32);
        for (int i = 0; i < n_deferred; i++) {
            const int sg = flag[4 + i];
            const int4* sp = reinterpret_cast<const int4*>(a.segs + sg);
            const int4 x = __ldg(sp), y = __ldg(sp + 1);
            uint16_t* out_row = reinterpret_cast<uint16_t*>(a.out) + ((size_t)x.w * a.geo.n_q + (size_t)(sg % Hkv) * n_rep) * D;
            merge_parts<D, BF16>(a, y.y, y.x, out_row, n_rep, C * 32 + lane, (C + 1) * 32);
        }
#ifdef CBKV_MEASURE
        if (lane == 0) {
            CBKV_STAMP(6);
            if ((a.debug & 4) && a.dbg_buf) {
                unsigned smid;
                asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
                a.dbg_buf[(size_t)blockIdx.x * 16 + 8] = (unsigned long long)kk;
                a.dbg_buf[(size_t)blockIdx.x * 16 + 9] = (unsigned long long)n_deferred;
                a.dbg_buf[(size_t)blockIdx.x * 16 + 10] = (unsigned long long)dbg_cut;
                a.dbg_buf[(size_t)blockIdx.x * 16 + 11] = (unsigned long long)smid;
                a.dbg_buf[(size_t)blockIdx.x * 16 + 12] = (unsigned long long)dbg_tiles;
                a.dbg_buf[(size_t)blockIdx.x * 16 + 13] = (unsigned long long)k;
            }
        }
#endif
        return;
    }

    // ---------------------------------------------------------------- consumers
    const int cw = warp - 1, g = lane >> 2, t = lane & 3;
    int4 it;
    bool have = get_item(0, it);  // plan and block tables were uploaded by a copy: always visible
    int seg = have ? it.z : 0, pb = have ? it.x : 0;
    Piece cur = load_piece(a, seg);
    if (have && g < a.geo.n_rep && t < (D * 2 + 127) / 128) {
        // ask for the first piece's q rows in L2 while the previous launch is still finishing (a request, not a
        // read: L2 is where that launch or a copy engine writes them, so nothing stale can be seen later)
        const char* qp = reinterpret_cast<const char*>(a.q) + ((size_t)cur.tok_off * a.geo.n_q + (size_t)cur.h * a.geo.n_rep + g) * D * 2 + t * 128;
        asm volatile("prefetch.global.L2 [%0];" ::"l"(qp));
    }
    pdl_wait();  // q, k_new and v_new come from earlier work in the stream
    if (a.in_flag != nullptr) {
        // ... or from copies on another stream, which end by writing this launch's number behind the data:
        // one lane looks until it is there (bounded like every wait; a copy engine makes progress whatever
        // this kernel does), the warp meets, and only then are the inputs read
        if (lane == 0) {
            const uint64_t t0 = global_ns(), lim = (uint64_t)a.wait_us * 1000ull;
            uint32_t seen;
            for (;;) {
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(a.in_flag) : "memory");
                if ((int32_t)(seen - a.in_seq) >= 0) break;
                if (global_ns() - t0 > lim) { atomicOr(a.status, ST_WAIT_TIMEOUT); break; }
            }
        }
        __syncwarp();
    }
    uint32_t qf[1][D / 16][2];
    if constexpr (Q8) load_q_frags_q8<D>(a, cur, g, t, qf);
    else load_q_frags<D>(a, cur, g, t, qf);
    if (tid == 32) CBKV_STAMP(3);
    int k = 0, kk = 0, nbase = 0;  // items read, pieces handed over, tiles of the CTA before the current item
#ifdef CBKV_MEASURE
    bool first_tile = true;
#endif
#pragma unroll 1
    while (have) {
        const int pe = min(it.y, cur.se);
        const bool more = pe < it.y;
        // what comes next (the item's next segment, or the first piece of the next item): its
        // metadata and queries arrive while this piece is processed
        int4 nit = it;
        bool nhave = true, nknown = true;
        int nseg = seg + 1;
        if (!more) {
            // The next item's queue entry is looked at without waiting: the producer runs a ring ahead, so
            // it is nearly always there; if not, it is waited for after this piece's tiles (a consumer
            // never waits for the queue while tiles it has to consume are outstanding).
            nknown = !failed && peek_item(k + 1, nit);
            nhave = nknown && nit.x >= 0;
            nseg = nit.z;
        }
        Piece nxt = cur;
        uint32_t qf_next[1][D / 16][2];
        if (nknown && nhave) {
            nxt = load_piece(a, nseg);
            if constexpr (Q8) load_q_frags_q8<D>(a, nxt, g, t, qf_next);
            else load_q_frags<D>(a, nxt, g, t, qf_next);
        }
        float o[1][D / 16][4], m[1][2] = {{-INFINITY, -INFINITY}}, l[1][2] = {{0.f, 0.f}};
#pragma unroll
        for (int mt = 0; mt < D / 16; mt++) { o[0][mt][0] = o[0][mt][1] = o[0][mt][2] = o[0][mt][3] = 0.f; }
        const int qpos[1][2] = {{cur.q_pos, cur.q_pos}};

        const int n0 = nbase + (pb - it.x);  // the piece's first tile, counted over the CTA's items
        const int n1 = n0 + (pe - pb);
        int T = n0 + (cw - n0 % C + C) % C;  // this warp's first tile of the piece
        // stage and revolution parity of this warp's tiles, advanced by C per tile (NS is a multiple of C)
        int st = T % NS, par = (T / NS) & 1;
#pragma unroll 1
        for (; T < n1; T += C, st += C) {
            if (st >= NS) { st -= NS; par ^= 1; }
            const uint32_t stage = ring + st * UNIT;
            const int u = pb + (T - n0);
            if (!failed && !mbar_wait_bounded(full0 + st * 8, par, lim)) {
                failed = true;
                if (lane == 0) { atomicOr(a.status, ST_WAIT_TIMEOUT); atomicExch(flag + 1, 1); }
            }
            // After a failure nothing is released any more: a stage given back before its copy has landed
            // would be armed a second time.  The producer then finds its own wait running out and stops.
            if (failed) break;
#ifdef CBKV_MEASURE
            if (first_tile && tid == 32) { CBKV_STAMP(4); first_tile = false; }
#endif
            const int lp = cur.page_lo + (u - cur.sb);
            if (!CBKV_DBG(1)) {
                if (!Q8 && a.k_new != nullptr && lp == cur.page_last) {
                    // fused append: put the new K/V row into the tile just fetched and into its page
                    const int slot = cur.q_pos & 15;
                    const int rec = __ldcg(a.unit_row + u);
                    for (int c = lane; c < 2 * (D / 8); c += 32) {
                        int kv = c / (D / 8), j = c - kv * (D / 8);
                        const uint4 val = *(reinterpret_cast<const uint4*>(kv ? a.v_new : a.k_new) +
                                            ((size_t)cur.tok_off * Hkv + cur.h) * (D / 8) + j);
                        uint32_t row = page_row(kv, slot, 16, true);
                        uint32_t addr = stage + (j >> 3) * 4096u + swz(row, j & 7);
                        asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(val.x), "r"(val.y), "r"(val.z), "r"(val.w) : "memory");
                        if (rec >= 0) {
                            size_t drow = (size_t)rec * 32 + row;
                            reinterpret_cast<uint4*>(a.arena)[drow * (D / 8) + j] = val;
                        }
                    }
                    fence_proxy_async();
                    __syncwarp();
                }
                const bool need_mask = (lp * 16 + 15 > cur.q_pos) || (a.window > 0 && lp * 16 + a.window <= cur.q_pos);
                if constexpr (Q8) {
                    if (a.k_new != nullptr && lp == cur.page_last) {
                        // fused append: quantise the new K/V row into the tile just fetched and into its record
                        const int rec = __ldcg(a.unit_row + u);
                        if (rec >= 0) {
                            const size_t rowi = ((size_t)cur.tok_off * Hkv + cur.h) * D;
                            q8_append_row<D, BF16>(stage, reinterpret_cast<uint8_t*>(a.arena) + (size_t)rec * UNIT,
                                                   reinterpret_cast<const uint16_t*>(a.k_new) + rowi,
                                                   reinterpret_cast<const uint16_t*>(a.v_new) + rowi, cur.q_pos & 15, lane);
                        }
                        fence_proxy_async();  // the stage is refilled by the copy engine later
                        __syncwarp();
                    }
                    Q8Tile<D> regs;
                    q8_load<D>(stage, lane, regs);
                    __syncwarp();
                    if (lane == 0) mbar_arrive(empty0 + st * 8);  // the tile is in registers: the stage may be refilled
#ifdef CBKV_MEASURE
                    q8_attend<D, BF16>(regs, qf, o, m, l, lp * 16, qpos, a.window, a.scale_log2, need_mask, lane, a.debug);
#else
                    q8_attend<D, BF16>(regs, qf, o, m, l, lp * 16, qpos, a.window, a.scale_log2, need_mask, lane);
#endif
                    continue;
                }
                attend_tile<D, 1, BF16>(stage, qf, o, m, l, lp * 16, qpos, a.window, a.scale_log2, need_mask, lane);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty0 + st * 8);  // the stage may be refilled
        }

        // ---- hand this warp's state for the piece to the merger (double-buffered)
        const int buf = NB == 2 ? (kk & 1) : 0, use = NB == 2 ? (kk >> 1) : kk;
        if (vflag[1] != 0) failed = true;  // another warp gave up: stop waiting
        if (use >= 1 && !failed && !mbar_wait_bounded(cempty0 + buf * 8, (use - 1) & 1, 4 * lim)) {
            failed = true;
            if (lane == 0) { atomicOr(a.status, ST_WAIT_TIMEOUT); atomicExch(flag + 1, 1); }
        }
#pragma unroll
        for (int j = 0; j < 2; j++) {
            l[0][j] += __shfl_xor_sync(0xffffffffu, l[0][j], 4);
            l[0][j] += __shfl_xor_sync(0xffffffffu, l[0][j], 8);
            l[0][j] += __shfl_xor_sync(0xffffffffu, l[0][j], 16);
        }
        float* co = comb_o + ((size_t)buf * C + cw) * ccols * DP;
        float* cml = comb_ml + (buf * C + cw) * 16;
#pragma unroll
        for (int mt = 0; mt < D / 16; mt++) {
            // the d-values behind rows g and g+8 of m-tile mt (permuted for quantised tiles, see q8_attend)
            const int d0 = Q8 ? 32 * (mt >> 1) + 4 * g + 2 * (mt & 1) : mt * 16 + g;
            const int d1 = Q8 ? d0 + 1 : d0 + 8;
            if (2 * t < ccols) {
                co[(2 * t) * DP + d0] = o[0][mt][0];
                co[(2 * t) * DP + d1] = o[0][mt][2];
            }
            if (2 * t + 1 < ccols) {
                co[(2 * t + 1) * DP + d0] = o[0][mt][1];
                co[(2 * t + 1) * DP + d1] = o[0][mt][3];
            }
        }
        if (g == 0) {
            cml[(2 * t) * 2 + 0] = m[0][0]; cml[(2 * t) * 2 + 1] = l[0][0];
            cml[(2 * t + 1) * 2 + 0] = m[0][1]; cml[(2 * t + 1) * 2 + 1] = l[0][1];
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(cfull0 + buf * 8);
        kk++;
        if (!nknown) {  // the entry was not there when the piece began: wait for it now
            nhave = get_item(k + 1, nit);
            if (nhave) {
                nseg = nit.z;
                nxt = load_piece(a, nseg);
                if constexpr (Q8) load_q_frags_q8<D>(a, nxt, g, t, qf_next);
                else load_q_frags<D>(a, nxt, g, t, qf_next);
            }
        }
        if (!nhave) break;
        if (more) {
            pb = pe;
        } else {
            // the filler slots up to the next multiple of C (see the producer): this warp owns at most one
            const int n_pad = (n1 + C - 1) / C * C;
            const int Tp = n1 + (cw - n1 % C + C) % C;
            if (Tp < n_pad) {
                const int fs = Tp % NS;
                if (!failed && !mbar_wait_bounded(full0 + fs * 8, (Tp / NS) & 1, lim)) {
                    failed = true;
                    if (lane == 0) { atomicOr(a.status, ST_WAIT_TIMEOUT); atomicExch(flag + 1, 1); }
                }
                __syncwarp();
                if (lane == 0 && !failed) mbar_arrive(empty0 + fs * 8);
            }
            nbase = n_pad;
            k++;
            it = nit;
            pb = it.x;
        }
        seg = nseg;
        cur = nxt;
#pragma unroll
        for (int ks = 0; ks < D / 16; ks++) { qf[0][ks][0] = qf_next[0][ks][0]; qf[0][ks][1] = qf_next[0][ks][1]; }
    }
    // idle now: help merge the segments whose last ticket this CTA drew
    consumer_sync((C + 1) * 32);
    const int n_deferred = flag[2];
    for (int i = 0; i < n_deferred; i++) {
        const int sg = flag[4 + i];
        const int4* sp = reinterpret_cast<const int4*>(a.segs + sg);
        const int4 x = __ldg(sp), y = __ldg(sp + 1);
        uint16_t* out_row = reinterpret_cast<uint16_t*>(a.out) + ((size_t)x.w * a.geo.n_q + (size_t)(sg % Hkv) * n_rep) * D;
        merge_parts<D, BF16>(a, y.y, y.x, out_row, n_rep, cw * 32 + lane, (C + 1) * 32);
    }
}

// ------------------------------------------------------------------ chunk (prefill)
// One warp per item = (sequence, kv head, block of 8*NT query columns); column c of a
// sequence is (new token c / n_rep, q head c % n_rep of the kv group).  Every warp
// streams the pages its columns can see through its own TMA ring.
template <int D, int NT, int W, int S, bool BF16>
__global__ void __launch_bounds__(W * 32) chunk_kernel(const __grid_constant__ CUtensorMap tmap, const ChunkArgs a) {
    constexpr uint32_t UNIT = 32u * D * 2u;
    constexpr int CPI = 8 * NT;
    extern __shared__ __align__(1024) uint8_t smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)W * S * UNIT);
    const int tid = threadIdx.x, w = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    if ((smem_u32(smem) & 1023u) != 0) {
        if (tid == 0) atomicOr(a.status, ST_SMEM_ALIGN);
        return;
    }
    const int item = blockIdx.x * W + w;
    if (item >= a.n_items) return;
    const uint32_t ring = smem_u32(smem) + (uint32_t)w * S * UNIT;
    const uint32_t bar0 = smem_u32(bars + w * S);
    if (lane == 0) {
#pragma unroll
        for (int i = 0; i < S; i++) mbar_init(bar0 + i * 8, 1);
        fence_mbar_init();
        fence_proxy_async();
    }
    __syncwarp();

    int lo = 0, hi = a.step.n_seqs - 1;  // last sequence whose first item is <= item
    while (lo < hi) {
        int mid = (lo + hi + 1) >> 1;
        if (a.item_begin[mid] <= item) lo = mid; else hi = mid - 1;
    }
    const int b = lo;
    const SeqMeta sm = a.step.seq_meta[b];
    const int Hkv = a.geo.n_kv, n_rep = a.geo.n_rep;
    const int ncols = sm.snew * n_rep;
    const int ncb = (ncols + CPI - 1) / CPI;
    const int local = item - a.item_begin[b];
    const int h = local / ncb, cb = local - h * ncb;
    const int c_lo = cb * CPI, c_hi = min(c_lo + CPI, ncols) - 1;
    const int q_min = sm.pos + c_lo / n_rep, q_max = sm.pos + c_hi / n_rep;
    const int lo_key = a.window > 0 ? max(0, q_min - a.window + 1) : 0;
    const int p_lo = lo_key >> 4, p_hi = q_max >> 4;
    const size_t blk = (size_t)sm.tok_off * a.geo.n_q;  // first packed q row of this sequence

    uint32_t qf[NT][D / 16][2];
    int qpos[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
        int c = c_lo + nt * 8 + g;  // the column this lane feeds into the B operand
        bool ok = c < ncols;
        int r = ok ? c / n_rep : 0, rep = ok ? c - r * n_rep : 0;
        const uint32_t* qrow = reinterpret_cast<const uint32_t*>(
            reinterpret_cast<const uint16_t*>(a.q) + (blk + (size_t)(h * n_rep + rep) * sm.snew + r) * D);
#pragma unroll
        for (int ks = 0; ks < D / 16; ks++) {
            qf[nt][ks][0] = ok ? __ldg(qrow + ks * 8 + t) : 0u;
            qf[nt][ks][1] = ok ? __ldg(qrow + ks * 8 + 4 + t) : 0u;
        }
#pragma unroll
        for (int j = 0; j < 2; j++) {
            int cc = min(c_lo + nt * 8 + 2 * t + j, ncols - 1);  // columns past the end mimic the last one
            qpos[nt][j] = sm.pos + cc / n_rep;
        }
    }
    float o[NT][D / 16][4], m[NT][2], l[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
        m[nt][0] = m[nt][1] = -INFINITY; l[nt][0] = l[nt][1] = 0.f;
#pragma unroll
        for (int mt = 0; mt < D / 16; mt++) { o[nt][mt][0] = o[nt][mt][1] = o[nt][mt][2] = o[nt][mt][3] = 0.f; }
    }

    auto issue = [&](int lp, int stage_idx) {
        if (lane == 0) {
            int phys = a.step.tables[sm.tbl_off + lp];
            if (phys < 0 || phys >= a.geo.num_pages) { atomicOr(a.status, ST_BAD_PAGE); phys = 0; }
            issue_tile<D>(&tmap, ring + stage_idx * UNIT, bar0 + stage_idx * 8, (phys * Hkv + h) * 32);
        }
    };
    int next = p_lo;
#pragma unroll 1
    for (int i = 0; i < S && next <= p_hi; i++, next++) issue(next, i);
    bool failed = false;
    int consumed = 0, issued = next - p_lo, fail_at = 0;
#pragma unroll 1
    for (int lp = p_lo; lp <= p_hi; lp++) {
        const int st = consumed % S;
        if (!failed && !mbar_wait_bounded(bar0 + st * 8, (consumed / S) & 1)) {
            failed = true;
            fail_at = consumed;
            atomicOr(a.status, ST_WAIT_TIMEOUT);
        }
        if (!failed) {
            const bool need_mask = (lp * 16 + 15 > q_min) || (a.window > 0 && lp * 16 + a.window <= q_max);
            attend_tile<D, NT, BF16>(ring + st * UNIT, qf, o, m, l, lp * 16, qpos, a.window, a.scale_log2, need_mask, lane);
        }
        __syncwarp();
        consumed++;
        if (next <= p_hi) { if (!failed) { issue(next, st); issued++; } next++; }
    }
    if (failed) {  // wait (bounded) for the copies still in flight, then leave without storing
        for (int i = fail_at; i < issued; i++) mbar_wait_bounded(bar0 + (i % S) * 8, (i / S) & 1, 20000000ull);
        return;
    }

#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
#pragma unroll
        for (int j = 0; j < 2; j++) {
            float ls = l[nt][j];
            ls += __shfl_xor_sync(0xffffffffu, ls, 4);
            ls += __shfl_xor_sync(0xffffffffu, ls, 8);
            ls += __shfl_xor_sync(0xffffffffu, ls, 16);
            int c = c_lo + nt * 8 + 2 * t + j;
            if (c < ncols) {
                int r = c / n_rep, rep = c - r * n_rep;
                uint16_t* orow = reinterpret_cast<uint16_t*>(a.out) + (blk + (size_t)(h * n_rep + rep) * sm.snew + r) * D;
                float inv = 1.f / ls;
#pragma unroll
                for (int mt = 0; mt < D / 16; mt++) {
                    orow[mt * 16 + g] = to_elem<BF16>(o[nt][mt][j] * inv);
                    orow[mt * 16 + g + 8] = to_elem<BF16>(o[nt][mt][j + 2] * inv);
                }
            }
        }
    }
}

// ------------------------------------------------------------------ generic
// Any page size and head_dim (multiple of 8, <= 512); one warp per query row.
template <bool BF16>
__global__ void generic_kernel(const GenericArgs a) {
    __shared__ float qs[4][512];
    const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t rid = (int64_t)blockIdx.x * 4 + w;  // packed q row: sequence blocks of [n_q][snew]
    if (rid >= (int64_t)a.step.n_tokens * a.geo.n_q) return;
    const int D = a.geo.d, P = a.geo.page_size, Hkv = a.geo.n_kv;
    int lo = 0, hi = a.step.n_seqs - 1;
    while (lo < hi) {
        int mid = (lo + hi + 1) >> 1;
        if ((int64_t)a.step.seq_meta[mid].tok_off * a.geo.n_q <= rid) lo = mid; else hi = mid - 1;
    }
    const SeqMeta sm = a.step.seq_meta[lo];
    const int64_t local = rid - (int64_t)sm.tok_off * a.geo.n_q;
    const int hq = (int)(local / sm.snew), r = (int)(local % sm.snew);
    const int h = hq / a.geo.n_rep;  // repeat_kv: q head i reads kv head i / n_rep, kv.rs:177-187
    const int q_pos = sm.pos + r;
    const uint16_t* q = reinterpret_cast<const uint16_t*>(a.q) + rid * D;
    for (int j = lane; j < D; j += 32) qs[w][j] = from_elem<BF16>(q[j]);
    __syncwarp();
    const uint16_t* arena = reinterpret_cast<const uint16_t*>(a.arena);
    const int t_lo = a.window > 0 ? max(0, q_pos - a.window + 1) : 0;
    float m = -INFINITY, l = 0.f, acc[16];
#pragma unroll
    for (int i = 0; i < 16; i++) acc[i] = 0.f;
    for (int t0 = t_lo; t0 <= q_pos; t0 += 32) {
        const int tk = t0 + lane;
        const bool ok = tk <= q_pos;
        float s = -INFINITY;
        if (ok) {
            int phys = a.step.tables[sm.tbl_off + tk / P];
            if (phys < 0 || phys >= a.geo.num_pages) { atomicOr(a.status, ST_BAD_PAGE); phys = 0; }
            const uint16_t* krow = arena + ((((int64_t)phys * Hkv + h) * 2 + 0) * P + tk % P) * D;
            float d = 0.f;
            for (int j = 0; j < D; j++) d += qs[w][j] * from_elem<BF16>(krow[j]);
            s = d * a.scale;
        }
        float mx = s;
        for (int off = 16; off; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
        const float m_new = fmaxf(m, mx);
        const float alpha = __expf(m - m_new);
        const float p = ok ? __expf(s - m_new) : 0.f;
        float ps = p;
        for (int off = 16; off; off >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, off);
        l = l * alpha + ps;
        m = m_new;
#pragma unroll
        for (int i = 0; i < 16; i++) acc[i] *= alpha;
        const int cnt = min(32, q_pos - t0 + 1);
        for (int kk = 0; kk < cnt; kk++) {
            const float pk = __shfl_sync(0xffffffffu, p, kk);
            const int tv = t0 + kk;
            int phys = a.step.tables[sm.tbl_off + tv / P];
            if (phys < 0 || phys >= a.geo.num_pages) phys = 0;
            const uint16_t* vrow = arena + ((((int64_t)phys * Hkv + h) * 2 + 1) * P + tv % P) * D;
#pragma unroll
            for (int i = 0; i < 16; i++) {
                int j = lane + 32 * i;
                if (j < D) acc[i] += pk * from_elem<BF16>(vrow[j]);
            }
        }
    }
    uint16_t* orow = reinterpret_cast<uint16_t*>(a.out) + rid * D;
#pragma unroll
    for (int i = 0; i < 16; i++) {
        int j = lane + 32 * i;
        if (j < D) orow[j] = to_elem<BF16>(acc[i] / l);
    }
}

// ------------------------------------------------------------------ launchers
// default consumer warps per CTA and CTAs per SM of the decode kernel
template <int D> struct DecodeCfg;
template <> struct DecodeCfg<64>  { static constexpr int C = 6, CTAS = 1; };
template <> struct DecodeCfg<128> { static constexpr int C = 6, CTAS = 1; };
template <> struct DecodeCfg<256> { static constexpr int C = 6, CTAS = 1; };

static int decode_smem_bytes(int d, int consumers, int stages, int comb_cols, int comb_bufs, bool q8 = false) {
    const int unit = q8 ? (int)qrec_bytes(16, d) : 32 * d * 2;
    return stages * unit + comb_bufs * (consumers * comb_cols * (d + 4) * 4 + consumers * 16 * 4) + QN * 16 +
           (2 * stages + 4 + 2 * QN) * 8 + (4 + DEFER_CAP) * 4;
}

template <int D> struct ChunkCfg;
template <> struct ChunkCfg<64>  { static constexpr int W = 4, S = 4, NT = 4; };
template <> struct ChunkCfg<128> { static constexpr int W = 4, S = 3, NT = 2; };
template <> struct ChunkCfg<256> { static constexpr int W = 4, S = 2, NT = 1; };

template <int D> constexpr int chunk_smem() { return ChunkCfg<D>::W * ChunkCfg<D>::S * 32 * D * 2 + ChunkCfg<D>::W * ChunkCfg<D>::S * 8; }

// Stage count: the largest multiple of the consumer count that fits next to the merge
// buffers when `ctas_per_sm` CTAs share the SM's shared memory (1 KB per CTA is
// reserved by the system), at most 8 stages per consumer.  Bytes in flight matter
// more than a second merge buffer: the merge area is double-buffered only when that
// costs no stage.
DecodeConfig decode_config(int d, int n_rep, int ctas_per_sm, int stages, int consumers, bool q8) {
    int c, ctas;
    switch (d) {
        case 64: c = DecodeCfg<64>::C; ctas = DecodeCfg<64>::CTAS; break;
        case 128: c = DecodeCfg<128>::C; ctas = DecodeCfg<128>::CTAS; break;
        case 256: c = DecodeCfg<256>::C; ctas = DecodeCfg<256>::CTAS; break;
        default: return {0, 0, 0, 0, 0, 0};
    }
    // int8 tiles are bound by the consumer warps' arithmetic, not by bytes in flight: two CTAs of four consumer
    // warps per SM (each with its own ring, producer and merger) let one CTA's set-up and merge run under the
    // other's tiles; measured 0.80 ms per cfg2 step against 0.85 with one CTA of eight
    if (q8 && d <= 128) { c = 4; ctas = 2; }
    if (consumers == 4 || consumers == 6 || consumers == 8 || (consumers == 12 && d <= 128)) c = consumers;  // 12 warps of head_dim 256 spill
    if (ctas_per_sm > 0) ctas = ctas_per_sm;
    const int comb_cols = std::min(8, (n_rep + 1) & ~1);
    const int smem_limit = std::min(227 * 1024, (228 * 1024) / ctas - 1024);
    if (stages <= 0) {
        stages = 8 * c;
        while (stages > c && decode_smem_bytes(d, c, stages, comb_cols, 1, q8) > smem_limit) stages -= c;
    }
    stages = std::max(c, (stages / c) * c);
    const int bufs = decode_smem_bytes(d, c, stages, comb_cols, 2, q8) <= smem_limit ? 2 : 1;
    return {c, stages, decode_smem_bytes(d, c, stages, comb_cols, bufs, q8), ctas, comb_cols, bufs};
}
ChunkConfig chunk_config(int d) {
    switch (d) {
        case 64: return {ChunkCfg<64>::W, ChunkCfg<64>::S, chunk_smem<64>(), 8 * ChunkCfg<64>::NT};
        case 128: return {ChunkCfg<128>::W, ChunkCfg<128>::S, chunk_smem<128>(), 8 * ChunkCfg<128>::NT};
        case 256: return {ChunkCfg<256>::W, ChunkCfg<256>::S, chunk_smem<256>(), 8 * ChunkCfg<256>::NT};
        default: return {0, 0, 0, 0};
    }
}

template <int D, bool BF16> static cudaError_t set_attrs() {
    cudaError_t e;
    e = cudaFuncSetAttribute(decode_kernel<D, 4, BF16, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(decode_kernel<D, 6, BF16, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(decode_kernel<D, 8, BF16, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(decode_kernel<D, 4, BF16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(decode_kernel<D, 6, BF16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(decode_kernel<D, 8, BF16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(decode_kernel<D, 12, BF16, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(decode_kernel<D, 12, BF16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(chunk_kernel<D, ChunkCfg<D>::NT, ChunkCfg<D>::W, ChunkCfg<D>::S, BF16>,
                                cudaFuncAttributeMaxDynamicSharedMemorySize, chunk_smem<D>());
}

cudaError_t kernels_init() {
    cudaError_t e;
    if ((e = set_attrs<64, false>()) != cudaSuccess) return e;
    if ((e = set_attrs<64, true>()) != cudaSuccess) return e;
    if ((e = set_attrs<128, false>()) != cudaSuccess) return e;
    if ((e = set_attrs<128, true>()) != cudaSuccess) return e;
    if ((e = set_attrs<256, false>()) != cudaSuccess) return e;
    if ((e = set_attrs<256, true>()) != cudaSuccess) return e;
    return cudaSuccess;
}

cudaError_t launch_append(const AppendArgs& a, bool bf16, cudaStream_t st) {
    (void)bf16;  // a bit copy: the element type does not matter
    int64_t total = (int64_t)a.step.n_tokens * a.geo.n_kv * 2 * (a.geo.d / 8);
    int blocks = (int)std::min<int64_t>((total + 255) / 256, 148 * 8);
    if (blocks <= 0) return cudaSuccess;
    append_kernel<uint16_t><<<blocks, 256, 0, st>>>(a);
    return cudaGetLastError();
}

template <int D, int C, bool BF16, bool Q8>
static cudaError_t launch_decode_t(const CUtensorMap& map, const DecodeArgs& a, int n_ctas, int smem, bool pdl, cudaStream_t st) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)n_ctas);
    cfg.blockDim = dim3((C + 2) * 32);
    cfg.dynamicSmemBytes = (size_t)smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, decode_kernel<D, C, BF16, Q8>, map, a);
}

template <int D, bool BF16, bool Q8>
static cudaError_t launch_decode_c(const CUtensorMap& map, const DecodeArgs& a, int n_ctas, int consumers, int smem, bool pdl, cudaStream_t st) {
    switch (consumers) {
        case 4: return launch_decode_t<D, 4, BF16, Q8>(map, a, n_ctas, smem, pdl, st);
        case 6: return launch_decode_t<D, 6, BF16, Q8>(map, a, n_ctas, smem, pdl, st);
        case 8: return launch_decode_t<D, 8, BF16, Q8>(map, a, n_ctas, smem, pdl, st);
        case 12: return launch_decode_t<D, 12, BF16, Q8>(map, a, n_ctas, smem, pdl, st);
        default: return cudaErrorInvalidValue;
    }
}
template <int D>
static cudaError_t launch_decode_d(const CUtensorMap& map, const DecodeArgs& a, int n_ctas, int consumers, int smem, bool pdl, bool bf16, bool q8, cudaStream_t st) {
    if (q8) return bf16 ? launch_decode_c<D, true, true>(map, a, n_ctas, consumers, smem, pdl, st) : launch_decode_c<D, false, true>(map, a, n_ctas, consumers, smem, pdl, st);
    return bf16 ? launch_decode_c<D, true, false>(map, a, n_ctas, consumers, smem, pdl, st) : launch_decode_c<D, false, false>(map, a, n_ctas, consumers, smem, pdl, st);
}

cudaError_t launch_decode(const CUtensorMap& map, const DecodeArgs& a, int n_ctas, int consumers, int smem, bool pdl, bool bf16, cudaStream_t st, bool q8) {
    if (a.n_stages < consumers || a.n_stages % consumers != 0) return cudaErrorInvalidValue;
    switch (a.geo.d) {
        case 64: return launch_decode_d<64>(map, a, n_ctas, consumers, smem, pdl, bf16, q8, st);
        case 128: return launch_decode_d<128>(map, a, n_ctas, consumers, smem, pdl, bf16, q8, st);
        case 256: return launch_decode_d<256>(map, a, n_ctas, consumers, smem, pdl, bf16, q8, st);
        default: return cudaErrorInvalidValue;
    }
}

template <int D, bool BF16>
static cudaError_t launch_chunk_t(const CUtensorMap& map, const ChunkArgs& a, cudaStream_t st) {
    int blocks = (a.n_items + ChunkCfg<D>::W - 1) / ChunkCfg<D>::W;
    if (blocks <= 0) return cudaSuccess;
    chunk_kernel<D, ChunkCfg<D>::NT, ChunkCfg<D>::W, ChunkCfg<D>::S, BF16><<<blocks, ChunkCfg<D>::W * 32, chunk_smem<D>(), st>>>(map, a);
    return cudaGetLastError();
}

cudaError_t launch_chunk(const CUtensorMap& map, const ChunkArgs& a, bool bf16, cudaStream_t st) {
    switch (a.geo.d) {
        case 64: return bf16 ? launch_chunk_t<64, true>(map, a, st) : launch_chunk_t<64, false>(map, a, st);
        case 128: return bf16 ? launch_chunk_t<128, true>(map, a, st) : launch_chunk_t<128, false>(map, a, st);
        case 256: return bf16 ? launch_chunk_t<256, true>(map, a, st) : launch_chunk_t<256, false>(map, a, st);
        default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_resolve_units(const SegInfo* segs, int n_segs, const int32_t* tables, int n_kv, int num_pages,
                                 int32_t* unit_row, int n_units, int32_t* status, cudaStream_t st,
                                 int32_t* zero_a, int n_a, int32_t* zero_b, int n_b) {
    if (!zero_a) n_a = 0;
    if (!zero_b) n_b = 0;
    if (n_units <= 0 && n_a <= 0 && n_b <= 0) return cudaSuccess;
    const int blocks = std::max(1, std::min((std::max(n_units, n_a) + 255) / 256, 148 * 4));
    resolve_units_kernel<<<blocks, 256, 0, st>>>(segs, n_segs, tables, n_kv, num_pages, unit_row, n_units, status, zero_a, n_a, zero_b, n_b);
    return cudaGetLastError();
}

cudaError_t launch_generic(const GenericArgs& a, bool bf16, cudaStream_t st) {
    int64_t rows = (int64_t)a.step.n_tokens * a.geo.n_q;
    int blocks = (int)((rows + 3) / 4);
    if (blocks <= 0) return cudaSuccess;
    if (bf16) generic_kernel<true><<<blocks, 128, 0, st>>>(a);
    else generic_kernel<false><<<blocks, 128, 0, st>>>(a);
    return cudaGetLastError();
}

}  // namespace cbkv
