// int8 KV pages: CacheConfig::quantize_kv of the reference (kv.rs:271-358, 464-475, 740-787).
//
//   append_quant_kernel    kv_quantize (kv.rs:284-313) fused with the page scatter
//                          (kv.rs:746-768): per 32-value group scale = max(absmax/127, 1e-8)
//                          in f32, q = clamp(round(x/scale), -127, 127), one byte q + 128 per
//                          value, scale kept in the element type
//   generic_quant_kernel   attention over quantised pages for any shape: kv_dequantize
//                          (kv.rs:319-358) happens on the fly, value = elem(q * scale), f32 math
//
// One record per (page, kv head), laid out for the decode kernel (qrec_* in kernels.hpp),
// so a decode step reads d + d/16 bytes per cached token and head instead of 2d.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>

#include "kernels.hpp"
#include "q8_unpack.cuh"

namespace cbkv {

namespace {

template <bool BF16> __device__ __forceinline__ float q_up(uint16_t v) {
    if (BF16) return __bfloat162float(__ushort_as_bfloat16(v));
    return __half2float(__ushort_as_half(v));
}
template <bool BF16> __device__ __forceinline__ uint16_t q_down(float f) {
    if (BF16) return __bfloat16_as_ushort(__float2bfloat16_rn(f));
    return __half_as_ushort(__float2half_rn(f));
}

template <bool BF16>
__global__ void __launch_bounds__(256) append_quant_kernel(const AppendArgs a) {
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const int d = a.geo.d, P = a.geo.page_size, Hkv = a.geo.n_kv;
    const int words = d >> 2;                                  // 4 values per packed word
    const int64_t kv_rows = (int64_t)a.step.n_tokens * Hkv;
    uint8_t* arena = reinterpret_cast<uint8_t*>(a.arena);
    const size_t rec = qrec_bytes(P, d);
    for (int64_t R = warp0; R < 2 * kv_rows; R += nwarps) {
        const int is_v = R >= kv_rows;
        const int64_t row = is_v ? R - kv_rows : R;
        int lo = 0, hi = a.step.n_seqs - 1;
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if ((int64_t)a.step.seq_meta[mid].tok_off * Hkv <= row) lo = mid; else hi = mid - 1;
        }
        const SeqMeta sm = a.step.seq_meta[lo];
        const int64_t local = row - (int64_t)sm.tok_off * Hkv;
        const int h = (int)(local / sm.snew), r = (int)(local - (int64_t)h * sm.snew);
        const int gpos = sm.pos + r;                            // kv.rs:749
        int phys = a.step.tables[sm.tbl_off + gpos / P];        // kv.rs:752
        if (phys < 0 || phys >= a.geo.num_pages) { if (lane == 0) atomicOr(a.status, ST_BAD_PAGE); continue; }
        const int slot = gpos % P;                              // kv.rs:750
        uint8_t* recp = arena + ((size_t)phys * Hkv + h) * rec;
        const uint2* src = reinterpret_cast<const uint2*>(is_v ? a.v : a.k) + row * words;
        // every lane runs every round (the shuffles below name the full warp)
        for (int c0 = 0; c0 < words; c0 += 32) {
            const int c = c0 + lane;
            const bool live = c < words;
            float x[4] = {0.f, 0.f, 0.f, 0.f};
            if (live) {
                const uint2 raw = src[c];
                x[0] = q_up<BF16>((uint16_t)(raw.x & 0xffff)); x[1] = q_up<BF16>((uint16_t)(raw.x >> 16));
                x[2] = q_up<BF16>((uint16_t)(raw.y & 0xffff)); x[3] = q_up<BF16>((uint16_t)(raw.y >> 16));
            }
            float amax = fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3])));
            // a group is 32 values = 8 consecutive lanes
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
            const float scale = fmaxf(__fdiv_rn(amax, 127.0f), 1e-8f);   // kv.rs:296-301
            if (live) {
                uint32_t word = 0;  // four bytes q + 128
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    float q = roundf(__fdiv_rn(x[i], scale));             // kv.rs:302-305
                    q = fminf(fmaxf(q, -127.f), 127.f);
                    word |= (uint32_t)((int)q + 128) << (8 * i);
                }
                if (!is_v) {
                    *reinterpret_cast<uint32_t*>(recp + qrec_value_off(0, slot, 4 * c, P, d)) = word;
                } else {  // the pair's other token sits between these bytes
#pragma unroll
                    for (int i = 0; i < 4; i++) recp[qrec_value_off(1, slot, 4 * c + i, P, d)] = (uint8_t)(word >> (8 * i));
                }
                if ((c & 7) == 0)
                    *reinterpret_cast<uint16_t*>(recp + qrec_scale_off(is_v, slot, c >> 3, P, d)) = q_down<BF16>(scale);
            }
        }
    }
}

// A fresh quantised arena reads as the reference's zero-filled one (kv.rs:699-705): packed words 0
// mean q = -128 in lanes 0-2 and q = 0 in lane 3, i.e. record bytes 0, 0, 0, 0x80; scales 0.
__global__ void init_quant_kernel(uint8_t* arena, size_t n_records, int P, int d) {
    const size_t rec = qrec_bytes(P, d), values = (size_t)2 * P * d;
    const size_t words = n_records * (rec / 4);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < words; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / (rec / 4), w = i - r * (rec / 4), off = w * 4;
        uint32_t v = 0;
        if (off < (size_t)P * d) v = 0x80000000u;                  // K: lane 3 is the top byte of each word
        else if (off < values) v = (w & 1) ? 0x80800000u : 0u;      // V: lane 3 of both tokens = bytes 6, 7 of each 8
        reinterpret_cast<uint32_t*>(arena)[i] = v;
    }
}

// kv_dequantize (kv.rs:319-358) of every page the step's sequences hold, into a float layer in the tiled
// row order, so that the tensor-core chunk kernels can run over an int8 layer.  One warp per
// (block-table entry, kv head): value = elem(q * scale), exactly what the reference's gather produces.
template <bool BF16>
__global__ void __launch_bounds__(256) dequant_pages_kernel(const int32_t* tables, int n_entries, GeomDev geo, const uint8_t* arena,
                                                            uint16_t* scratch, int32_t* status) {
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const int D = geo.d, P = geo.page_size, Hkv = geo.n_kv, G = D / 32;
    const size_t rec = qrec_bytes(P, D);
    const int k_chunks = P * D / 16, sw = qrec_swizzled(D) ? 1 : 0;
    const bool tiled = geo.tiled != 0;
    for (int64_t it = warp0; it < (int64_t)n_entries * Hkv; it += nwarps) {
        const int e = (int)(it / Hkv), h = (int)(it - (int64_t)e * Hkv);
        const int phys = tables[e];
        if (phys < 0 || phys >= geo.num_pages) { if (lane == 0) atomicOr(status, ST_BAD_PAGE); continue; }
        const uint8_t* recp = arena + ((size_t)phys * Hkv + h) * rec;
        const uint16_t* ksc = reinterpret_cast<const uint16_t*>(recp + (size_t)2 * P * D);
        const uint32_t* vsc = reinterpret_cast<const uint32_t*>(ksc + P * G);  // group-major: one word = two neighbouring tokens
        uint16_t* dst = scratch + ((size_t)phys * Hkv + h) * 2 * P * D;
        // a lane takes 16-byte pieces of the record as they lie (coalesced) and works out which values they hold
        for (int c = lane; c < 2 * k_chunks; c += 32) {
            const uint4 raw = __ldg(reinterpret_cast<const uint4*>(recp) + c);
            if (c < k_chunks) {  // K: 16 consecutive d of one token, inside one 32-value group (qrec_value_off)
                const int off = c * 16, slot = off / D, pos = off - slot * D;
                const int grp = (pos >> 5) ^ qrec_swz(slot, D), j0 = grp * 32 + (pos & 31);
                const uint32_t s1 = ksc[slot * G + grp];
                uint4 lo, hi;
                q8_unpack_k16<BF16>(raw, s1 | (s1 << 16), lo, hi);
                uint4* out = reinterpret_cast<uint4*>(dst + (size_t)page_row(0, slot, P, tiled) * D + j0);
                out[0] = lo; out[1] = hi;
            } else {             // V: 8 consecutive d of a token pair, interleaved per d
                const int off = (c - k_chunks) * 16, pair = off / (2 * D), rem = off - pair * 2 * D;
                const int grp = (rem >> 6) ^ (sw * (pair & 1));
                const int chunk = ((rem & 63) >> 3) ^ (sw * 4 * ((pair >> 1) & 1));
                const int j0 = grp * 32 + chunk * 4;
                uint4 even, odd;
                q8_unpack_v8x2<BF16>(raw, vsc[(grp * P + 2 * pair) >> 1], even, odd);
                *reinterpret_cast<uint4*>(dst + (size_t)page_row(1, 2 * pair, P, tiled) * D + j0) = even;
                *reinterpret_cast<uint4*>(dst + (size_t)page_row(1, 2 * pair + 1, P, tiled) * D + j0) = odd;
            }
        }
    }
}

// One warp per query row, any page size and head_dim (multiple of 32, <= 512).
template <bool BF16>
__global__ void generic_quant_kernel(const GenericArgs a) {
    __shared__ float qs[4][512];
    const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t rid = (int64_t)blockIdx.x * 4 + w;
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
    const int h = hq / a.geo.n_rep;
    const int q_pos = sm.pos + r;
    const uint16_t* q = reinterpret_cast<const uint16_t*>(a.q) + rid * D;
    for (int j = lane; j < D; j += 32) qs[w][j] = q_up<BF16>(q[j]);
    __syncwarp();
    const uint8_t* arena = reinterpret_cast<const uint8_t*>(a.arena);
    const size_t rec = qrec_bytes(P, D);
    // kv_dequantize (kv.rs:319-358): value = elem(q * scale); every byte of a record is q + 128
    auto value = [&](const uint8_t* recp, int is_v, int slot, int j) -> float {
        const uint8_t b = recp[qrec_value_off(is_v, slot, j, P, D)];
        const int qi = (int)b - 128;
        const float sc = q_up<BF16>(*reinterpret_cast<const uint16_t*>(recp + qrec_scale_off(is_v, slot, j >> 5, P, D)));
        return q_up<BF16>(q_down<BF16>(__fmul_rn((float)qi, sc)));
    };
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
            const uint8_t* recp = arena + ((size_t)phys * Hkv + h) * rec;
            float dot = 0.f;
            for (int j = 0; j < D; j++) dot += qs[w][j] * value(recp, 0, tk % P, j);
            s = dot * a.scale;
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
            const uint8_t* recp = arena + ((size_t)phys * Hkv + h) * rec;
#pragma unroll
            for (int i = 0; i < 16; i++) {
                const int j = lane + 32 * i;
                if (j < D) acc[i] += pk * value(recp, 1, tv % P, j);
            }
        }
    }
    uint16_t* out = reinterpret_cast<uint16_t*>(a.out) + rid * D;
    const float inv = 1.f / l;
#pragma unroll
    for (int i = 0; i < 16; i++) {
        const int j = lane + 32 * i;
        if (j < D) out[j] = q_down<BF16>(acc[i] * inv);
    }
}

}  // namespace

cudaError_t launch_init_quant(void* arena, size_t n_records, int page_size, int d, cudaStream_t st) {
    init_quant_kernel<<<148 * 8, 256, 0, st>>>(reinterpret_cast<uint8_t*>(arena), n_records, page_size, d);
    return cudaGetLastError();
}

cudaError_t launch_append_quant(const AppendArgs& a, bool bf16, cudaStream_t st) {
    const int64_t rows = 2 * (int64_t)a.step.n_tokens * a.geo.n_kv;
    if (rows <= 0) return cudaSuccess;
    const int blocks = (int)std::min<int64_t>((rows + 7) / 8, 148 * 8);
    if (bf16) append_quant_kernel<true><<<blocks, 256, 0, st>>>(a);
    else append_quant_kernel<false><<<blocks, 256, 0, st>>>(a);
    return cudaGetLastError();
}

cudaError_t launch_dequant_pages(const int32_t* tables, int n_entries, const GeomDev& geo, const void* arena, void* scratch,
                                 int32_t* status, bool bf16, cudaStream_t st) {
    const int64_t items = (int64_t)n_entries * geo.n_kv;
    if (items <= 0) return cudaSuccess;
    const int blocks = (int)std::min<int64_t>((items + 7) / 8, 148 * 8);
    if (bf16) dequant_pages_kernel<true><<<blocks, 256, 0, st>>>(tables, n_entries, geo, reinterpret_cast<const uint8_t*>(arena), reinterpret_cast<uint16_t*>(scratch), status);
    else dequant_pages_kernel<false><<<blocks, 256, 0, st>>>(tables, n_entries, geo, reinterpret_cast<const uint8_t*>(arena), reinterpret_cast<uint16_t*>(scratch), status);
    return cudaGetLastError();
}

cudaError_t launch_generic_quant(const GenericArgs& a, bool bf16, cudaStream_t st) {
    const int64_t rows = (int64_t)a.step.n_tokens * a.geo.n_q;
    if (rows <= 0) return cudaSuccess;
    const int blocks = (int)((rows + 3) / 4);
    if (bf16) generic_quant_kernel<true><<<blocks, 128, 0, st>>>(a);
    else generic_quant_kernel<false><<<blocks, 128, 0, st>>>(a);
    return cudaGetLastError();
}

}  // namespace cbkv
