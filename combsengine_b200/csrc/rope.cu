// Rotary position embedding and per-head QK norm fused into the append.
//
// The reference runs these as separate tensor ops right before the cache call
// (llama.rs:273-285): rms_norm of q and k over head_dim (norm.rs:11-39), then
// RotaryEmbedding::apply on both (rope.rs:180-204), and only then the cache scatters k
// and v into pages (kv.rs:721-739).  Here one launch reads the un-rotated q, k, v of
// the step once, writes the rotated q to a dense buffer for the attention kernel and
// writes the rotated k and the plain v straight into their page slots.
//
// Arithmetic follows the reference's tensor dtype: the norm is f32 math on up-cast
// inputs rounded once; the rotation is element-wise in the storage type, out =
// x*cos + rotate_half(x)*sin with both products and the sum each rounded to that type
// (a product of two 11-bit or 8-bit significands is exact in f32, and so is the sum
// whenever rounding could depend on it, so f32 ops followed by a rounding conversion
// give the correctly rounded storage-type result).
//
// HBM-bound: every input byte is read once,
// every output byte written once, the (cos, sin) row of a token is shared by its heads
// through L2.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cmath>

#include "kernels.hpp"

namespace cbkv {

// ------------------------------------------------------------------ host: tables
// scaled_inv_freq (rope.rs:31-125) and build_tables_scaled (rope.rs:129-151); f64 math.
int32_t rope_inv_freq(const cbkv_rope_config& c, std::vector<double>* inv, double* mscale) {
    const int half = c.head_dim / 2;
    const double pi = 3.14159265358979323846;
    inv->resize((size_t)half);
    for (int i = 0; i < half; i++) (*inv)[(size_t)i] = std::pow(c.theta, -2.0 * (double)i / (double)c.head_dim);
    *mscale = 1.0;
    switch (c.scaling) {
        case CBKV_ROPE_NONE: return CBKV_OK;
        case CBKV_ROPE_LINEAR:
            for (double& f : *inv) f = f / c.factor;
            return CBKV_OK;
        case CBKV_ROPE_LLAMA3: {
            const double orig = (double)c.original_max_position;
            const double low_wavelen = orig / c.low_freq_factor, high_wavelen = orig / c.high_freq_factor;
            for (double& f : *inv) {
                const double wavelen = 2.0 * pi / f;
                if (wavelen < high_wavelen) continue;
                if (wavelen > low_wavelen) { f = f / c.factor; continue; }
                const double smooth = (orig / wavelen - c.low_freq_factor) / (c.high_freq_factor - c.low_freq_factor);
                f = (1.0 - smooth) * f / c.factor + smooth * f;
            }
            return CBKV_OK;
        }
        case CBKV_ROPE_YARN: {
            const double dim = (double)c.head_dim, orig = (double)c.original_max_position;
            auto corr_dim = [&](double rotations) { return dim * std::log(orig / (rotations * 2.0 * pi)) / (2.0 * std::log(c.theta)); };
            const double low = std::max(std::floor(corr_dim(c.beta_fast)), 0.0);
            double high = std::min(std::ceil(corr_dim(c.beta_slow)), dim - 1.0);
            if (std::fabs(high - low) < 2.220446049250313e-16) high += 0.001;
            for (int i = 0; i < half; i++) {
                const double pos_freq = std::pow(c.theta, 2.0 * (double)i / dim);
                const double extrapolation = 1.0 / pos_freq, interpolation = 1.0 / (c.factor * pos_freq);
                const double ramp = std::min(1.0, std::max(0.0, ((double)i - low) / (high - low)));
                const double keep = 1.0 - ramp;
                (*inv)[(size_t)i] = interpolation * (1.0 - keep) + extrapolation * keep;
            }
            *mscale = c.has_attention_factor ? c.attention_factor : 0.1 * std::log(c.factor) + 1.0;
            return CBKV_OK;
        }
        case CBKV_ROPE_LONGROPE: {
            for (int i = 0; i < half; i++)
                (*inv)[(size_t)i] /= (c.short_factor && i < c.n_short_factor) ? c.short_factor[i] : 1.0;
            if (c.has_attention_factor) *mscale = c.attention_factor;
            else if (c.factor <= 1.0) *mscale = 1.0;
            else *mscale = std::sqrt(1.0 + std::log(c.factor) / std::log((double)c.original_max_position));
            return CBKV_OK;
        }
    }
    return CBKV_ERR_ARG;
}

void rope_tables(const cbkv_rope_config& c, const std::vector<double>& inv, double mscale, float* cos_out, float* sin_out) {
    const int half = c.head_dim / 2;
    for (int64_t pos = 0; pos < c.max_position; pos++)
        for (int i = 0; i < half; i++) {
            const double angle = (double)pos * inv[(size_t)i];
            const float cv = (float)(std::cos(angle) * mscale), sv = (float)(std::sin(angle) * mscale);
            cos_out[pos * c.head_dim + i] = cos_out[pos * c.head_dim + half + i] = cv;
            sin_out[pos * c.head_dim + i] = sin_out[pos * c.head_dim + half + i] = sv;
        }
}

// ------------------------------------------------------------------ device
// Two storage-type elements in one 32-bit word, with the non-fusing 2-wide instructions:
// each product and each sum is rounded on its own, never contracted into a multiply-add.
template <bool BF16> struct Pack;
template <> struct Pack<false> {
    using V2 = __half2;
    static __device__ __forceinline__ float2 up(uint32_t v) { return __half22float2(*reinterpret_cast<__half2*>(&v)); }
    static __device__ __forceinline__ float rt(float f) { return __half2float(__float2half_rn(f)); }
    static __device__ __forceinline__ uint32_t down(float a, float b) {
        __half2 h = __floats2half2_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&h);
    }
};
template <> struct Pack<true> {
    using V2 = __nv_bfloat162;
    static __device__ __forceinline__ float2 up(uint32_t v) { return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&v)); }
    static __device__ __forceinline__ float rt(float f) { return __bfloat162float(__float2bfloat16_rn(f)); }
    static __device__ __forceinline__ uint32_t down(float a, float b) {
        __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&h);
    }
};

// rope.rs:196-201 on two (i, i+half) pairs: out[i] = x1*cos + (-x2)*sin, out[i+half] = x2*cos + x1*sin.
template <bool BF16>
__device__ __forceinline__ void rotate2(uint32_t& x1, uint32_t& x2, uint32_t c, uint32_t s) {
    using V2 = typename Pack<BF16>::V2;
    const V2 a = *reinterpret_cast<V2*>(&x1), b = *reinterpret_cast<V2*>(&x2);
    const V2 cc = *reinterpret_cast<V2*>(&c), ss = *reinterpret_cast<V2*>(&s);
    V2 o1 = __hadd2_rn(__hmul2_rn(a, cc), __hmul2_rn(__hneg2(b), ss));
    V2 o2 = __hadd2_rn(__hmul2_rn(b, cc), __hmul2_rn(a, ss));
    x1 = *reinterpret_cast<uint32_t*>(&o1);
    x2 = *reinterpret_cast<uint32_t*>(&o2);
}

// y = x * inv_rms * w in f32, rounded once (norm.rs:27-28); gemma: w + 1 formed in the storage type.
template <bool BF16>
__device__ __forceinline__ uint32_t norm2(uint32_t x, uint32_t w, float inv_rms, bool gemma) {
    using P = Pack<BF16>;
    const float2 u = P::up(x);
    float2 wf = P::up(w);
    if (gemma) { wf.x = P::rt(__fadd_rn(wf.x, 1.f)); wf.y = P::rt(__fadd_rn(wf.y, 1.f)); }
    return P::down(__fmul_rn(__fmul_rn(u.x, inv_rms), wf.x), __fmul_rn(__fmul_rn(u.y, inv_rms), wf.y));
}

template <bool BF16>
__device__ __forceinline__ float sumsq2(uint32_t x) {
    const float2 u = Pack<BF16>::up(x);
    return __fadd_rn(__fmul_rn(u.x, u.x), __fmul_rn(u.y, u.y));
}

// Which sequence a packed row belongs to: the last one whose first row is <= row.
__device__ __forceinline__ int seq_of_row(const StepDev& s, int64_t row, int heads) {
    int lo = 0, hi = s.n_seqs - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if ((int64_t)s.seq_meta[mid].tok_off * heads <= row) lo = mid; else hi = mid - 1;
    }
    return lo;
}

// Table row of a position: head_dim/2 cosines, then head_dim/2 sines, storage type.

// ---- any head_dim that is a multiple of 4, up to 512: one warp per row, two elements per lane and round
constexpr int ROPE_MAX_IT = 4;

template <bool BF16>
__global__ void __launch_bounds__(256) rope_append_kernel(const RopeArgs a) {
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const int d = a.geo.d, half = d >> 1, chunks = half >> 1;  // a chunk = 2 elements = 4 bytes
    const int64_t q_rows = (int64_t)a.step.n_tokens * a.geo.n_q, kv_rows = (int64_t)a.step.n_tokens * a.geo.n_kv;
    const int64_t total = q_rows + (a.k_out ? 1 : 2) * kv_rows;
    for (int64_t R = warp0; R < total; R += nwarps) {
        const int kind = R < q_rows ? 0 : (R < q_rows + kv_rows ? 1 : 2);  // 0 = q, 1 = k, 2 = v
        const int64_t row = kind == 0 ? R : (kind == 1 ? R - q_rows : R - q_rows - kv_rows);
        const int heads = kind == 0 ? a.geo.n_q : a.geo.n_kv;
        const int b = seq_of_row(a.step, row, heads);
        const SeqMeta sm = a.step.seq_meta[b];
        const int64_t local = row - (int64_t)sm.tok_off * heads;
        const int h = (int)(local / sm.snew), r = (int)(local - (int64_t)h * sm.snew);
        const int gpos = sm.pos + r;  // absolute position of the row's token (kv.rs:725, rope.rs:185-194)
        const uint32_t* src = reinterpret_cast<const uint32_t*>(kind == 0 ? a.q : (kind == 1 ? a.k : a.v)) + row * (d >> 1);
        uint32_t* dst;
        if (kind == 0) {
            dst = reinterpret_cast<uint32_t*>(a.q_out) + row * (d >> 1);
        } else if (a.k_out) {
            dst = reinterpret_cast<uint32_t*>(a.k_out) + row * (d >> 1);
        } else {
            int phys = a.step.tables[sm.tbl_off + gpos / a.geo.page_size];  // kv.rs:728
            if (phys < 0 || phys >= a.geo.num_pages) { if (lane == 0) atomicOr(a.status, ST_BAD_PAGE); continue; }
            const int slot = gpos % a.geo.page_size;                        // kv.rs:726
            const int64_t drow = ((int64_t)phys * a.geo.n_kv + h) * 2 * a.geo.page_size +
                                 page_row(kind == 2, slot, a.geo.page_size, a.geo.tiled != 0);
            dst = reinterpret_cast<uint32_t*>(a.arena) + drow * (d >> 1);
        }
        if (kind == 2) {  // v: a bit copy
            for (int c = lane; c < d >> 1; c += 32) dst[c] = src[c];
            continue;
        }
        uint32_t x1[ROPE_MAX_IT], x2[ROPE_MAX_IT], cw[ROPE_MAX_IT], sw[ROPE_MAX_IT];
        const int tpos = min(gpos, (int)a.max_position - 1);  // the host refuses a step past the table
        const uint32_t* trow = reinterpret_cast<const uint32_t*>(a.table) + (int64_t)tpos * half;  // 2 * chunks words
#pragma unroll
        for (int it = 0; it < ROPE_MAX_IT; it++) {
            const int c = lane + it * 32;
            if (c < chunks) {
                x1[it] = src[c];
                x2[it] = src[chunks + c];
                cw[it] = trow[c];
                sw[it] = trow[chunks + c];
            }
        }
        const void* wv = kind == 0 ? a.q_weight : a.k_weight;
        if (wv) {  // mean(x^2) over head_dim, norm.rs:22-23
            float ss = 0.f;
#pragma unroll
            for (int it = 0; it < ROPE_MAX_IT; it++)
                if (lane + it * 32 < chunks) ss = __fadd_rn(ss, __fadd_rn(sumsq2<BF16>(x1[it]), sumsq2<BF16>(x2[it])));
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss = __fadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, o));
            const float inv_rms = __frcp_rn(__fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)d), a.eps)));
            const uint32_t* w32 = reinterpret_cast<const uint32_t*>(wv);
#pragma unroll
            for (int it = 0; it < ROPE_MAX_IT; it++) {
                const int c = lane + it * 32;
                if (c < chunks) {
                    x1[it] = norm2<BF16>(x1[it], w32[c], inv_rms, a.gemma != 0);
                    x2[it] = norm2<BF16>(x2[it], w32[chunks + c], inv_rms, a.gemma != 0);
                }
            }
        }
#pragma unroll
        for (int it = 0; it < ROPE_MAX_IT; it++) {
            const int c = lane + it * 32;
            if (c < chunks) {
                rotate2<BF16>(x1[it], x2[it], cw[it], sw[it]);
                dst[c] = x1[it];
                dst[chunks + c] = x2[it];
            }
        }
    }
}

// ---- head_dim in {16, 32, 64, 128, 256, 512}: T = head_dim/16 lanes share a row, each lane owns 8
// consecutive elements of the first half and the matching 8 of the second half (two 16-byte loads of
// data, one each of cosines and sines), so a warp keeps 32/T rows in flight, and a k/v row's
// block-table look-up overlaps its data loads.
constexpr int ROPE_SEQ_SMEM = 1024;

template <bool BF16, int T>
__global__ void __launch_bounds__(256) rope_append_vec_kernel(const RopeArgs a) {
    __shared__ int s_tok[ROPE_SEQ_SMEM];
    const int n_seqs = a.step.n_seqs;
    const bool in_smem = n_seqs <= ROPE_SEQ_SMEM;
    if (in_smem) {
        for (int i = threadIdx.x; i < n_seqs; i += blockDim.x) s_tok[i] = a.step.seq_meta[i].tok_off;
        __syncthreads();
    }
    const int lane = threadIdx.x & 31, t = lane % T, sub = lane / T;
    constexpr int RPW = 32 / T;  // rows per warp per round
    // row counts fit 32 bits (the launcher checks)
    const uint32_t warp0 = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = (gridDim.x * blockDim.x) >> 5;
    const uint32_t q_rows = (uint32_t)a.step.n_tokens * a.geo.n_q, kv_rows = (uint32_t)a.step.n_tokens * a.geo.n_kv;
    const uint32_t total = q_rows + (a.k_out ? 1u : 2u) * kv_rows;
    for (uint32_t R0 = warp0 * RPW; R0 < total; R0 += nwarps * RPW) {
        const uint32_t R = R0 + sub;
        const bool live = R < total;
        const uint32_t Rc = live ? R : total - 1;
        const int kind = Rc < q_rows ? 0 : (Rc < q_rows + kv_rows ? 1 : 2);
        const uint32_t row = kind == 0 ? Rc : (kind == 1 ? Rc - q_rows : Rc - q_rows - kv_rows);
        const uint32_t heads = kind == 0 ? a.geo.n_q : a.geo.n_kv;
        // data first: its address does not depend on the sequence look-up
        const uint4* src = reinterpret_cast<const uint4*>(kind == 0 ? a.q : (kind == 1 ? a.k : a.v)) + (size_t)row * (2 * T);
        const uint4 xa = src[t], xb = src[T + t];
        int b;
        if (in_smem) {
            int lo = 0, hi = n_seqs - 1;
            while (lo < hi) {
                const int mid = (lo + hi + 1) >> 1;
                if ((uint32_t)s_tok[mid] * heads <= row) lo = mid; else hi = mid - 1;
            }
            b = lo;
        } else {
            b = seq_of_row(a.step, row, (int)heads);
        }
        const SeqMeta sm = a.step.seq_meta[b];
        const uint32_t local = row - (uint32_t)sm.tok_off * heads;
        const uint32_t h = local / (uint32_t)sm.snew, r = local - h * (uint32_t)sm.snew;
        const int gpos = sm.pos + (int)r;
        uint4 tc = make_uint4(0, 0, 0, 0), ts = tc;
        if (kind != 2) {
            const int tpos = min(gpos, (int)a.max_position - 1);
            const uint4* trow = reinterpret_cast<const uint4*>(a.table) + (size_t)tpos * (2 * T);
            tc = trow[t]; ts = trow[T + t];
        }
        uint4* dst;
        bool ok = live;
        if (kind == 0) {
            dst = reinterpret_cast<uint4*>(a.q_out) + (size_t)row * (2 * T);
        } else if (a.k_out) {
            dst = reinterpret_cast<uint4*>(a.k_out) + (size_t)row * (2 * T);
        } else {
            int phys = a.step.tables[sm.tbl_off + gpos / a.geo.page_size];
            if (phys < 0 || phys >= a.geo.num_pages) { if (live && t == 0) atomicOr(a.status, ST_BAD_PAGE); phys = 0; ok = false; }
            const int slot = gpos % a.geo.page_size;
            const int64_t drow = ((int64_t)phys * a.geo.n_kv + h) * 2 * a.geo.page_size +
                                 page_row(kind == 2, slot, a.geo.page_size, a.geo.tiled != 0);
            dst = reinterpret_cast<uint4*>(a.arena) + drow * (2 * T);
        }
        uint32_t A[4] = {xa.x, xa.y, xa.z, xa.w}, B[4] = {xb.x, xb.y, xb.z, xb.w};
        const void* wv = kind == 0 ? a.q_weight : (kind == 1 ? a.k_weight : nullptr);
        if (wv) {
            float ss = 0.f;
#pragma unroll
            for (int j = 0; j < 4; j++) ss = __fadd_rn(ss, __fadd_rn(sumsq2<BF16>(A[j]), sumsq2<BF16>(B[j])));
            // sum over the T lanes of the row; rows of other kinds in this warp may skip the norm, so the
            // shuffle names only the lanes of this row
            const unsigned grp = T == 32 ? 0xffffffffu : (((1u << T) - 1u) << (sub * T));
#pragma unroll
            for (int o = T / 2; o > 0; o >>= 1) ss = __fadd_rn(ss, __shfl_xor_sync(grp, ss, o));
            const float inv_rms = __frcp_rn(__fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)a.geo.d), a.eps)));
            const uint4* w4 = reinterpret_cast<const uint4*>(wv);
            const uint4 wa = w4[t], wb = w4[T + t];
            const uint32_t WA[4] = {wa.x, wa.y, wa.z, wa.w}, WB[4] = {wb.x, wb.y, wb.z, wb.w};
#pragma unroll
            for (int j = 0; j < 4; j++) {
                A[j] = norm2<BF16>(A[j], WA[j], inv_rms, a.gemma != 0);
                B[j] = norm2<BF16>(B[j], WB[j], inv_rms, a.gemma != 0);
            }
        }
        if (kind != 2) {
            const uint32_t TC[4] = {tc.x, tc.y, tc.z, tc.w}, TS[4] = {ts.x, ts.y, ts.z, ts.w};
#pragma unroll
            for (int j = 0; j < 4; j++) rotate2<BF16>(A[j], B[j], TC[j], TS[j]);
        }
        if (ok) {
            dst[t] = make_uint4(A[0], A[1], A[2], A[3]);
            dst[T + t] = make_uint4(B[0], B[1], B[2], B[3]);
        }
    }
}

template <bool BF16>
static cudaError_t launch_rope_t(const RopeArgs& a, int64_t rows, cudaStream_t st) {
    const int t = a.geo.d / 16;
    const int rpw = t ? 32 / t : 0;
    auto grid = [&](int per_block) { return (int)std::min<int64_t>((rows + per_block - 1) / per_block, 148 * 8); };
    const bool vec = rows < ((int64_t)1 << 31) - 64;  // the vector kernels count rows in 32 bits
    switch (vec ? a.geo.d : 0) {
        case 16: rope_append_vec_kernel<BF16, 1><<<grid(8 * rpw), 256, 0, st>>>(a); break;
        case 32: rope_append_vec_kernel<BF16, 2><<<grid(8 * rpw), 256, 0, st>>>(a); break;
        case 64: rope_append_vec_kernel<BF16, 4><<<grid(8 * rpw), 256, 0, st>>>(a); break;
        case 128: rope_append_vec_kernel<BF16, 8><<<grid(8 * rpw), 256, 0, st>>>(a); break;
        case 256: rope_append_vec_kernel<BF16, 16><<<grid(8 * rpw), 256, 0, st>>>(a); break;
        case 512: rope_append_vec_kernel<BF16, 32><<<grid(8 * rpw), 256, 0, st>>>(a); break;
        default: rope_append_kernel<BF16><<<grid(8), 256, 0, st>>>(a); break;  // one warp per row
    }
    return cudaGetLastError();
}

cudaError_t launch_rope_append(const RopeArgs& a, bool bf16, cudaStream_t st) {
    const int64_t rows = (int64_t)a.step.n_tokens * (a.geo.n_q + (a.k_out ? 1 : 2) * a.geo.n_kv);
    if (rows <= 0) return cudaSuccess;
    return bf16 ? launch_rope_t<true>(a, rows, st) : launch_rope_t<false>(a, rows, st);
}

}  // namespace cbkv
