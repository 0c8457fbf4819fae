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
// One warp per row of head_dim elements; HBM-bound: every input byte is read once,
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
template <bool BF16> struct Pack;
template <> struct Pack<false> {
    static __device__ __forceinline__ float2 up(uint32_t v) { return __half22float2(*reinterpret_cast<__half2*>(&v)); }
    static __device__ __forceinline__ float rt(float f) { return __half2float(__float2half_rn(f)); }
    static __device__ __forceinline__ uint32_t down(float a, float b) {
        __half2 h = __floats2half2_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&h);
    }
};
template <> struct Pack<true> {
    static __device__ __forceinline__ float2 up(uint32_t v) { return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&v)); }
    static __device__ __forceinline__ float rt(float f) { return __bfloat162float(__float2bfloat16_rn(f)); }
    static __device__ __forceinline__ uint32_t down(float a, float b) {
        __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&h);
    }
};

// Which sequence a packed row belongs to: the last one whose first row is <= row.
__device__ __forceinline__ int seq_of_row(const StepDev& s, int64_t row, int heads) {
    int lo = 0, hi = s.n_seqs - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if ((int64_t)s.seq_meta[mid].tok_off * heads <= row) lo = mid; else hi = mid - 1;
    }
    return lo;
}

constexpr int ROPE_MAX_IT = 4;  // head_dim <= 512: a lane keeps at most 4 element pairs of each half

template <bool BF16>
__global__ void __launch_bounds__(256) rope_append_kernel(const RopeArgs a) {
    using P = Pack<BF16>;
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const int d = a.geo.d, half = d >> 1, chunks = half >> 1;  // a chunk = 2 elements = 4 bytes
    const int64_t q_rows = (int64_t)a.step.n_tokens * a.geo.n_q, kv_rows = (int64_t)a.step.n_tokens * a.geo.n_kv;
    const int64_t total = q_rows + 2 * kv_rows;
    for (int64_t R = warp0; R < total; R += nwarps) {
        // 0 = q, 1 = k, 2 = v
        const int kind = R < q_rows ? 0 : (R < q_rows + kv_rows ? 1 : 2);
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
        uint32_t x1[ROPE_MAX_IT], x2[ROPE_MAX_IT];
        uint2 cs[ROPE_MAX_IT];
        const int tpos = min(gpos, (int)a.max_position - 1);  // the host refuses a step past the table
        const uint2* trow = reinterpret_cast<const uint2*>(a.table) + (int64_t)tpos * chunks;
#pragma unroll
        for (int it = 0; it < ROPE_MAX_IT; it++) {
            const int c = lane + it * 32;
            if (c < chunks) {
                x1[it] = src[c];
                x2[it] = src[chunks + c];
                cs[it] = trow[c];
            }
        }
        const void* wv = kind == 0 ? a.q_weight : a.k_weight;
        float inv_rms = 0.f;
        if (wv) {  // mean(x^2) over head_dim, norm.rs:22-23
            float ss = 0.f;
#pragma unroll
            for (int it = 0; it < ROPE_MAX_IT; it++) {
                if (lane + it * 32 < chunks) {
                    const float2 u = P::up(x1[it]), v = P::up(x2[it]);
                    ss = __fadd_rn(ss, __fadd_rn(__fadd_rn(__fmul_rn(u.x, u.x), __fmul_rn(u.y, u.y)),
                                                 __fadd_rn(__fmul_rn(v.x, v.x), __fmul_rn(v.y, v.y))));
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss = __fadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, o));
            inv_rms = __frcp_rn(__fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)d), a.eps)));
        }
        const uint32_t* w32 = reinterpret_cast<const uint32_t*>(wv);
#pragma unroll
        for (int it = 0; it < ROPE_MAX_IT; it++) {
            const int c = lane + it * 32;
            if (c < chunks) {
                float2 u = P::up(x1[it]), v = P::up(x2[it]);
                if (wv) {  // y = x * inv_rms * w, rounded to the storage type (norm.rs:27-28)
                    float2 w1 = P::up(w32[c]), w2 = P::up(w32[chunks + c]);
                    if (a.gemma) {  // weight + 1 in the storage type (norm.rs:38)
                        w1.x = P::rt(__fadd_rn(w1.x, 1.f)); w1.y = P::rt(__fadd_rn(w1.y, 1.f));
                        w2.x = P::rt(__fadd_rn(w2.x, 1.f)); w2.y = P::rt(__fadd_rn(w2.y, 1.f));
                    }
                    u.x = P::rt(__fmul_rn(__fmul_rn(u.x, inv_rms), w1.x)); u.y = P::rt(__fmul_rn(__fmul_rn(u.y, inv_rms), w1.y));
                    v.x = P::rt(__fmul_rn(__fmul_rn(v.x, inv_rms), w2.x)); v.y = P::rt(__fmul_rn(__fmul_rn(v.y, inv_rms), w2.y));
                }
                // table chunk: (cos_i, sin_i, cos_{i+1}, sin_{i+1}); i and i + half share the frequency
                const float2 t0 = P::up(cs[it].x), t1 = P::up(cs[it].y);
                // out[i] = x1*cos + (-x2)*sin ; out[i+half] = x2*cos + x1*sin     (rope.rs:196-201)
                const float o1x = __fadd_rn(P::rt(__fmul_rn(u.x, t0.x)), P::rt(__fmul_rn(-v.x, t0.y)));
                const float o1y = __fadd_rn(P::rt(__fmul_rn(u.y, t1.x)), P::rt(__fmul_rn(-v.y, t1.y)));
                const float o2x = __fadd_rn(P::rt(__fmul_rn(v.x, t0.x)), P::rt(__fmul_rn(u.x, t0.y)));
                const float o2y = __fadd_rn(P::rt(__fmul_rn(v.y, t1.x)), P::rt(__fmul_rn(u.y, t1.y)));
                dst[c] = P::down(o1x, o1y);
                dst[chunks + c] = P::down(o2x, o2y);
            }
        }
    }
}

cudaError_t launch_rope_append(const RopeArgs& a, bool bf16, cudaStream_t st) {
    const int64_t rows = (int64_t)a.step.n_tokens * (a.geo.n_q + 2 * a.geo.n_kv);
    if (rows <= 0) return cudaSuccess;
    const int blocks = (int)std::min<int64_t>((rows + 7) / 8, 148 * 8);
    if (bf16) rope_append_kernel<true><<<blocks, 256, 0, st>>>(a);
    else rope_append_kernel<false><<<blocks, 256, 0, st>>>(a);
    return cudaGetLastError();
}

}  // namespace cbkv
