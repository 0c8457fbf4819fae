/*
 * rope_oracle.c — CPU restatement of the step immediately before the paged KV path:
 * rotary position embedding and the per-head QK norm.
 *
 * TEST INFRASTRUCTURE ONLY (the checker for the fused rotate-and-append kernel);
 * nothing in the product library links, imports or calls it.
 *
 * Restates
 *   engine/core/combs-models/src/rope.rs   scaled_inv_freq :31-125, build_tables_scaled
 *                                          :129-151, RotaryEmbedding::apply :180-204
 *   engine/core/combs-models/src/norm.rs   rms_norm :11-29, gemma_rms_norm :33-39
 * and is pinned by the known-answer tests the reference keeps next to that code
 * (rope.rs:211-330): tests/test_rope_oracle.py repeats every one of them.
 *
 * Arithmetic types: the frequency and table math is f64 on the host, the tables are
 * stored as f32 and converted to the tensor element type when they reach the device
 * (rope.rs:167-176), and `apply` is element-wise arithmetic in that element type:
 * out = x*cos + rotate_half(x)*sin, every product and the sum rounded on its own.
 * The norm is f32 math on up-cast inputs, rounded once at the end (norm.rs:20-28).
 *
 * Built into the same two libraries as kv_oracle.c (elem = float, or -DORC_F16 half).
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

#ifdef ORC_F16
typedef uint16_t elem_t;
static inline float ld(elem_t x) { _Float16 h; memcpy(&h, &x, 2); return (float)h; }
static inline elem_t st(float f) { _Float16 h = (_Float16)f; elem_t x; memcpy(&x, &h, 2); return x; }
#else
typedef float elem_t;
static inline float ld(elem_t x) { return x; }
static inline elem_t st(float f) { return f; }
#endif

enum { ORC_ROPE_NONE = 0, ORC_ROPE_LINEAR = 1, ORC_ROPE_LLAMA3 = 2, ORC_ROPE_YARN = 3, ORC_ROPE_LONGROPE = 4 };

static double clampd(double x, double lo, double hi) { return x < lo ? lo : (x > hi ? hi : x); }

/* scaled_inv_freq, rope.rs:31-125.  `attention_factor` NaN = not given.  Returns 0,
 * or -1 for an unknown kind.  inv has head_dim/2 entries. */
int orc_rope_inv_freq(int head_dim, double theta, int kind, double factor, double low_freq_factor,
                      double high_freq_factor, double beta_fast, double beta_slow, int64_t original_max_position,
                      double attention_factor, const double* short_factor, int n_short, double* inv, double* mscale) {
    const int half = head_dim / 2;
    const double pi = 3.14159265358979323846;
    for (int i = 0; i < half; i++) inv[i] = pow(theta, -2.0 * (double)i / (double)head_dim); /* :33-35 */
    *mscale = 1.0;
    switch (kind) {
        case ORC_ROPE_NONE: return 0;                                                          /* :37 */
        case ORC_ROPE_LINEAR:                                                                  /* :38 */
            for (int i = 0; i < half; i++) inv[i] = inv[i] / factor;
            return 0;
        case ORC_ROPE_LLAMA3: {                                                                /* :39-64 */
            const double orig = (double)original_max_position;
            const double low_wavelen = orig / low_freq_factor, high_wavelen = orig / high_freq_factor;
            for (int i = 0; i < half; i++) {
                const double f = inv[i], wavelen = 2.0 * pi / f;
                if (wavelen < high_wavelen) inv[i] = f;
                else if (wavelen > low_wavelen) inv[i] = f / factor;
                else {
                    const double smooth = (orig / wavelen - low_freq_factor) / (high_freq_factor - low_freq_factor);
                    inv[i] = (1.0 - smooth) * f / factor + smooth * f;
                }
            }
            return 0;
        }
        case ORC_ROPE_YARN: {                                                                  /* :65-96 */
            const double dim = (double)head_dim, orig = (double)original_max_position;
            const double c_fast = dim * log(orig / (beta_fast * 2.0 * pi)) / (2.0 * log(theta));
            const double c_slow = dim * log(orig / (beta_slow * 2.0 * pi)) / (2.0 * log(theta));
            const double low = fmax(floor(c_fast), 0.0);
            double high = fmin(ceil(c_slow), dim - 1.0);
            if (fabs(high - low) < 2.220446049250313e-16) high += 0.001;
            for (int i = 0; i < half; i++) {
                const double pos_freq = pow(theta, 2.0 * (double)i / dim);
                const double extrapolation = 1.0 / pos_freq, interpolation = 1.0 / (factor * pos_freq);
                const double ramp = clampd(((double)i - low) / (high - low), 0.0, 1.0);
                const double ef = 1.0 - ramp;
                inv[i] = interpolation * (1.0 - ef) + extrapolation * ef;
            }
            *mscale = isnan(attention_factor) ? 0.1 * log(factor) + 1.0 : attention_factor;
            return 0;
        }
        case ORC_ROPE_LONGROPE: {                                                              /* :97-124 */
            for (int i = 0; i < half; i++) inv[i] = inv[i] / (i < n_short ? short_factor[i] : 1.0);
            if (!isnan(attention_factor)) *mscale = attention_factor;
            else if (factor <= 1.0) *mscale = 1.0;
            else *mscale = sqrt(1.0 + log(factor) / log((double)original_max_position));
            return 0;
        }
    }
    return -1;
}

/* build_tables_scaled, rope.rs:129-151: [max_position][head_dim] f32, the half-dim
 * frequencies appearing twice. */
void orc_rope_tables(int head_dim, int64_t max_position, const double* inv, double mscale, float* cos_out, float* sin_out) {
    const int half = head_dim / 2;
    for (int64_t pos = 0; pos < max_position; pos++)
        for (int rep = 0; rep < 2; rep++)
            for (int i = 0; i < half; i++) {
                const double angle = (double)pos * inv[i];
                cos_out[pos * head_dim + rep * half + i] = (float)(cos(angle) * mscale);
                sin_out[pos * head_dim + rep * half + i] = (float)(sin(angle) * mscale);
            }
}

/* RotaryEmbedding::apply, rope.rs:180-204, in place on x [heads][seq][d]; the first
 * row of every head is at absolute position `pos`.  The tables are converted to the
 * element type first (they live on the device in it, rope.rs:167-176). */
void orc_rope_apply(elem_t* x, int heads, int64_t seq, int d, int64_t pos, const float* cos_t, const float* sin_t) {
    const int half = d / 2;
    for (int h = 0; h < heads; h++)
        for (int64_t r = 0; r < seq; r++) {
            elem_t* row = x + ((int64_t)h * seq + r) * d;
            const float* c = cos_t + (pos + r) * d;
            const float* s = sin_t + (pos + r) * d;
            for (int i = 0; i < half; i++) {
                const float x1 = ld(row[i]), x2 = ld(row[i + half]);
                /* rotated = cat(-x2, x1); out = x*cos + rotated*sin, each op rounded to elem */
                const float a1 = ld(st(x1 * ld(st(c[i])))), b1 = ld(st(-x2 * ld(st(s[i]))));
                const float a2 = ld(st(x2 * ld(st(c[i + half])))), b2 = ld(st(x1 * ld(st(s[i + half]))));
                row[i] = st(a1 + b1);
                row[i + half] = st(a2 + b2);
            }
        }
}

/* rms_norm / gemma_rms_norm over the last dim, norm.rs:11-39, in place on x [rows][d].
 * gemma: weight + 1 is formed in the element type before the up-cast (norm.rs:38). */
void orc_rms_norm(elem_t* x, int64_t rows, int d, const elem_t* w, double eps, int gemma) {
    for (int64_t r = 0; r < rows; r++) {
        elem_t* row = x + r * d;
        float sum = 0.f;
        for (int i = 0; i < d; i++) { const float v = ld(row[i]); sum += v * v; }
        const float mean_sq = sum / (float)d;
        const float inv_rms = 1.0f / sqrtf(mean_sq + (float)eps);
        for (int i = 0; i < d; i++) {
            const float wf = gemma ? ld(st(ld(w[i]) + 1.0f)) : ld(w[i]);
            row[i] = st(ld(row[i]) * inv_rms * wf);
        }
    }
}
