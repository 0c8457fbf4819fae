// Bytes of an int8 KV record -> f16 / bf16 numbers, in registers (kv_dequantize, kv.rs:319-358).
//
// Every value byte of a record is b = q + 128.  f16: a byte under the exponent byte 0x64 reads as
// 1024 + b, and subtracting 1152 leaves q.  bf16 has one mantissa bit less than a byte is wide, so
// there the bytes are first made two's complement (one XOR per word, q8_fix): the low seven bits
// under 0x43 read as 128 + (b & 127), the sign bit under 0x43 reads as 128 or 256, and their
// difference is q.  Both subtractions are exact, and so is q * scale before its one rounding, so
// mul2(q8_pair(..), scale) equals elem(q as f32 * scale as f32) of the reference bit for bit.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdint>

namespace cbkv {

template <bool BF16> __device__ __forceinline__ uint32_t q8_fix(uint32_t w) { return BF16 ? (w ^ 0x80808080u) : w; }

// two bytes of `src` (selected by `sel`, which also places the exponent bytes) -> two numbers q
template <bool BF16>
__device__ __forceinline__ uint32_t q8_pair(uint32_t src, uint32_t sel) {
    uint32_t v = __byte_perm(src, BF16 ? 0x43434343u : 0x64646464u, sel);
    if constexpr (BF16) {
        uint32_t lo = v & 0xff7fff7fu, hi = v & 0xff80ff80u;
        __nv_bfloat162 r = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&lo), *reinterpret_cast<__nv_bfloat162*>(&hi));
        return *reinterpret_cast<uint32_t*>(&r);
    } else {
        const uint32_t bias = 0x64806480u;  // 1152, 1152
        __half2 r = __hsub2(*reinterpret_cast<__half2*>(&v), *reinterpret_cast<const __half2*>(&bias));
        return *reinterpret_cast<uint32_t*>(&r);
    }
}
template <bool BF16>
__device__ __forceinline__ uint32_t mul2(uint32_t a, uint32_t b) {
    if constexpr (BF16) {
        __nv_bfloat162 r = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
        return *reinterpret_cast<uint32_t*>(&r);
    } else {
        __half2 r = __hmul2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
        return *reinterpret_cast<uint32_t*>(&r);
    }
}
constexpr uint32_t SEL_LO = 0x5140u;    // bytes 0 and 1 of the source, each under an exponent byte
constexpr uint32_t SEL_HI = 0x7362u;    // bytes 2 and 3
constexpr uint32_t SEL_EVEN = 0x5240u;  // bytes 0 and 2
constexpr uint32_t SEL_ODD = 0x7341u;   // bytes 1 and 3

// 16 bytes of a K row (16 consecutive d of one token, one scale group) -> 16 numbers q * scale.
// `scale2` holds the group's scale in both halves.
template <bool BF16>
__device__ __forceinline__ void q8_unpack_k16(const uint4& raw, uint32_t scale2, uint4& lo, uint4& hi) {
    const uint32_t w0 = q8_fix<BF16>(raw.x), w1 = q8_fix<BF16>(raw.y), w2 = q8_fix<BF16>(raw.z), w3 = q8_fix<BF16>(raw.w);
    lo.x = mul2<BF16>(q8_pair<BF16>(w0, SEL_LO), scale2); lo.y = mul2<BF16>(q8_pair<BF16>(w0, SEL_HI), scale2);
    lo.z = mul2<BF16>(q8_pair<BF16>(w1, SEL_LO), scale2); lo.w = mul2<BF16>(q8_pair<BF16>(w1, SEL_HI), scale2);
    hi.x = mul2<BF16>(q8_pair<BF16>(w2, SEL_LO), scale2); hi.y = mul2<BF16>(q8_pair<BF16>(w2, SEL_HI), scale2);
    hi.z = mul2<BF16>(q8_pair<BF16>(w3, SEL_LO), scale2); hi.w = mul2<BF16>(q8_pair<BF16>(w3, SEL_HI), scale2);
}
// 16 bytes of the V area (8 consecutive d of a token pair, interleaved per d) -> 8 numbers of the
// even token and 8 of the odd one.  `scales` = the group's scale of the even token in its low half, of
// the odd token in its high half (as the record stores them).
template <bool BF16>
__device__ __forceinline__ void q8_unpack_v8x2(const uint4& raw, uint32_t scales, uint4& even, uint4& odd) {
    const uint32_t w0 = q8_fix<BF16>(raw.x), w1 = q8_fix<BF16>(raw.y), w2 = q8_fix<BF16>(raw.z), w3 = q8_fix<BF16>(raw.w);
    const uint32_t se = __byte_perm(scales, 0, 0x1010), so = __byte_perm(scales, 0, 0x3232);
    even.x = mul2<BF16>(q8_pair<BF16>(w0, SEL_EVEN), se); odd.x = mul2<BF16>(q8_pair<BF16>(w0, SEL_ODD), so);
    even.y = mul2<BF16>(q8_pair<BF16>(w1, SEL_EVEN), se); odd.y = mul2<BF16>(q8_pair<BF16>(w1, SEL_ODD), so);
    even.z = mul2<BF16>(q8_pair<BF16>(w2, SEL_EVEN), se); odd.z = mul2<BF16>(q8_pair<BF16>(w2, SEL_ODD), so);
    even.w = mul2<BF16>(q8_pair<BF16>(w3, SEL_EVEN), se); odd.w = mul2<BF16>(q8_pair<BF16>(w3, SEL_ODD), so);
}

}  // namespace cbkv
