// FP8 E4M3 codec of the KV store, byte-for-byte the reference's (metal_infer/fp8.h:19-118): one scale per
// cache row, scale = absmax / 240 (1 when the row is all zero), encode by round-half-up of the 3-bit mantissa,
// decode = value * scale.  The reference's encoder has two properties a textbook E4M3 conversion does not, and
// both are kept because the stored bytes are part of the cache layout a caller can export:
//   * magnitudes in [2^-9, 2^-6) -- E4M3's subnormal range -- take the normal-number branch with the exponent
//     clamped to -6, which makes the mantissa term negative; OR-ed into the byte as a two's-complement int it
//     yields 0xFA..0xFF (mantissa term -6..-1) or exponent 1 / mantissa 0 (term 0);
//   * the decoder treats only 0x7F as NaN, so 0xFF decodes to -480 * scale.
// A cache row therefore decodes to what the reference's CPU attention would have read.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace fm {

// metal_infer/fp8.h:19-57.  floorf(log2f(mag)) is taken from the exponent field: the two differ only for
// magnitudes a few ulps below a power of two, where log2f rounds up to the integer -- and there both give the
// same byte (the mantissa carries into the next exponent on one side and is zero on the other).
__device__ __forceinline__ uint8_t fp8_e4m3_encode_ref(float x, float inv_scale) {
    float scaled = x * inv_scale;
    if (scaled != scaled) return 0x7F;
    scaled = fminf(fmaxf(scaled, -448.0f), 448.0f);
    const uint32_t bits = __float_as_uint(scaled);
    const uint32_t sign = bits >> 31;
    const float mag = fabsf(scaled);
    if (mag < 0.001953125f) {  // below 2^-9
        int m = (int)(mag / 0.001953125f + 0.5f);
        if (m > 7) m = 7;
        return (uint8_t)((sign << 7) | (uint32_t)m);
    }
    int e = (int)((bits >> 23) & 0xFF) - 127;
    if (e < -6) e = -6;
    if (e > 8) e = 8;
    const float frac = mag / __uint_as_float((uint32_t)(e + 127) << 23) - 1.0f;
    int mant = (int)(__fadd_rn(__fmul_rn(frac, 8.0f), 0.5f));
    if (mant > 7) { mant = 0; e++; }
    int eb = e + 7;
    if (eb < 0) { eb = 0; mant = 0; }
    if (eb > 15) { eb = 15; mant = 6; }
    if (eb == 15 && mant >= 7) mant = 6;
    return (uint8_t)((int)(sign << 7) | (eb << 3) | mant);  // a negative mant sets every upper bit, as in the reference
}

// metal_infer/fp8.h:63-82
__device__ __forceinline__ float fp8_e4m3_decode_ref(uint8_t b, float scale) {
    if (b == 0x7F) return __uint_as_float(0x7FC00000u);
    const int eb = (b >> 3) & 0xF, mant = b & 7;
    float val = eb == 0 ? (float)mant * 0.001953125f : (1.0f + (float)mant / 8.0f) * __uint_as_float((uint32_t)(eb - 7 + 127) << 23);
    if (b & 0x80) val = -val;
    return __fmul_rn(val, scale);
}

// Two E4M3 bytes of `r` (selector: a byte-permute selector that puts them in the high byte of each 16-bit lane; the
// low bytes are zero) as two fp16 numbers.  The hardware conversion gives the exact values; E4M3's NaN codes come out as
// NaN, and the maximum with -480 turns them into -480 (max returns its other operand for a NaN, and every other
// value is above -448): that is what the reference's decoder makes of 0xFF (it knows only 0x7F as NaN; 0x7F is never
// produced from finite data, and reads as -480 here).
#ifndef FM_FP8_HW_CVT
#define FM_FP8_HW_CVT 1
#endif
#if FM_FP8_HW_CVT
__device__ __forceinline__ uint32_t fp8x2_cvt(uint32_t pair16) {
    uint32_t d;
    asm("{\n\t.reg .b16 p;\n\tcvt.u16.u32 p, %1;\n\tcvt.rn.f16x2.e4m3x2 %0, p;\n\tmax.f16x2 %0, %0, %2;\n\t}\n" : "=r"(d) : "r"(pair16), "r"(0xDF80DF80u));
    return d;
}
__device__ __forceinline__ uint32_t fp8x2_to_f16x2_scaled(uint32_t r, uint32_t selector) {
    // the same byte pairs as the permute form below, as the two bytes of a 16-bit word
    if (selector == 0x1404u) return fp8x2_cvt(r & 0xffffu);
    if (selector == 0x3424u) return fp8x2_cvt(r >> 16);
    return fp8x2_cvt(__byte_perm(r, 0u, selector == 0x2404u ? 0x4420u : 0x4431u));
}
constexpr float kFp8HalfScale = 1.0f;
#else
// Without the conversion instruction: the byte's exponent and mantissa bits are simply placed in the fp16
// exponent / mantissa fields (E4M3 normal -> fp16 normal, E4M3 subnormal -> fp16 subnormal, both short by the
// same factor 2^-8 because the biases differ by 8), and the sign is moved up by one bit.  0xFF comes out as
// -480 * 2^-8, matching the reference's decoder; 0x7F as +480 * 2^-8.
__device__ __forceinline__ uint32_t fp8x2_to_f16x2_scaled(uint32_t r, uint32_t selector) {
    const uint32_t t = __byte_perm(r, 0u, selector) >> 1;  // per lane: bit 14 sign, bits 13..7 exponent | mantissa
    return t + (t & 0x40004000u);                          // carry the sign into bit 15
}
constexpr float kFp8HalfScale = 256.0f;  // what this form leaves out
#endif

}  // namespace fm
