// Device-side arithmetic shared by every kernel that quantizes or dequantizes a value.
// Each function states the reference lines whose fp32 operation order it keeps; the explicit
// __f*_rn intrinsics stop the compiler from contracting a*b+c into one rounding.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace chxq {

// Saturating float -> uint8 conversions (one instruction each): floor / nearest-even, clamped to [0, 255].
__device__ __forceinline__ int cvt_floor_sat_u8(float t) {
    uint32_t q;
    asm("cvt.rmi.sat.u8.f32 %0, %1;" : "=r"(q) : "f"(t));
    return (int)q;
}
__device__ __forceinline__ int cvt_rne_sat_u8(float t) {
    uint32_t q;
    asm("cvt.rni.sat.u8.f32 %0, %1;" : "=r"(q) : "f"(t));
    return (int)q;
}

// One element of quantize_array (runtime/ops/quantize.cc:29-34): t = x / s; (+zp); min(hi);
// max(lo); + 0.5f; truncate.  ROUND_RNE instead gives saturate(rint(x / s) + zp).
template <bool kSigned>
__device__ __forceinline__ int quantize_one(float x, float scale, float zp_f, bool has_zp, int round_mode) {
    const float lo = kSigned ? -128.f : 0.f;
    const float hi = kSigned ? 127.f : 255.f;
    float t = __fdiv_rn(x, scale);
    if (!kSigned) {
        // uint8: clamp, +0.5f and truncation fold into one saturating conversion with the same result for every
        // input: clamp(t) + 0.5f >= 0.5 makes the truncation a floor, and floor(t + 0.5f) saturated to [0, 255]
        // agrees with it on both sides of the clamp.  (Not so for int8, where truncation is toward zero.)
        if (round_mode != 0) return cvt_rne_sat_u8(__fadd_rn(rintf(t), zp_f));
        if (has_zp) t = __fadd_rn(t, zp_f);
        return cvt_floor_sat_u8(__fadd_rn(t, 0.5f));
    }
    if (round_mode != 0) {
        t = __fadd_rn(rintf(t), zp_f);
        t = fminf(t, hi);
        t = fmaxf(lo, t);
        return (int)t;
    }
    if (has_zp) t = __fadd_rn(t, zp_f);
    t = t < hi ? t : hi;
    t = lo > t ? lo : t;
    t = __fadd_rn(t, 0.5f);
    return (int)t;  // cvt.rzi: C++ static_cast truncation, as AsType does
}

__device__ __forceinline__ int quantize_any(float x, float scale, float zp_f, bool has_zp, int round_mode, bool is_signed) {
    return is_signed ? quantize_one<true>(x, scale, zp_f, has_zp, round_mode) : quantize_one<false>(x, scale, zp_f, has_zp, round_mode);
}

// dequantize_array (runtime/ops/quantize.cc:37-44).
__device__ __forceinline__ float dequantize_one(int q, float scale, float zp_f, bool has_zp) {
    float v = (float)q;
    if (has_zp) v = __fsub_rn(v, zp_f);
    return __fmul_rn(v, scale);
}

// Parameters of a requantizing epilogue (QLinearConv / QLinearMatMul and the fused residual tail).
struct RequantParams {
    float y_scale;
    float y_zp_f;
    int y_has_zp;
    int y_signed;
    int round_mode;
    int clamp_hi_q;  // -1 = off
    // residual tail (res == nullptr: off)
    float res_scale, res_zp_f;
    int res_has_zp;
    int res_relu;
    float out_scale, out_zp_f;
    int out_has_zp;
    // Folded arithmetic (fold != 0): one multiplier per channel, (x_scale * w_scale[m]) / y_scale, instead of a multiply
    // and a divide per element; the residual tail uses the pre-divided scales below.
    int fold;
    float y_over_out;    // y_scale / out_scale
    float res_over_out;  // res_scale / out_scale
};

// acc (exact int32, bias already added) -> quantized output value.
__device__ __forceinline__ int requant_one(int acc, float mult, const RequantParams& p) {
    const float yf = __fmul_rn((float)acc, mult);
    int q = quantize_any(yf, p.y_scale, p.y_zp_f, p.y_has_zp != 0, p.round_mode, p.y_signed != 0);
    if (p.clamp_hi_q >= 0 && q > p.clamp_hi_q) q = p.clamp_hi_q;
    return q;
}

// requant_one for a uint8 output without the optional upper clamp (the caller applies it).
__device__ __forceinline__ int requant_u8_fast(int acc, float mult, const RequantParams& p) {
    return quantize_one<false>(__fmul_rn((float)acc, mult), p.y_scale, p.y_zp_f, p.y_has_zp != 0, p.round_mode);
}

// Folded requantization of a uint8 output (RequantParams::fold; no counterpart in the reference): one multiplier and one
// additive term per channel,
//     M = (x_scale * w_scale[c]) / y_scale,        B = fma(float(bias), M, y_zp + 0.5)        (round-half-up)
//     y = min(max(floor(fma(float(acc), M, B)), 0), hi)
// or, for round-half-to-even, B = fma(float(bias), M, y_zp) and y = clamp(rint(fma(float(acc), M, B)), 0, hi).
// `acc` is the accumulator without the bias.
__device__ __forceinline__ float fold_offset(int bias, float m, const RequantParams& p) {
    return __fmaf_rn((float)bias, m, p.round_mode != 0 ? p.y_zp_f : __fadd_rn(p.y_zp_f, 0.5f));
}

__device__ __forceinline__ int requant_u8_fold(int acc, int bias, float m, const RequantParams& p) {
    const float t = __fmaf_rn((float)acc, m, fold_offset(bias, m, p));
    int q = p.round_mode != 0 ? cvt_rne_sat_u8(rintf(t)) : cvt_floor_sat_u8(t);
    if (p.clamp_hi_q >= 0 && q > p.clamp_hi_q) q = p.clamp_hi_q;
    return q;
}

// Folded residual tail: v = fma(r - res_zp, res_scale / out_scale, (q - y_zp) * (y_scale / out_scale)), Relu, then
// floor(v + (out_zp + 0.5)) (round-half-up) or rint(v) + out_zp (round-half-to-even), saturated to uint8.
__device__ __forceinline__ int residual_fold(int q, int r, const RequantParams& p) {
    const float u = __fmul_rn(__fsub_rn((float)q, p.y_zp_f), p.y_over_out);
    float v = __fmaf_rn(__fsub_rn((float)r, p.res_zp_f), p.res_over_out, u);
    if (p.res_relu) v = fmaxf(v, 0.f);
    if (p.round_mode != 0) return cvt_rne_sat_u8(__fadd_rn(rintf(v), p.out_zp_f));
    return cvt_floor_sat_u8(__fadd_rn(v, __fadd_rn(p.out_zp_f, 0.5f)));
}

// ---- conversion-free forms for the tensor-core epilogue -------------------------------------------------------------
// Float <-> integer conversions issue on the quarter-rate pipe; the epilogue handles billions of bytes, so it rounds and
// converts with ordinary adds instead.  For 0 <= x < 2^23, x + 2^23 rounded toward minus infinity is the float
// 2^23 + floor(x), whose low mantissa bits are the integer; a byte b becomes the float 2^23 + b by placing it under the
// exponent pattern 0x4B000000.  Every function below returns exactly what its cvt-based counterpart returns.
constexpr float kMagic23 = 8388608.f;         // 2^23
constexpr float kMagicRne = 12582912.f;       // 1.5 * 2^23: (x + c) - c == rint(x) for |x| <= 2^22

// Round-half-up uint8 quantization of a value that already holds t + zp + 0.5: returns the float 2^23 + q with
// q = min(max(floor(tp), 0), hi); hi_plus_half = hi + 0.5f.  floor(clamp(tp, 0, hi + 0.5)) is that value, and the add
// that rounds toward minus infinity takes the floor.
__device__ __forceinline__ float quant_u8_up_magic(float tp, float hi_plus_half) {
    return __fadd_rd(fminf(fmaxf(tp, 0.f), hi_plus_half), kMagic23);
}

__device__ __forceinline__ uint32_t magic_byte(float f) {
    return __float_as_uint(f) & 0xffu;
}

// The float 2^23 + byte `sel` (0..3) of word w.
__device__ __forceinline__ float byte_to_magic(uint32_t w, int sel) {
    return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540 | sel) );
}

// DequantizeLinear(y), DequantizeLinear(r), Add, Relu, QuantizeLinear on one element.
__device__ __forceinline__ int residual_one(int q, int r, const RequantParams& p) {
    float v = __fadd_rn(dequantize_one(q, p.y_scale, p.y_zp_f, p.y_has_zp != 0), dequantize_one(r, p.res_scale, p.res_zp_f, p.res_has_zp != 0));
    if (p.res_relu) v = v > 0.f ? v : 0.f;
    return quantize_one<false>(v, p.out_scale, p.out_zp_f, p.out_has_zp != 0, p.round_mode);
}

}  // namespace chxq
