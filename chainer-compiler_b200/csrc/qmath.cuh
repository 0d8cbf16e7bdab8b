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

// Folded requantization of a uint8 output: t = float(acc) * m with m = (x_scale * w_scale[c]) / y_scale computed once per
// channel; then the zero point, the rounding and the saturation exactly as quantize_one does them.
__device__ __forceinline__ int requant_u8_fold(int acc, float m, const RequantParams& p) {
    float t = __fmul_rn((float)acc, m);
    if (p.round_mode != 0) return cvt_rne_sat_u8(__fadd_rn(rintf(t), p.y_zp_f));
    if (p.y_has_zp) t = __fadd_rn(t, p.y_zp_f);
    return cvt_floor_sat_u8(__fadd_rn(t, 0.5f));
}

// Folded residual tail: v = (q - y_zp) * (y_scale / out_scale) + (r - res_zp) * (res_scale / out_scale) with the second
// product fused into the sum (one rounding), Relu, then zero point, rounding and saturation of the output.
__device__ __forceinline__ int residual_fold(int q, int r, const RequantParams& p) {
    float u = (float)q;
    if (p.y_has_zp) u = __fsub_rn(u, p.y_zp_f);
    u = __fmul_rn(u, p.y_over_out);
    float w = (float)r;
    if (p.res_has_zp) w = __fsub_rn(w, p.res_zp_f);
    float v = __fmaf_rn(w, p.res_over_out, u);
    if (p.res_relu) v = v > 0.f ? v : 0.f;
    if (p.round_mode != 0) return cvt_rne_sat_u8(__fadd_rn(rintf(v), p.out_zp_f));
    if (p.out_has_zp) v = __fadd_rn(v, p.out_zp_f);
    return cvt_floor_sat_u8(__fadd_rn(v, 0.5f));
}

// DequantizeLinear(y), DequantizeLinear(r), Add, Relu, QuantizeLinear on one element.
__device__ __forceinline__ int residual_one(int q, int r, const RequantParams& p) {
    float v = __fadd_rn(dequantize_one(q, p.y_scale, p.y_zp_f, p.y_has_zp != 0), dequantize_one(r, p.res_scale, p.res_zp_f, p.res_has_zp != 0));
    if (p.res_relu) v = v > 0.f ? v : 0.f;
    return quantize_one<false>(v, p.out_scale, p.out_zp_f, p.out_has_zp != 0, p.round_mode);
}

}  // namespace chxq
