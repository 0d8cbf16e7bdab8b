// Device-side arithmetic shared by every kernel that quantizes or dequantizes a value.
// Each function states the reference lines whose fp32 operation order it keeps; the explicit
// __f*_rn intrinsics stop the compiler from contracting a*b+c into one rounding.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

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

// Division by a scale that is constant for a whole kernel, without the per-element reciprocal of the general IEEE
// sequence: q0 = x * r with r = RN(1/s) from the host, then two residual corrections q <- fma(fma(-q, s, x), r, q).
// After the first correction the quotient is faithful; the second, from an exact residual, makes it the correctly
// rounded x / s (Markstein's scheme; a scale whose significand is all ones is the known exception and is sent to the
// general path by make_qdiv, as are scales outside a safe exponent range).  Quotients of magnitude >= 1e18 (and NaN) take
// the general division; below 2^-60 the value returned may be inexact, which no quantization can observe.
struct QDiv {
    float s, r;
    int fast;
};

inline QDiv make_qdiv(float s) {
    QDiv d;
    d.s = s;
    d.r = 1.0f / s;
    uint32_t bits;
    memcpy(&bits, &s, 4);
    const float a = s < 0 ? -s : s;
    d.fast = (a > 1e-15f && a < 1e15f && (bits & 0x7fffffu) != 0x7fffffu) ? 1 : 0;
    return d;
}

// The corrected quotient without the magnitude guard, and the guard on its own: a caller dividing many values can test
// them together and redo the few that need the general division.
__device__ __forceinline__ float qdiv_unguarded(float x, const QDiv& d, bool* needs_general) {
    const float q0 = __fmul_rn(x, d.r);
    float rem = __fmaf_rn(-q0, d.s, x);
    float q = __fmaf_rn(rem, d.r, q0);
    rem = __fmaf_rn(-q, d.s, x);
    q = __fmaf_rn(rem, d.r, q);
    *needs_general = *needs_general || !(fabsf(q0) < 1.0e18f);
    return q;
}

__device__ __forceinline__ float qdiv(float x, const QDiv& d) {
    if (!d.fast) return __fdiv_rn(x, d.s);
    const float q0 = __fmul_rn(x, d.r);
    float rem = __fmaf_rn(-q0, d.s, x);
    float q = __fmaf_rn(rem, d.r, q0);
    rem = __fmaf_rn(-q, d.s, x);
    q = __fmaf_rn(rem, d.r, q);
    if (!(fabsf(q0) < 1.0e18f)) q = __fdiv_rn(x, d.s);
    return q;
}

// quantize_one for a uint8 output (round-half-up) on a pre-divided value, conversion-free: byte in the low bits of
// the returned word.
__device__ __forceinline__ uint32_t quantize_u8_up_bits(float t, float zp_f) {
    t = __fadd_rn(__fadd_rn(t, zp_f), 0.5f);  // adding a zero zero point is exact
    return __float_as_uint(__fadd_rd(fminf(fmaxf(t, 0.f), 255.5f), 8388608.f)) & 0xffu;
}

// uint8, round-half-to-even on a pre-divided value, conversion-free: saturate(rint(t) + zp).  (t + 1.5 * 2^23) - 1.5 * 2^23
// is rint(t) for |t| <= 2^22; beyond +-4e6 the result saturates whatever the zero point, so t is clamped there first.
__device__ __forceinline__ uint32_t quantize_u8_rne_bits(float t, float zp_f) {
    const float tc = fminf(fmaxf(t, -4.0e6f), 4.0e6f);
    const float r = __fsub_rn(__fadd_rn(tc, 12582912.f), 12582912.f);
    const float u = __fadd_rn(r, zp_f);
    return __float_as_uint(__fadd_rn(fminf(fmaxf(u, 0.f), 255.f), 8388608.f)) & 0xffu;
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
    // constant-divisor forms of y_scale and out_scale (see QDiv)
    QDiv y_div, out_div;
};

inline void finish_requant_params(RequantParams* p) {
    p->y_div = make_qdiv(p->y_scale);
    p->out_div = make_qdiv(p->out_scale != 0.f ? p->out_scale : 1.f);
}

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

// uint8, round-half-up requantization of one accumulator (+ optional residual tail) without conversion instructions other
// than the int -> float of the accumulator; equals requant_one / residual_one (reference operation order, fold == 0) or
// requant_u8_fold / residual_fold (fold != 0) bit for bit.  Returns the output byte.
__device__ __forceinline__ uint32_t requant_u8_up_fast(int acc, int bias, float mult, bool has_res, uint32_t res_byte, const RequantParams& p) {
    const float hi_ph = (p.clamp_hi_q >= 0 ? (float)p.clamp_hi_q : 255.f) + 0.5f;
    float tp;
    if (p.fold) {
        const float m = __fdiv_rn(mult, p.y_scale);
        tp = __fmaf_rn((float)acc, m, __fmaf_rn((float)bias, m, __fadd_rn(p.y_zp_f, 0.5f)));
    } else {
        tp = qdiv(__fmul_rn((float)(int)((unsigned)acc + (unsigned)bias), mult), p.y_div);
        tp = __fadd_rn(__fadd_rn(tp, p.y_zp_f), 0.5f);
    }
    float f = quant_u8_up_magic(tp, hi_ph);
    if (has_res) {
        const float u = __fsub_rn(f, __fadd_rn(kMagic23, p.y_zp_f));
        const float w = __fsub_rn(__uint_as_float(0x4B000000u | (res_byte & 0xffu)), __fadd_rn(kMagic23, p.res_zp_f));
        float v;
        if (p.fold) {
            v = __fmaf_rn(w, p.res_over_out, __fmul_rn(u, p.y_over_out));
            if (p.res_relu) v = fmaxf(v, 0.f);
            v = __fadd_rn(v, __fadd_rn(p.out_zp_f, 0.5f));
        } else {
            v = __fadd_rn(__fmul_rn(u, p.y_scale), __fmul_rn(w, p.res_scale));
            if (p.res_relu) v = fmaxf(v, 0.f);
            v = __fadd_rn(__fadd_rn(qdiv(v, p.out_div), p.out_zp_f), 0.5f);
        }
        f = quant_u8_up_magic(v, 255.5f);
    }
    return __float_as_uint(f) & 0xffu;
}

// DequantizeLinear(y), DequantizeLinear(r), Add, Relu, QuantizeLinear on one element.
__device__ __forceinline__ int residual_one(int q, int r, const RequantParams& p) {
    float v = __fadd_rn(dequantize_one(q, p.y_scale, p.y_zp_f, p.y_has_zp != 0), dequantize_one(r, p.res_scale, p.res_zp_f, p.res_has_zp != 0));
    if (p.res_relu) v = v > 0.f ? v : 0.f;
    return quantize_one<false>(v, p.out_scale, p.out_zp_f, p.out_has_zp != 0, p.round_mode);
}

}  // namespace chxq
