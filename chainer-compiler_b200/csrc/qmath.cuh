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

// ---- packed pairs of floats (one 64-bit register) and the saturating scalar forms -----------------------------------
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    uint64_t d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(lo), "f"(hi));
    return d;
}
__device__ __forceinline__ float lo_of(uint64_t v) { return __uint_as_float((uint32_t)v); }
__device__ __forceinline__ float hi_of(uint64_t v) { return __uint_as_float((uint32_t)(v >> 32)); }
__device__ __forceinline__ uint64_t add_rm_x2(uint64_t a, uint64_t b) {  // round toward minus infinity
    uint64_t d;
    asm("add.rm.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t add_x2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t sub_x2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t mul_x2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t fma_x2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t fma_rm_x2(uint64_t a, uint64_t b, uint64_t c) {  // round toward minus infinity
    uint64_t d;
    asm("fma.rm.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ float fma_sat(float a, float b, float c) {  // clamp(fma(a, b, c), 0, 1)
    float d;
    asm("fma.rn.sat.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ float add_sat(float a, float b) {
    float d;
    asm("add.rn.sat.f32 %0, %1, %2;" : "=f"(d) : "f"(a), "f"(b));
    return d;
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

// Four uint8 round-half-up quantizations at once, bit-identical to quantize_u8_up_bits(qdiv_unguarded(x)) per element, with
// half the arithmetic instructions: the division runs on packed pairs (mul / fma .f32x2) and scaled by 2^-8 (divisor 256 s,
// reciprocal r / 256 -- powers of two, so every intermediate is the unscaled one times 2^-8 exactly), so that the lower clamp
// is the .sat of the add of the rounding half, the upper clamp one min against 255.5 / 256, and the floor an add toward minus
// infinity against 2^15 (whose ulp is 2^-8): the byte is the low 8 bits of that sum.  *needs_general is raised when a
// quotient is NaN or >= 1e18 in magnitude, as in qdiv_unguarded.
struct QDiv8 {
    uint64_t s2, r2, zp2;  // packed {256 s, 256 s}, {r / 256, r / 256}, {zp / 256, zp / 256}
};
__device__ __forceinline__ QDiv8 make_qdiv8(const QDiv& d, float zp_f) {
    QDiv8 o;
    const float s8 = __fmul_rn(d.s, 256.f), r8 = __fmul_rn(d.r, 0.00390625f), z8 = __fmul_rn(zp_f, 0.00390625f);
    o.s2 = pack2(-s8, -s8);
    o.r2 = pack2(r8, r8);
    o.zp2 = pack2(z8, z8);
    return o;
}
__device__ __forceinline__ uint32_t quantize4_u8_up(const float4 v, const QDiv8& d, bool* needs_general) {
    const uint64_t xa = pack2(v.x, v.y), xb = pack2(v.z, v.w);
    const uint64_t q0a = mul_x2(xa, d.r2), q0b = mul_x2(xb, d.r2);
    uint64_t qa = fma_x2(fma_x2(q0a, d.s2, xa), d.r2, q0a), qb = fma_x2(fma_x2(q0b, d.s2, xb), d.r2, q0b);
    qa = fma_x2(fma_x2(qa, d.s2, xa), d.r2, qa);
    qb = fma_x2(fma_x2(qb, d.s2, xb), d.r2, qb);
    const float lim = 3.90625e15f;  // 1e18 / 256
    *needs_general = *needs_general || !(fabsf(lo_of(q0a)) < lim) || !(fabsf(hi_of(q0a)) < lim) || !(fabsf(lo_of(q0b)) < lim) ||
                     !(fabsf(hi_of(q0b)) < lim);
    const uint64_t ua = add_x2(qa, d.zp2), ub = add_x2(qb, d.zp2);
    const float hi = 0.998046875f;  // 255.5 / 256
    const float t0 = fminf(add_sat(lo_of(ua), 0.001953125f), hi), t1 = fminf(add_sat(hi_of(ua), 0.001953125f), hi);
    const float t2 = fminf(add_sat(lo_of(ub), 0.001953125f), hi), t3 = fminf(add_sat(hi_of(ub), 0.001953125f), hi);
    const uint64_t m2 = pack2(32768.f, 32768.f);
    const uint64_t fa = add_rm_x2(pack2(t0, t1), m2), fb = add_rm_x2(pack2(t2, t3), m2);
    return __byte_perm(__byte_perm((uint32_t)fa, (uint32_t)(fa >> 32), 0x0040), __byte_perm((uint32_t)fb, (uint32_t)(fb >> 32), 0x0040), 0x5410);
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
    float fold_a, fold_r, fold_c;  // round-half-up residual tail in units of the output range (see residual_fold)
    // constant-divisor forms of y_scale and out_scale (see QDiv)
    QDiv y_div, out_div;
};

inline void finish_requant_params(RequantParams* p) {
    p->y_div = make_qdiv(p->y_scale);
    p->out_div = make_qdiv(p->out_scale != 0.f ? p->out_scale : 1.f);
}

// Constants of the folded residual tail; call once y_over_out / res_over_out and the zero points are set.  The additive term
// is evaluated in double and rounded once, so that every implementation of it (this one, the CPU oracle's) gives the same float.
inline void finish_fold_params(RequantParams* p) {
    p->fold_a = p->y_over_out / 255.5f;
    p->fold_r = p->res_over_out / 255.5f;
    p->fold_c = (float)((((double)p->out_zp_f + 0.5) - (double)p->y_zp_f * (double)p->y_over_out - (double)p->res_zp_f * (double)p->res_over_out) / 255.5);
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

// Folded requantization of a uint8 output (RequantParams::fold; no counterpart in the reference).
//
// Round-half-up (the reference's rounding).  Per channel, with hp = hi + 0.5 (hi = 255 or the optional upper clamp):
//     M  = (x_scale * w_scale[c]) / y_scale        B  = fma(float(bias), M, y_zp + 0.5)
//     Ms = M / hp                                  Bs = B / hp
// per element, with sat(v) = min(max(v, 0), 1):
//     t = sat(fma(float(acc), Ms, Bs))             y = floor(t * hp)        (the product is exact, one floor)
// i.e. the value is computed in units of the output range, where the saturation of one fused multiply-add is both clamps
// (a zero lower bound is the ReLU when y_zp == 0) and one more multiply-add with a round-down places the integer.
// Round-half-to-even keeps the plain form: B = fma(float(bias), M, y_zp), y = clamp(rint(fma(float(acc), M, B)), 0, hi).
// `acc` is the accumulator without the bias.
struct FoldCh {
    float ms, bs;
};

__device__ __forceinline__ float fold_hi_ph(const RequantParams& p) {
    return (p.clamp_hi_q >= 0 ? (float)p.clamp_hi_q : 255.f) + 0.5f;
}

// m = (x_scale * w_scale[c]) / y_scale
__device__ __forceinline__ FoldCh fold_channel(int bias, float m, const RequantParams& p) {
    FoldCh c;
    if (p.round_mode != 0) {
        c.ms = m;
        c.bs = __fmaf_rn((float)bias, m, p.y_zp_f);
        return c;
    }
    const float hp = fold_hi_ph(p);
    c.ms = __fdiv_rn(m, hp);
    c.bs = __fdiv_rn(__fmaf_rn((float)bias, m, __fadd_rn(p.y_zp_f, 0.5f)), hp);
    return c;
}

// floor(t * hp) for t in [0, 1], hp < 256: the fused multiply-add onto 2^23 rounded toward minus infinity leaves the
// integer in the low mantissa bits.
__device__ __forceinline__ int fold_place(float t, float hp) {
    return (int)(__float_as_uint(__fmaf_rd(t, hp, 8388608.f)) & 0x1ffu);
}

__device__ __forceinline__ int requant_u8_fold(int acc, int bias, float m, const RequantParams& p) {
    const FoldCh c = fold_channel(bias, m, p);
    const float t = __fmaf_rn((float)acc, c.ms, c.bs);
    if (p.round_mode != 0) {
        int q = cvt_rne_sat_u8(rintf(t));
        if (p.clamp_hi_q >= 0 && q > p.clamp_hi_q) q = p.clamp_hi_q;
        return q;
    }
    return fold_place(__saturatef(t), fold_hi_ph(p));
}

// Folded residual tail.  Round-half-up: with the host-side constants (finish_fold_params)
//     A = (y_scale / out_scale) / 255.5        R = (res_scale / out_scale) / 255.5
//     C = (out_zp + 0.5 - y_zp * (y_scale / out_scale) - res_zp * (res_scale / out_scale)) / 255.5
//     t = sat(fma(float(q), A, fma(float(r), R, C)))        out = floor(t * 255.5),
// and, when a Relu sits in front of the final QuantizeLinear, out = max(out, out_zp) (the Relu of the sum is the clamp of the
// quantized value at the zero point).  Round-half-to-even: v = fma(r - res_zp, res_scale / out_scale, (q - y_zp) * (y_scale /
// out_scale)), Relu, rint(v) + out_zp, saturated.
__device__ __forceinline__ int residual_fold(int q, int r, const RequantParams& p) {
    if (p.round_mode != 0) {
        const float u = __fmul_rn(__fsub_rn((float)q, p.y_zp_f), p.y_over_out);
        float v = __fmaf_rn(__fsub_rn((float)r, p.res_zp_f), p.res_over_out, u);
        if (p.res_relu) v = fmaxf(v, 0.f);
        return cvt_rne_sat_u8(__fadd_rn(rintf(v), p.out_zp_f));
    }
    const float t = __saturatef(__fmaf_rn((float)q, p.fold_a, __fmaf_rn((float)r, p.fold_r, p.fold_c)));
    int o = fold_place(t, 255.5f);
    if (p.res_relu) o = max(o, (int)p.out_zp_f);
    return o;
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
// than the int -> float of the accumulator; equals requant_one / residual_one (reference operation order, fold == 0) bit for
// bit; fold != 0 is requant_u8_fold / residual_fold.  Returns the output byte.
__device__ __forceinline__ uint32_t requant_u8_up_fast(int acc, int bias, float mult, bool has_res, uint32_t res_byte, const RequantParams& p) {
    const float hi_ph = (p.clamp_hi_q >= 0 ? (float)p.clamp_hi_q : 255.f) + 0.5f;
    if (p.fold) {
        int q = requant_u8_fold(acc, bias, __fdiv_rn(mult, p.y_scale), p);
        if (has_res) q = residual_fold(q, (int)(res_byte & 0xffu), p);
        return (uint32_t)q;
    }
    float tp = qdiv(__fmul_rn((float)(int)((unsigned)acc + (unsigned)bias), mult), p.y_div);
    tp = __fadd_rn(__fadd_rn(tp, p.y_zp_f), 0.5f);
    float f = quant_u8_up_magic(tp, hi_ph);
    if (has_res) {
        const float u = __fsub_rn(f, __fadd_rn(kMagic23, p.y_zp_f));
        const float w = __fsub_rn(__uint_as_float(0x4B000000u | (res_byte & 0xffu)), __fadd_rn(kMagic23, p.res_zp_f));
        float v = __fadd_rn(__fmul_rn(u, p.y_scale), __fmul_rn(w, p.res_scale));
        if (p.res_relu) v = fmaxf(v, 0.f);
        v = __fadd_rn(__fadd_rn(qdiv(v, p.out_div), p.out_zp_f), 0.5f);
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
