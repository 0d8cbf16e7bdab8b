/*
 * CPU oracle for chainer-compiler's quantized-inference VM ops.
 *
 * TEST INFRASTRUCTURE ONLY.  This file restates, in plain C, the arithmetic of the
 * reference's op bodies so that the CUDA kernels can be checked against it.  It is
 * never linked into, imported by or called from the product library; only the test
 * suite, the smoke check and the bench's CPU-baseline leg may use it.
 *
 * PARITY UNPINNED: the reference pins these ops only through ONNX backend node tests
 * whose data directory (third_party/onnx) is an empty submodule in the reference
 * checkout, and the reference itself cannot be built (ChainerX, ONNX and protobuf are
 * absent).  The functions below are therefore a by-specification restatement of the
 * reference sources cited next to each one, cross-checked against an independent
 * int64/float64 numpy formulation in the test suite.
 *
 * Layouts follow the reference: activations NCHW, weights OIHW, matrices row-major.
 * All float arithmetic is IEEE fp32 unless a function says otherwise; the file must be
 * compiled without -ffast-math and with -ffp-contract=off so that a*b+c is two roundings,
 * as it is in ChainerX's elementwise kernels.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_ROUND_REF_HALF_UP 0 /* (t + 0.5f) then C truncation: runtime/ops/quantize.cc:33-34 */
#define ORC_ROUND_RNE 1         /* ONNX: saturate(rint(x/s) + zp) */

int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void orc_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* One element of quantize_array (runtime/ops/quantize.cc:16-35).
 * out_signed selects int8 limits (-128,127) instead of uint8 (0,255), as the dtype of
 * y_zero_point does at :19-25.  Returns the value as int (already in range). */
static inline int quantize_one(float x, float scale, int zp, int out_signed, int round_mode) {
    const float lo = out_signed ? -128.f : 0.f;
    const float hi = out_signed ? 127.f : 255.f;
    if (round_mode == ORC_ROUND_RNE) {
        float r = nearbyintf(x / scale) + (float)zp;
        r = fminf(r, hi);
        r = fmaxf(lo, r);
        return (int)r;
    }
    float t = x / scale;               /* :29  y / Scalar(y_scale)            */
    if (zp != 0) t = t + (float)zp;    /* :30-32                              */
    t = t < hi ? t : hi;               /* :34  Minimum(scaled, max)           */
    t = lo > t ? lo : t;               /* :34  Maximum(min, .)                */
    t = t + 0.5f;                      /* :34  + 0.5f                         */
    return (int)t;                     /* :34  AsType = C++ static_cast       */
}

/* QuantizeLinearOp::RunImpl, runtime/ops/quantize.cc:48-53. */
void orc_quantize_linear(const float* x, int64_t n, float scale, int zp, int out_signed, int round_mode, void* y) {
    uint8_t* yu = (uint8_t*)y;
    int8_t* ys = (int8_t*)y;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        int q = quantize_one(x[i], scale, zp, out_signed, round_mode);
        if (out_signed)
            ys[i] = (int8_t)q;
        else
            yu[i] = (uint8_t)q;
    }
}

/* Count of elements where the reference rounding and round-half-to-even disagree. */
int64_t orc_quantize_mode_diff(const float* x, int64_t n, float scale, int zp, int out_signed) {
    int64_t cnt = 0;
#pragma omp parallel for schedule(static) reduction(+ : cnt)
    for (int64_t i = 0; i < n; ++i) {
        cnt += quantize_one(x[i], scale, zp, out_signed, ORC_ROUND_REF_HALF_UP) !=
               quantize_one(x[i], scale, zp, out_signed, ORC_ROUND_RNE);
    }
    return cnt;
}

/* dequantize_array, runtime/ops/quantize.cc:37-44. */
static inline float dequantize_one(int q, float scale, int zp) {
    float v = (float)q;
    if (zp != 0) v = v - (float)zp;
    return v * scale;
}

/* DequantizeLinearOp::RunImpl, runtime/ops/quantize.cc:55-60. */
void orc_dequantize_linear(const void* x, int x_signed, int64_t n, float scale, int zp, float* y) {
    const uint8_t* xu = (const uint8_t*)x;
    const int8_t* xs = (const int8_t*)x;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        int q = x_signed ? (int)xs[i] : (int)xu[i];
        y[i] = dequantize_one(q, scale, zp);
    }
}

static inline int load_q(const void* p, int is_signed, int64_t i) {
    return is_signed ? (int)((const int8_t*)p)[i] : (int)((const uint8_t*)p)[i];
}

/* MatMulIntegerOp::RunImpl, runtime/ops/quantize.cc:96-114 with NumpyMatMul
 * (runtime/chainerx_util.cc:210-230) for equal leading dims.
 * a: [batch, M, K], b: [batch, K, N], y: int32 [batch, M, N].
 * Zero points are subtracted by numpy broadcasting, so a 1-D zero point aligns with the
 * LAST axis of its operand: a_zp has length 0 (absent), 1 or K; b_zp has length 0, 1 or N.
 * The product wraps in int32 like ChainerX's int32 Dot. */
void orc_matmul_integer(
        const void* a, int a_signed, const void* b, int b_signed, int64_t batch, int64_t M, int64_t N, int64_t K,
        const int32_t* a_zp, int64_t a_zp_len, const int32_t* b_zp, int64_t b_zp_len, int32_t* y) {
    for (int64_t bt = 0; bt < batch; ++bt) {
        const int64_t ao = bt * M * K, bo = bt * K * N, yo = bt * M * N;
#pragma omp parallel
        {
            int32_t* arow = (int32_t*)malloc(sizeof(int32_t) * (size_t)K);
            uint32_t* acc = (uint32_t*)malloc(sizeof(uint32_t) * (size_t)N);
#pragma omp for schedule(static)
            for (int64_t m = 0; m < M; ++m) {
                for (int64_t k = 0; k < K; ++k) {
                    int32_t za = a_zp_len == 0 ? 0 : (a_zp_len == 1 ? a_zp[0] : a_zp[k]);
                    arow[k] = load_q(a, a_signed, ao + m * K + k) - za;
                }
                memset(acc, 0, sizeof(uint32_t) * (size_t)N);
                for (int64_t k = 0; k < K; ++k) {
                    const uint32_t av = (uint32_t)arow[k];
                    if (b_zp_len == 0) {
                        for (int64_t n = 0; n < N; ++n) acc[n] += av * (uint32_t)load_q(b, b_signed, bo + k * N + n);
                    } else {
                        for (int64_t n = 0; n < N; ++n) {
                            int32_t zb = b_zp_len == 1 ? b_zp[0] : b_zp[n];
                            acc[n] += av * (uint32_t)(load_q(b, b_signed, bo + k * N + n) - zb);
                        }
                    }
                }
                for (int64_t n = 0; n < N; ++n) y[yo + m * N + n] = (int32_t)acc[n];
            }
            free(arow);
            free(acc);
        }
    }
}

/* Convolution geometry: ComplementStride/Pad (runtime/chainerx_util.cc:180-200),
 * CalculateAutoPad (:276-311), output size of chainerx::Conv with cover_all=false.
 * strides/pads may be empty (n_strides/n_pads == 0) -> 1 / 0.  pads holds one value per
 * spatial dim (the emitter requires begin == end: compiler/chxvm/simple_node_emitter.cc:76-86).
 * auto_pad is "" or "SAME_UPPER".  Writes {sh, sw, pad_top, pad_left, pad_bottom, pad_right, Ho, Wo}.
 * Returns 0, or -1 for an unsupported auto_pad / empty output. */
int orc_conv_geometry(
        int64_t H, int64_t W, int64_t KH, int64_t KW, const int64_t* strides, int n_strides, const int64_t* pads, int n_pads,
        const char* auto_pad, int64_t out[8]) {
    int64_t sh = n_strides ? strides[0] : 1, sw = n_strides ? strides[1] : 1;
    int64_t pt = n_pads ? pads[0] : 0, pl = n_pads ? pads[1] : 0;
    int64_t pb = pt, pr = pl;
    if (auto_pad && auto_pad[0]) {
        if (strcmp(auto_pad, "SAME_UPPER") != 0) return -1;
        int64_t th = (H + sh - 1) / sh, tw = (W + sw - 1) / sw;
        int64_t nh = (th - 1) * sh + KH - H, nw = (tw - 1) * sw + KW - W;
        /* C++ integer division truncates toward zero, as the reference's does. */
        pt = nh / 2;
        pb = nh - pt;
        pl = nw / 2;
        pr = nw - pl;
        /* :303 only materialises end pads when one of them is positive; otherwise the
         * (possibly negative or zero) begin pads are used on both sides. */
        if (!(pb > 0 || pr > 0)) {
            pb = pt;
            pr = pl;
        }
    }
    int64_t Ho = (H + pt + pb - KH) / sh + 1, Wo = (W + pl + pr - KW) / sw + 1;
    out[0] = sh; out[1] = sw; out[2] = pt; out[3] = pl; out[4] = pb; out[5] = pr; out[6] = Ho; out[7] = Wo;
    if (H + pt + pb < KH || W + pl + pr < KW) return -1;
    return 0;
}

/* ConvIntegerOp::RunImpl, runtime/ops/quantize.cc:116-146 + GroupedConv
 * (runtime/chainerx_util.cc:313-340).  x: [N,C,H,W] (u8 or i8), w: [M,C/group,KH,KW],
 * y: int32 [N,M,Ho,Wo].  x_zp is subtracted BEFORE zero padding (so padding contributes 0
 * in the zero-point-subtracted domain); w_zp has length 0, 1 or M (per output channel). */
void orc_conv_integer(
        const void* x, int x_signed, const void* w, int w_signed, int64_t N, int64_t C, int64_t H, int64_t W, int64_t M, int64_t KH,
        int64_t KW, int64_t sh, int64_t sw, int64_t pt, int64_t pl, int64_t Ho, int64_t Wo, int64_t group, int has_x_zp, int32_t x_zp,
        const int32_t* w_zp, int64_t w_zp_len, int32_t* y) {
    const int64_t Cg = C / group, Mg = M / group;
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        for (int64_t m = 0; m < M; ++m) {
            const int64_t g = m / Mg;
            int32_t* yo = y + (n * M + m) * Ho * Wo;
            for (int64_t i = 0; i < Ho * Wo; ++i) yo[i] = 0;
            const int32_t zw = w_zp_len == 0 ? 0 : (w_zp_len == 1 ? w_zp[0] : w_zp[m]);
            for (int64_t c = 0; c < Cg; ++c) {
                const int64_t xc = (n * C + g * Cg + c) * H * W;
                for (int64_t kh = 0; kh < KH; ++kh) {
                    for (int64_t kw = 0; kw < KW; ++kw) {
                        const uint32_t wv = (uint32_t)(load_q(w, w_signed, ((m * Cg + c) * KH + kh) * KW + kw) - zw);
                        for (int64_t ho = 0; ho < Ho; ++ho) {
                            const int64_t hi = ho * sh - pt + kh;
                            if (hi < 0 || hi >= H) continue;
                            for (int64_t wo = 0; wo < Wo; ++wo) {
                                const int64_t wi = wo * sw - pl + kw;
                                if (wi < 0 || wi >= W) continue;
                                int32_t xv = load_q(x, x_signed, xc + hi * W + wi);
                                if (has_x_zp) xv -= x_zp;
                                yo[ho * Wo + wo] = (int32_t)((uint32_t)yo[ho * Wo + wo] + wv * (uint32_t)xv);
                            }
                        }
                    }
                }
            }
        }
    }
}

/* fp32 convolution used by the QLinearConv emulation: accumulates each output element in
 * (c, kh, kw) order starting from +0.0f, then adds the bias.  ChainerX's own accumulation
 * order is not knowable from the reference checkout; results that depend on it can move a
 * requantized value by one step, which is why the parity bound on QLinearConv is 1 LSB. */
static void conv_f32(
        const float* xf, const float* wf, const float* bias, int64_t N, int64_t C, int64_t H, int64_t W, int64_t M, int64_t KH, int64_t KW,
        int64_t sh, int64_t sw, int64_t pt, int64_t pl, int64_t Ho, int64_t Wo, int64_t group, float* yf) {
    const int64_t Cg = C / group, Mg = M / group;
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        for (int64_t m = 0; m < M; ++m) {
            const int64_t g = m / Mg;
            float* yo = yf + (n * M + m) * Ho * Wo;
            for (int64_t i = 0; i < Ho * Wo; ++i) yo[i] = 0.f;
            for (int64_t c = 0; c < Cg; ++c) {
                const float* xc = xf + (n * C + g * Cg + c) * H * W;
                for (int64_t kh = 0; kh < KH; ++kh) {
                    for (int64_t kw = 0; kw < KW; ++kw) {
                        const float wv = wf[((m * Cg + c) * KH + kh) * KW + kw];
                        for (int64_t ho = 0; ho < Ho; ++ho) {
                            const int64_t hi = ho * sh - pt + kh;
                            if (hi < 0 || hi >= H) continue;
                            int64_t wo0 = 0, wo1 = Wo;
                            /* wi = wo*sw - pl + kw in [0, W) */
                            while (wo0 < Wo && wo0 * sw - pl + kw < 0) ++wo0;
                            while (wo1 > wo0 && (wo1 - 1) * sw - pl + kw >= W) --wo1;
                            const float* xr = xc + hi * W - pl + kw;
                            float* yr = yo + ho * Wo;
                            for (int64_t wo = wo0; wo < wo1; ++wo) yr[wo] = yr[wo] + wv * xr[wo * sw];
                        }
                    }
                }
            }
            if (bias) {
                const float bv = bias[m];
                for (int64_t i = 0; i < Ho * Wo; ++i) yo[i] = yo[i] + bv;
            }
        }
    }
}

#define ORC_BIAS_NONE 0
#define ORC_BIAS_ONNX 1 /* int32 bias with scale x_scale*w_scale[m] (ONNX QLinearConv) */
#define ORC_BIAS_RAW 2  /* the reference hands the int32 values to the fp32 conv unscaled: runtime/ops/quantize.cc:72,93 */

/* QLinearConvOp::RunImpl, runtime/ops/quantize.cc:62-94: dequantize x, dequantize w per
 * output channel (w_params_len == M) or per tensor (w_params_len == 1), fp32 GroupedConv,
 * quantize.  Extensions used by the fused-epilogue parity tests, all off when zero:
 *   clamp_hi_q >= 0 : the quantized output is clamped to at most this value (ReLU6 folded
 *                     into the output range; with y_zp as the lower bound this is Clip(0,6)).
 * y: [N,M,Ho,Wo] u8 or i8. */
void orc_qlinear_conv(
        const void* x, int x_signed, float x_scale, int x_zp, const void* w, int w_signed, const float* w_scale, const int32_t* w_zp,
        int64_t w_params_len, float y_scale, int y_zp, int y_signed, const int32_t* bias, int bias_mode, int64_t N, int64_t C, int64_t H,
        int64_t W, int64_t M, int64_t KH, int64_t KW, int64_t sh, int64_t sw, int64_t pt, int64_t pl, int64_t Ho, int64_t Wo,
        int64_t group, int round_mode, int clamp_hi_q, void* y) {
    const int64_t Cg = C / group;
    const int64_t nx = N * C * H * W, nw = M * Cg * KH * KW, ny = N * M * Ho * Wo;
    float* xf = (float*)malloc(sizeof(float) * (size_t)nx);
    float* wf = (float*)malloc(sizeof(float) * (size_t)nw);
    float* yf = (float*)malloc(sizeof(float) * (size_t)ny);
    float* bf = NULL;
    orc_dequantize_linear(x, x_signed, nx, x_scale, x_zp, xf);
    for (int64_t m = 0; m < M; ++m) {
        const float s = w_params_len == 1 ? w_scale[0] : w_scale[m];
        const int z = w_params_len == 1 ? w_zp[0] : w_zp[m];
        for (int64_t i = 0; i < Cg * KH * KW; ++i) wf[m * Cg * KH * KW + i] = dequantize_one(load_q(w, w_signed, m * Cg * KH * KW + i), s, z);
    }
    if (bias && bias_mode != ORC_BIAS_NONE) {
        bf = (float*)malloc(sizeof(float) * (size_t)M);
        for (int64_t m = 0; m < M; ++m) {
            const float s = w_params_len == 1 ? w_scale[0] : w_scale[m];
            bf[m] = bias_mode == ORC_BIAS_RAW ? (float)bias[m] : (float)bias[m] * (x_scale * s);
        }
    }
    conv_f32(xf, wf, bf, N, C, H, W, M, KH, KW, sh, sw, pt, pl, Ho, Wo, group, yf);
    orc_quantize_linear(yf, ny, y_scale, y_zp, y_signed, round_mode, y);
    if (clamp_hi_q >= 0) {
        if (y_signed) {
            int8_t* p = (int8_t*)y;
            for (int64_t i = 0; i < ny; ++i) p[i] = p[i] > clamp_hi_q ? (int8_t)clamp_hi_q : p[i];
        } else {
            uint8_t* p = (uint8_t*)y;
            for (int64_t i = 0; i < ny; ++i) p[i] = p[i] > clamp_hi_q ? (uint8_t)clamp_hi_q : p[i];
        }
    }
    free(xf);
    free(wf);
    free(yf);
    free(bf);
}

/* The requantization the integer-domain kernels apply to an exact int32 accumulator
 * acc = sum (x - x_zp)(w - w_zp[m]) (+ bias[m]):  yf = float(acc) * (x_scale * w_scale[m]);
 * y = quantize(yf; y_scale, y_zp).  It is the QLinearConv / QLinearMatMul arithmetic of the
 * reference with the fp32 products and sums replaced by their exact integer value, so it
 * agrees with orc_qlinear_conv except where fp32 accumulation error crosses a rounding
 * boundary.  acc: [rows, M] (channel is the LAST axis) or, when chan_stride > 1, NCHW with
 * chan_stride = Ho*Wo: channel of element i = (i / chan_stride) % M. */
/* fold != 0 is the library's optional folded form for uint8 outputs (no counterpart in the reference; restated here so that
 * the kernels implementing it can be checked bit for bit).  Per channel M = (x_scale * w_scale[c]) / y_scale.
 * Round-half-up: values run in units of the output range hp = hi + 0.5 (hi = 255 or the upper clamp):
 *   B = fma(float(bias), M, zp + 0.5);  Ms = M / hp;  Bs = B / hp;
 *   t = min(max(fma(float(acc), Ms, Bs), 0), 1);  y = floor(t * hp)   (exact product, one floor).
 * Round-half-to-even: B = fma(float(bias), M, zp); y = clamp(rint(fma(float(acc), M, B)), 0, hi). */
static inline int fold_place(float t, float hp) {
    if (!(t > 0.f)) t = 0.f; /* also NaN */
    if (t > 1.f) t = 1.f;
    return (int)floor((double)t * (double)hp); /* 24 x 24 bits: exact in double */
}

static inline int fold_quantize_u8(int32_t acc, int32_t bias, float M, int zp, int round_mode, int clamp_hi_q) {
    if (round_mode == ORC_ROUND_RNE) {
        const float B = fmaf((float)bias, M, (float)zp);
        float t = nearbyintf(fmaf((float)acc, M, B));
        t = fminf(t, 255.f);
        t = fmaxf(0.f, t);
        int q = (int)t;
        if (clamp_hi_q >= 0 && q > clamp_hi_q) q = clamp_hi_q;
        return q;
    }
    const float hp = (clamp_hi_q >= 0 ? (float)clamp_hi_q : 255.f) + 0.5f;
    const float B = fmaf((float)bias, M, (float)zp + 0.5f);
    const float Ms = M / hp, Bs = B / hp;
    return fold_place(fmaf((float)acc, Ms, Bs), hp);
}

static inline int quantize_prescaled_u8(float v, int zp, int round_mode) {
    float t = round_mode == ORC_ROUND_RNE ? nearbyintf(v) + (float)zp : floorf(v + ((float)zp + 0.5f));
    t = fminf(t, 255.f);
    t = fmaxf(0.f, t);
    return (int)t;
}

void orc_requantize(
        const int32_t* acc, int64_t n, int64_t M, int64_t chan_stride, float x_scale, const float* w_scale, int64_t w_params_len,
        const int32_t* bias, float y_scale, int y_zp, int y_signed, int round_mode, int clamp_hi_q, int fold, void* y) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        const int64_t m = (i / chan_stride) % M;
        const float mult = x_scale * (w_params_len == 1 ? w_scale[0] : w_scale[m]);
        const int32_t a = (int32_t)((uint32_t)acc[i] + (uint32_t)(bias ? bias[m] : 0));
        if (fold) {
            ((uint8_t*)y)[i] = (uint8_t)fold_quantize_u8(acc[i], bias ? bias[m] : 0, mult / y_scale, y_zp, round_mode, clamp_hi_q);
            continue;
        }
        const float yf = (float)a * mult;
        int q = quantize_one(yf, y_scale, y_zp, y_signed, round_mode);
        if (clamp_hi_q >= 0 && q > clamp_hi_q) q = clamp_hi_q;
        if (y_signed)
            ((int8_t*)y)[i] = (int8_t)q;
        else
            ((uint8_t*)y)[i] = (uint8_t)q;
    }
}

/* fp32 row-major matmul accumulating over k in ascending order. */
static void matmul_f32(const float* a, const float* b, int64_t M, int64_t N, int64_t K, float* y) {
#pragma omp parallel for schedule(static)
    for (int64_t m = 0; m < M; ++m) {
        float* yr = y + m * N;
        for (int64_t n = 0; n < N; ++n) yr[n] = 0.f;
        for (int64_t k = 0; k < K; ++k) {
            const float av = a[m * K + k];
            const float* br = b + k * N;
            for (int64_t n = 0; n < N; ++n) yr[n] = yr[n] + av * br[n];
        }
    }
}

/* QLinearMatMul as the reference executes it: ReplaceQLinearMatMul
 * (compiler/simplifier.cc:675-694) expands it to DequantizeLinear(a), DequantizeLinear(b),
 * MatMul (fp32), QuantizeLinear(y) with scalar parameters. */
void orc_qlinear_matmul(
        const void* a, int a_signed, float a_scale, int a_zp, const void* b, int b_signed, float b_scale, int b_zp, float y_scale, int y_zp,
        int y_signed, int64_t M, int64_t N, int64_t K, int round_mode, void* y) {
    float* af = (float*)malloc(sizeof(float) * (size_t)(M * K));
    float* bf = (float*)malloc(sizeof(float) * (size_t)(K * N));
    float* yf = (float*)malloc(sizeof(float) * (size_t)(M * N));
    orc_dequantize_linear(a, a_signed, M * K, a_scale, a_zp, af);
    orc_dequantize_linear(b, b_signed, K * N, b_scale, b_zp, bf);
    matmul_f32(af, bf, M, N, K, yf);
    orc_quantize_linear(yf, M * N, y_scale, y_zp, y_signed, round_mode, y);
    free(af);
    free(bf);
    free(yf);
}

/* QuantizeData, compiler/quantize.cc:70-89.  to_int8 != 0: symmetric ("Linear_Scaled"),
 * scale = max(|rmin|,|rmax|) * 2 / 254, q = rint(w / scale) with the division in fp32 and the
 * rint in fp64 (SlowRound, runtime/chainerx_util.cc:397-410), zero point 0.  Otherwise
 * asymmetric uint8: scale = (rmax - rmin) / 255 (1 if equal), zp = rint((0 - rmin) / scale),
 * q = rint(w / scale) + zp, cast by truncation.  rmin/rmax always include 0 (:71-72). */
void orc_quantize_data(const float* w, int64_t n, int to_int8, void* q, float* scale_out, int32_t* zp_out) {
    float rmin = 0.f, rmax = 0.f;
    for (int64_t i = 0; i < n; ++i) {
        rmin = w[i] < rmin ? w[i] : rmin;
        rmax = w[i] > rmax ? w[i] : rmax;
    }
    if (to_int8) {
        const float max_range = fmaxf(fabsf(rmin), fabsf(rmax));
        const float scale = max_range * 2 / 254.f;
        for (int64_t i = 0; i < n; ++i) ((int8_t*)q)[i] = (int8_t)(float)rint((double)(w[i] / scale));
        *scale_out = scale;
        *zp_out = 0;
    } else {
        const float scale = rmin != rmax ? (rmax - rmin) / 255.f : 1.f;
        const int64_t zp = (int64_t)rint((double)((0 - rmin) / scale));
        for (int64_t i = 0; i < n; ++i) {
            /* SlowRound(...) + zero_point is a float32 array plus an integer scalar. */
            float v = (float)rint((double)(w[i] / scale)) + (float)zp;
            ((uint8_t*)q)[i] = (uint8_t)v;
        }
        *scale_out = scale;
        *zp_out = (int32_t)zp;
    }
}

/* QuantizeWeightConvolution, compiler/quantize.cc:98-129: per-output-channel QuantizeData
 * over w[m] (axis 0).  w: [M, inner]. */
void orc_quantize_weight_per_channel(const float* w, int64_t M, int64_t inner, int to_int8, void* q, float* scales, int32_t* zps) {
    for (int64_t m = 0; m < M; ++m) {
        orc_quantize_data(w + m * inner, inner, to_int8, (char*)q + m * inner, scales + m, zps + m);
    }
}

/* Dynamic activation parameters emitted by QuantizeInputs, compiler/quantize.cc:172-202,
 * for the uint8 ("Linear_NonScaled") input type: scale = (max - min) / 255,
 * zp = cast_u8(floor((0 - min) / scale)).  min/max are NOT widened to include 0 here.
 * Returns the float zero point before the cast so that callers can see out-of-range cases. */
void orc_dynamic_params_u8(const float* x, int64_t n, float* scale_out, float* zp_float_out) {
    float mn = x[0], mx = x[0];
    for (int64_t i = 1; i < n; ++i) {
        mn = x[i] < mn ? x[i] : mn;
        mx = x[i] > mx ? x[i] : mx;
    }
    const float scale = (mx - mn) / 255.f;
    *scale_out = scale;
    *zp_float_out = floorf((0.f - mn) / scale);
}

/* Fused elementwise groups (compiler/nvrtc_builder.cc:35-87, :118-137).  A group is a list
 * of nodes in topological order; value ids 0..n_inputs-1 are the group inputs, node j
 * defines value n_inputs + j.  Each node is evaluated as its own fp32 pass, which is what
 * the reference's CPU path does when it inlines a group (compiler/chxvm/emitter.cc:702-726).
 * Sigmoid uses the generated kernel's formula tanh(x*0.5)*0.5+0.5 (nvrtc_builder.cc:133-136). */
enum {
    ORC_EW_IDENTITY = 0,
    ORC_EW_TANH = 1,
    ORC_EW_EXP = 2,
    ORC_EW_SIGMOID = 3,
    ORC_EW_ADD = 4,
    ORC_EW_SUB = 5,
    ORC_EW_MUL = 6,
    ORC_EW_DIV = 7,
    ORC_EW_CONST = 8
};

typedef struct {
    int32_t op;
    int32_t in0, in1;
    float cval;
} orc_ew_node;

void orc_eltwise_f32(
        const orc_ew_node* nodes, int n_nodes, const float* const* inputs, int n_inputs, int64_t n, const int32_t* out_ids, int n_outputs,
        float* const* outputs) {
    float** vals = (float**)calloc((size_t)(n_inputs + n_nodes), sizeof(float*));
    for (int i = 0; i < n_inputs; ++i) vals[i] = (float*)inputs[i];
    for (int j = 0; j < n_nodes; ++j) {
        float* o = (float*)malloc(sizeof(float) * (size_t)n);
        vals[n_inputs + j] = o;
        const orc_ew_node nd = nodes[j];
        const float* a = nd.op == ORC_EW_CONST ? NULL : vals[nd.in0];
        const float* b = nd.op >= ORC_EW_ADD && nd.op <= ORC_EW_DIV ? vals[nd.in1] : NULL;
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < n; ++i) {
            switch (nd.op) {
                case ORC_EW_IDENTITY: o[i] = a[i]; break;
                case ORC_EW_TANH: o[i] = tanhf(a[i]); break;
                case ORC_EW_EXP: o[i] = expf(a[i]); break;
                case ORC_EW_SIGMOID: o[i] = tanhf(a[i] * 0.5f) * 0.5f + 0.5f; break;
                case ORC_EW_ADD: o[i] = a[i] + b[i]; break;
                case ORC_EW_SUB: o[i] = a[i] - b[i]; break;
                case ORC_EW_MUL: o[i] = a[i] * b[i]; break;
                case ORC_EW_DIV: o[i] = a[i] / b[i]; break;
                default: o[i] = nd.cval; break;
            }
        }
    }
    for (int k = 0; k < n_outputs; ++k) memcpy(outputs[k], vals[out_ids[k]], sizeof(float) * (size_t)n);
    for (int j = 0; j < n_nodes; ++j) free(vals[n_inputs + j]);
    free(vals);
}

/* Same DAG evaluated in fp64 end to end: the "truth" the 1e-5 relative bound is taken
 * against, since neither fp32 sigmoid formula is privileged. */
void orc_eltwise_f64(
        const orc_ew_node* nodes, int n_nodes, const float* const* inputs, int n_inputs, int64_t n, const int32_t* out_ids, int n_outputs,
        double* const* outputs) {
#pragma omp parallel
    {
        double* v = (double*)malloc(sizeof(double) * (size_t)(n_inputs + n_nodes));
#pragma omp for schedule(static)
        for (int64_t i = 0; i < n; ++i) {
            for (int k = 0; k < n_inputs; ++k) v[k] = (double)inputs[k][i];
            for (int j = 0; j < n_nodes; ++j) {
                const orc_ew_node nd = nodes[j];
                double a = nd.op == ORC_EW_CONST ? 0.0 : v[nd.in0];
                double b = nd.op >= ORC_EW_ADD && nd.op <= ORC_EW_DIV ? v[nd.in1] : 0.0;
                double r;
                switch (nd.op) {
                    case ORC_EW_IDENTITY: r = a; break;
                    case ORC_EW_TANH: r = tanh(a); break;
                    case ORC_EW_EXP: r = exp(a); break;
                    case ORC_EW_SIGMOID: r = 1.0 / (1.0 + exp(-a)); break;
                    case ORC_EW_ADD: r = a + b; break;
                    case ORC_EW_SUB: r = a - b; break;
                    case ORC_EW_MUL: r = a * b; break;
                    case ORC_EW_DIV: r = a / b; break;
                    default: r = (double)nd.cval; break;
                }
                v[n_inputs + j] = r;
            }
            for (int k = 0; k < n_outputs; ++k) outputs[k][i] = v[out_ids[k]];
        }
        free(v);
    }
}

/* ---- fp32 glue ops a quantized CNN graph runs between the int8 ops (reference bodies are
 * one-line ChainerX calls: runtime/ops/activation.cc:20-22 Relu, pooling.cc:47-75 MaxPool /
 * AveragePool, connection.cc:12-15 Linear, math.cc:31-33 Add). Restated for NCHW. ---- */

/* MaxPool over uint8/int8 or float NCHW; cover_all adds the partial windows at the end
 * (Chainer's max_pooling_2d default, used by the ResNet-50 definition scripts/resnet50.py:97). */
void orc_maxpool_u8(
        const uint8_t* x, int64_t N, int64_t C, int64_t H, int64_t W, int64_t k, int64_t s, int64_t p, int64_t Ho, int64_t Wo, uint8_t* y) {
#pragma omp parallel for schedule(static)
    for (int64_t nc = 0; nc < N * C; ++nc) {
        for (int64_t ho = 0; ho < Ho; ++ho)
            for (int64_t wo = 0; wo < Wo; ++wo) {
                int best = 0;
                for (int64_t kh = 0; kh < k; ++kh)
                    for (int64_t kw = 0; kw < k; ++kw) {
                        int64_t hi = ho * s - p + kh, wi = wo * s - p + kw;
                        if (hi < 0 || hi >= H || wi < 0 || wi >= W) continue;
                        int v = x[nc * H * W + hi * W + wi];
                        best = v > best ? v : best;
                    }
                y[nc * Ho * Wo + ho * Wo + wo] = (uint8_t)best;
            }
    }
}

/* Global average pool of a dequantized uint8 map: mean over H*W of (q - zp) * scale, with
 * the sum taken exactly in integers and one fp32 divide, then the scale. */
void orc_global_avgpool_dq(const uint8_t* x, int64_t N, int64_t C, int64_t HW, float scale, int zp, float* y) {
#pragma omp parallel for schedule(static)
    for (int64_t nc = 0; nc < N * C; ++nc) {
        int64_t s = 0;
        for (int64_t i = 0; i < HW; ++i) s += (int)x[nc * HW + i] - zp;
        y[nc] = ((float)s / (float)HW) * scale;
    }
}

/* Linear / Gemm: y[n, o] = sum_k x[n,k] * w[o,k] + b[o], fp32, k ascending, each step a fused multiply-add (the
 * accumulation order inside ChainerX's Dot is not knowable from the reference checkout; this is the library's). */
void orc_linear_f32(const float* x, const float* w, const float* b, int64_t N, int64_t K, int64_t O, float* y) {
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t n = 0; n < N; ++n)
        for (int64_t o = 0; o < O; ++o) {
            float acc = 0.f;
            for (int64_t k = 0; k < K; ++k) acc = fmaf(x[n * K + k], w[o * K + k], acc);
            y[n * O + o] = acc + (b ? b[o] : 0.f);
        }
}

/* The library's folded residual tail (see orc_requantize, fold), a = the convolution's own output, b = the residual.
 * Round-half-up, in units of the output range: ka = a_scale / y_scale, kb = b_scale / y_scale (fp32),
 *   A = ka / 255.5;  R = kb / 255.5;  C = float((y_zp + 0.5 - a_zp * ka - b_zp * kb) / 255.5) evaluated in double;
 *   t = min(max(fma(float(a), A, fma(float(b), R, C)), 0), 1);  y = floor(t * 255.5);  Relu: y = max(y, y_zp).
 * Round-half-to-even: v = fma(b - b_zp, kb, (a - a_zp) * ka), Relu, rint(v) + y_zp, saturated. */
void orc_qadd_relu_fold(
        const uint8_t* a, float a_scale, int a_zp, const uint8_t* b, float b_scale, int b_zp, int64_t n, float y_scale, int y_zp, int relu,
        int round_mode, uint8_t* y) {
    const float ka = a_scale / y_scale, kb = b_scale / y_scale;
    const float A = ka / 255.5f, R = kb / 255.5f;
    const float C = (float)((((double)y_zp + 0.5) - (double)a_zp * (double)ka - (double)b_zp * (double)kb) / 255.5);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        if (round_mode == ORC_ROUND_RNE) {
            const float u = ((float)a[i] - (float)a_zp) * ka;
            float v = fmaf((float)b[i] - (float)b_zp, kb, u);
            if (relu) v = v > 0.f ? v : 0.f;
            y[i] = (uint8_t)quantize_prescaled_u8(v, y_zp, round_mode);
            continue;
        }
        int q = fold_place(fmaf((float)a[i], A, fmaf((float)b[i], R, C)), 255.5f);
        if (relu && q < y_zp) q = y_zp;
        y[i] = (uint8_t)q;
    }
}

/* Residual join of two quantized maps as the reference graph runs it:
 * DequantizeLinear(a), DequantizeLinear(b), Add, Relu, QuantizeLinear. */
void orc_qadd_relu(
        const uint8_t* a, float a_scale, int a_zp, const uint8_t* b, float b_scale, int b_zp, int64_t n, float y_scale, int y_zp, int relu,
        int round_mode, uint8_t* y) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        float v = dequantize_one(a[i], a_scale, a_zp) + dequantize_one(b[i], b_scale, b_zp);
        if (relu) v = v > 0.f ? v : 0.f;
        y[i] = (uint8_t)quantize_one(v, y_scale, y_zp, 0, round_mode);
    }
}
