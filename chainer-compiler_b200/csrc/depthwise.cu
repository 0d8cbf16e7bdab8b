// Depthwise QLinearConv (group == C == M) on NHWC u8/s8 maps: HBM-bound, so the kernel is built
// around moving each byte once.  A CTA owns an 8x8 tile of output positions x 64 channels; the input
// halo tile is staged into shared memory with 128-bit loads (positions in the convolution's padding
// are filled with the activation zero point, i.e. 0 after zero-point subtraction, which is where the
// reference pads: runtime/ops/quantize.cc:65-72 dequantizes before chainerx::Conv zero-pads), the
// per-channel taps are staged as 32-bit (w - w_zp), every thread accumulates 16 channels of one position in registers
// (one byte permute and one integer multiply-add per tap and channel) and stores one 128-bit word of requantized output.
//
// The reference runs this as `group` separate fp32 convolutions plus a concatenate
// (runtime/chainerx_util.cc:328-339): 960 launches for one MobileNetV2 layer.
#include "common.h"
#include "kernels.h"

namespace chxq {
namespace {

constexpr int kTH = 8, kTW = 8, kCC = 64;
constexpr int kMaxTaps = 25;  // up to 5x5

struct DwDesc {
    int N, C, H, W, KH, KW, sh, sw, pt, pl, Ho, Wo;
    int x_cs, y_cs;
    int x_signed, w_signed;
    int x_zp;
    int64_t w_zp_len;
    int tiles_w;
};

// Byte `sel` of word w, zero- or sign-extended, in one permute: prmt's selector nibble n picks byte n of {w, 0}; with
// bit 3 of the nibble set it replicates that byte's sign bit instead.
template <bool kSigned>
__device__ __forceinline__ int byte_of(uint32_t w, int sel) {
    const uint32_t s8 = 8u | (uint32_t)sel;
    const uint32_t selector = kSigned ? ((uint32_t)sel | (s8 << 4) | (s8 << 8) | (s8 << 12)) : (0x4440u | (uint32_t)sel);
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(w), "r"(0u), "r"(selector));
    return (int)d;
}

template <bool kXSigned>
__global__ void __launch_bounds__(256) depthwise_kernel(
        const uint8_t* __restrict__ x, const void* __restrict__ w, const void* __restrict__ w_zp, DwDesc d, EpiArgs epi, uint8_t* __restrict__ y) {
    extern __shared__ __align__(16) uint8_t smem[];
    const int IH = (kTH - 1) * d.sh + d.KH, IW = (kTW - 1) * d.sw + d.KW;
    const int taps = d.KH * d.KW;
    uint8_t* s_in = smem;                                                     // [IH][IW][64] bytes
    int* s_w = reinterpret_cast<int*>(smem + ((IH * IW * kCC + 15) & ~15));  // [taps][64]: w - w_zp
    int* s_wsum = s_w + taps * kCC;                                          // [64]: sum over taps of (w - w_zp)

    const int tile = blockIdx.x;
    const int th = tile / d.tiles_w, tw = tile % d.tiles_w;
    const int c0 = blockIdx.y * kCC;
    const int n = blockIdx.z;
    const int ho0 = th * kTH, wo0 = tw * kTW;
    const int hi0 = ho0 * d.sh - d.pt, wi0 = wo0 * d.sw - d.pl;
    const int tid = threadIdx.x;

    // Stage the taps of this channel block as 32-bit (w - w_zp).
    for (int i = tid; i < taps * kCC; i += 256) {
        const int c = i % kCC, tap = i / kCC;
        int v = 0;
        if (c0 + c < d.C) {
            const int64_t wi = (int64_t)(c0 + c) * taps + tap;
            v = d.w_signed ? (int)static_cast<const int8_t*>(w)[wi] : (int)static_cast<const uint8_t*>(w)[wi];
            if (d.w_zp_len > 0) {
                const int64_t zi = d.w_zp_len == 1 ? 0 : (c0 + c);
                v -= d.w_signed ? (int)static_cast<const int8_t*>(w_zp)[zi] : (int)static_cast<const uint8_t*>(w_zp)[zi];
            }
        }
        s_w[i] = v;
    }
    // Stage the input halo tile, 16 channels (one 128-bit word) per load; padding holds the activation zero point.
    const uint32_t padw = (uint32_t)(d.x_zp & 0xff) * 0x01010101u;
    for (int i = tid; i < IH * IW * 4; i += 256) {
        const int cg = i & 3;
        const int p = i >> 2;
        const int iw = p % IW, ih = p / IW;
        const int hi = hi0 + ih, wi = wi0 + iw;
        uint4 v = make_uint4(padw, padw, padw, padw);
        if (hi >= 0 && hi < d.H && wi >= 0 && wi < d.W && c0 + cg * 16 < d.C)
            v = *reinterpret_cast<const uint4*>(x + (((int64_t)n * d.H + hi) * d.W + wi) * d.x_cs + c0 + cg * 16);
        *reinterpret_cast<uint4*>(s_in + (size_t)p * kCC + cg * 16) = v;
    }
    __syncthreads();
    if (tid < kCC) {
        int sum = 0;
        for (int t = 0; t < taps; ++t) sum += s_w[t * kCC + tid];
        s_wsum[tid] = sum;
    }
    __syncthreads();

    const int cg = tid & 3;
    const int p = tid >> 2;
    const int pw = p % kTW, ph = p / kTW;
    const int ho = ho0 + ph, wo = wo0 + pw;
    if (ho >= d.Ho || wo >= d.Wo || c0 + cg * 16 >= d.C) return;

    // acc = sum_taps x_q * (w - w_zp); the activation zero point comes off afterwards as x_zp * sum_taps (w - w_zp)
    // (padding positions hold x_zp, so they cancel exactly).
    int acc[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) acc[j] = 0;
    for (int kh = 0; kh < d.KH; ++kh) {
        for (int kw = 0; kw < d.KW; ++kw) {
            const int ih = ph * d.sh + kh, iw = pw * d.sw + kw;
            const uint4 xv = *reinterpret_cast<const uint4*>(s_in + (size_t)(ih * IW + iw) * kCC + cg * 16);
            const int4* wp = reinterpret_cast<const int4*>(s_w + (kh * d.KW + kw) * kCC + cg * 16);
            const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                const int4 w4 = wp[g];
                acc[4 * g + 0] += byte_of<kXSigned>(xw[g], 0) * w4.x;
                acc[4 * g + 1] += byte_of<kXSigned>(xw[g], 1) * w4.y;
                acc[4 * g + 2] += byte_of<kXSigned>(xw[g], 2) * w4.z;
                acc[4 * g + 3] += byte_of<kXSigned>(xw[g], 3) * w4.w;
            }
        }
    }
    if (d.x_zp != 0) {
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[j] -= d.x_zp * s_wsum[cg * 16 + j];
    }
    const int64_t o = (((int64_t)n * d.Ho + ho) * d.Wo + wo) * d.y_cs + c0 + cg * 16;
    uint32_t resw[4] = {0u, 0u, 0u, 0u};
    if (epi.residual) {
        const uint4 r = *reinterpret_cast<const uint4*>(epi.residual + o);
        resw[0] = r.x; resw[1] = r.y; resw[2] = r.z; resw[3] = r.w;
    }
    const bool fast = !epi.rq.y_signed && epi.rq.round_mode == 0;
    uint32_t outw[4];
#pragma unroll
    for (int wv = 0; wv < 4; ++wv) {
        uint32_t o32 = 0u;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const int j = wv * 4 + b, c = c0 + cg * 16 + j;
            const int bias = epi.bias ? epi.bias[c] : 0;
            const uint32_t rb = (resw[wv] >> (8 * b)) & 0xffu;
            uint32_t q;
            if (fast)
                q = requant_u8_up_fast(acc[j], bias, epi_mult(epi, c), epi.residual != nullptr, rb, epi.rq);
            else
                q = (uint32_t)epi_requant(epi, acc[j], epi_mult(epi, c), bias, (int)rb) & 0xffu;
            o32 |= q << (8 * b);
        }
        outw[wv] = o32;
    }
    *reinterpret_cast<uint4*>(y + o) = make_uint4(outw[0], outw[1], outw[2], outw[3]);
}

// ---- 3x3 depthwise, uint8 activations with zero point 0, symmetric weights: rows of three taps as dp4a --------------------------------
// A thread owns four channels (one 32-bit word of the NHWC map) of one output column and slides down a strip of output rows.  For an
// input row it loads the three words of its window's columns and permutes them into one word PER CHANNEL holding that channel's three
// horizontal neighbours (2 byte permutes per channel; the fourth byte meets a zero weight); a kernel row is then ONE dp4a per channel
// against the word (w[c][kh][0], w[c][kh][1], w[c][kh][2], 0), and the permuted words of an input row serve the three (stride 2: two)
// output rows that read it.  ~12 instructions per output instead of ~25: three dp4a, 2/3 of two permutes, a quarter of three loads and
// one store, and the requantization.  Lanes run along the channels, then the columns, so every load and store is coalesced; the two
// neighbouring columns come out of L1.  Accumulators are exact int32: results equal every other path's.
struct Dw3Desc {
    int N, C, H, W, Ho, Wo, pt, pl;
    int x_cs, y_cs;
    int rows_per_strip, images_per_thread;
    int w_row_stride, w_tap_stride, w_diag;  // weight of (channel c, tap t) at c * w_row_stride + t * w_tap_stride (+ (c & 63) in a diagonal-block pack)
};

template <bool kWSigned>
__device__ __forceinline__ int dot4(uint32_t xw, uint32_t ww, int acc) {
    int d;
    if (kWSigned)
        asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(xw), "r"(ww), "r"(acc));
    else
        asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(xw), "r"(ww), "r"(acc));
    return d;
}

template <int S, bool kWSigned>
__global__ void __launch_bounds__(256) dw3x3_rows_kernel(const uint8_t* __restrict__ x, const uint8_t* __restrict__ w, Dw3Desc d, EpiArgs epi,
                                                         uint8_t* __restrict__ y) {
    const int c4n = d.C >> 2;
    const int idx = blockIdx.x * 256 + threadIdx.x;
    if (idx >= d.Wo * c4n) return;
    const int wo = idx / c4n, cw = idx - wo * c4n;
    const int c0 = cw * 4;
    const int h_begin = blockIdx.y * d.rows_per_strip;
    const int h_end = min(d.Ho, h_begin + d.rows_per_strip);
    // weights: one word per (kernel row, channel)
    uint32_t wr[3][4];
    if (d.w_row_stride == 12 && d.w_tap_stride == 1 && (reinterpret_cast<uintptr_t>(w) & 3u) == 0) {
        // the nine taps of a channel in three aligned words: (t0 t1 t2 t3) (t4 t5 t6 t7) (t8 . . .)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const uint32_t* wc = reinterpret_cast<const uint32_t*>(w + (int64_t)(c0 + c) * 12);
            const uint32_t a = __ldg(wc), b = __ldg(wc + 1), e = __ldg(wc + 2);
            wr[0][c] = a & 0x00ffffffu;
            wr[1][c] = __byte_perm(a, b, 0x4543) & 0x00ffffffu;   // t3 t4 t5
            wr[2][c] = __byte_perm(b, e, 0x4432) & 0x00ffffffu;   // t6 t7 t8
        }
    } else {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const uint8_t* wc = w + (int64_t)(c0 + c) * d.w_row_stride + (d.w_diag ? ((c0 + c) & 63) : 0);
#pragma unroll
            for (int kh = 0; kh < 3; ++kh)
                wr[kh][c] = (uint32_t)wc[(kh * 3) * d.w_tap_stride] | ((uint32_t)wc[(kh * 3 + 1) * d.w_tap_stride] << 8) |
                            ((uint32_t)wc[(kh * 3 + 2) * d.w_tap_stride] << 16);
        }
    }
    // requantization per channel
    const RequantParams rq = epi.rq;
    const bool fold = rq.fold != 0;
    float ms[4], bs[4];
    int bias[4];
    const float hp = fold_hi_ph(rq);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        bias[c] = epi.bias ? epi.bias[c0 + c] : 0;
        ms[c] = epi_mult(epi, c0 + c);
        bs[c] = 0.f;
        if (fold) {
            const FoldCh fc = fold_channel(bias[c], __fdiv_rn(ms[c], rq.y_scale), rq);
            ms[c] = fc.ms;
            bs[c] = fc.bs;
        }
    }
    const int wi0 = wo * S - d.pl;
    const bool in0 = wi0 >= 0 && wi0 < d.W, in1 = wi0 + 1 >= 0 && wi0 + 1 < d.W, in2 = wi0 + 2 >= 0 && wi0 + 2 < d.W;
    const int64_t x_row = (int64_t)d.W * d.x_cs, y_row = (int64_t)d.Wo * d.y_cs;  // bytes between rows
    // small maps: a thread walks several images, so that the set-up above (weights, per-channel requantization) is paid once per ~28 rows
    for (int n = blockIdx.z * d.images_per_thread; n < min(d.N, (int)(blockIdx.z + 1) * d.images_per_thread); ++n) {
    const uint8_t* xn = x + (int64_t)n * d.H * x_row + (int64_t)wi0 * d.x_cs + c0;
    uint8_t* yp = y + ((int64_t)n * d.Ho + h_begin) * y_row + (int64_t)wo * d.y_cs + c0;
    // raw words of an input row's three columns (zeros outside the map: the padding of a zero-point-0 map); fetched one row ahead of
    // their use, so that the loads of the next row are in flight while the current one is worked on
    struct Raw {
        uint32_t x0, x1, x2;
    };
    auto fetch = [&](int hi) {
        Raw r{0u, 0u, 0u};
        if (hi >= 0 && hi < d.H) {
            const uint8_t* row = xn + hi * x_row;
            if (in0) r.x0 = __ldg(reinterpret_cast<const uint32_t*>(row));
            if (in1) r.x1 = __ldg(reinterpret_cast<const uint32_t*>(row + d.x_cs));
            if (in2) r.x2 = __ldg(reinterpret_cast<const uint32_t*>(row + 2 * d.x_cs));
        }
        return r;
    };
    // the four per-channel neighbour words of a row
    auto permute = [&](uint32_t (&r)[4], const Raw& v) {
        r[0] = __byte_perm(__byte_perm(v.x0, v.x1, 0x0040), v.x2, 0x0410);
        r[1] = __byte_perm(__byte_perm(v.x0, v.x1, 0x0051), v.x2, 0x0510);
        r[2] = __byte_perm(__byte_perm(v.x0, v.x1, 0x0062), v.x2, 0x0610);
        r[3] = __byte_perm(__byte_perm(v.x0, v.x1, 0x0073), v.x2, 0x0710);
    };
    auto emit = [&](int ho, const uint32_t (&r0)[4], const uint32_t (&r1)[4], const uint32_t (&r2)[4]) {
        uint32_t q[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            int acc = dot4<kWSigned>(r0[c], wr[0][c], 0);
            acc = dot4<kWSigned>(r1[c], wr[1][c], acc);
            acc = dot4<kWSigned>(r2[c], wr[2][c], acc);
            if (fold)
                q[c] = (uint32_t)fold_place(__saturatef(__fmaf_rn((float)acc, ms[c], bs[c])), hp);
            else
                q[c] = requant_u8_up_fast(acc, bias[c], ms[c], false, 0u, rq);
        }
        const uint32_t word = (q[0] & 0xffu) | ((q[1] & 0xffu) << 8) | ((q[2] & 0xffu) << 16) | (q[3] << 24);
        (void)ho;
        *reinterpret_cast<uint32_t*>(yp) = word;
        yp += y_row;
    };
    uint32_t ra[4], rb[4], rc[4];
    int ho = h_begin;
    if (ho >= h_end) return;
    if (S == 1) {
        const int base = ho - d.pt;  // input row of the first tap of output row h_begin
        Raw v = fetch(base);
        Raw v1 = fetch(base + 1);
        Raw nx = fetch(base + 2);
        permute(ra, v);
        permute(rb, v1);
        int hn = base + 3;  // next input row to fetch
        while (true) {
            permute(rc, nx); nx = fetch(hn++); emit(ho, ra, rb, rc); if (++ho >= h_end) break;
            permute(ra, nx); nx = fetch(hn++); emit(ho, rb, rc, ra); if (++ho >= h_end) break;
            permute(rb, nx); nx = fetch(hn++); emit(ho, rc, ra, rb); if (++ho >= h_end) break;
        }
    } else {
        const int base = 2 * ho - d.pt;
        Raw v = fetch(base);
        Raw p1 = fetch(base + 1), p2 = fetch(base + 2);
        permute(ra, v);
        int hn = base + 3;
        while (true) {
            permute(rb, p1); permute(rc, p2); p1 = fetch(hn); p2 = fetch(hn + 1); hn += 2; emit(ho, ra, rb, rc); if (++ho >= h_end) break;
            permute(ra, p1); permute(rb, p2); p1 = fetch(hn); p2 = fetch(hn + 1); hn += 2; emit(ho, rc, ra, rb); if (++ho >= h_end) break;
            permute(rc, p1); permute(ra, p2); p1 = fetch(hn); p2 = fetch(hn + 1); hn += 2; emit(ho, rb, rc, ra); if (++ho >= h_end) break;
        }
    }
    }  // images
}

}  // namespace

bool depthwise_eligible(const chxq_conv_geom& g, const void* x, const void* y, const void* residual) {
    const int xcs = g.x_cstride > 0 ? g.x_cstride : g.C;
    const int ycs = g.y_cstride > 0 ? g.y_cstride : g.M;
    return g.group == g.C && g.M == g.C && g.x_layout == CHXQ_NHWC && g.y_layout == CHXQ_NHWC && g.C % 16 == 0 && xcs % 16 == 0 && ycs % 16 == 0 &&
           g.KH * g.KW <= kMaxTaps && g.N <= 65535 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0 && (reinterpret_cast<uintptr_t>(y) & 15u) == 0 &&
           (reinterpret_cast<uintptr_t>(residual) & 15u) == 0 && g.stride_h <= 4 && g.stride_w <= 4;
}

int launch_depthwise(
        const void* x, const void* w, const chxq_conv_geom& g, int x_zp, const void* w_zp, int64_t w_zp_len, const EpiArgs& epi, void* y,
        cudaStream_t s) {
    if ((int64_t)g.N * g.Ho * g.Wo == 0) return CHXQ_OK;
    DwDesc d;
    d.N = g.N; d.C = g.C; d.H = g.H; d.W = g.W; d.KH = g.KH; d.KW = g.KW; d.sh = g.stride_h; d.sw = g.stride_w;
    d.pt = g.pad_top; d.pl = g.pad_left; d.Ho = g.Ho; d.Wo = g.Wo;
    d.x_cs = g.x_cstride > 0 ? g.x_cstride : g.C;
    d.y_cs = g.y_cstride > 0 ? g.y_cstride : g.M;
    d.x_signed = g.x_dtype == CHXQ_INT8;
    d.w_signed = g.w_dtype == CHXQ_INT8;
    d.x_zp = x_zp;
    d.w_zp_len = w_zp_len;
    d.tiles_w = (g.Wo + kTW - 1) / kTW;
    const int tiles_h = (g.Ho + kTH - 1) / kTH;
    const int IH = (kTH - 1) * d.sh + d.KH, IW = (kTW - 1) * d.sw + d.KW;
    const size_t smem = ((size_t)(IH * IW * kCC + 15) & ~(size_t)15) + (size_t)g.KH * g.KW * kCC * 4 + kCC * 4;
    dim3 grid((unsigned)(d.tiles_w * tiles_h), (unsigned)((g.C + kCC - 1) / kCC), (unsigned)g.N);
    if (d.x_signed) {
        if (smem > 48 * 1024) CHXQ_CUDA(cudaFuncSetAttribute(depthwise_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        depthwise_kernel<true><<<grid, 256, smem, s>>>(static_cast<const uint8_t*>(x), w, w_zp, d, epi, static_cast<uint8_t*>(y));
    } else {
        if (smem > 48 * 1024) CHXQ_CUDA(cudaFuncSetAttribute(depthwise_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        depthwise_kernel<false><<<grid, 256, smem, s>>>(static_cast<const uint8_t*>(x), w, w_zp, d, epi, static_cast<uint8_t*>(y));
    }
    CHXQ_LAUNCH_CHECK();
    return CHXQ_OK;
}

bool depthwise3x3_eligible(const chxq_conv_geom& g, const void* x, const void* y, int x_zp, const EpiArgs& epi) {
    const int xcs = g.x_cstride > 0 ? g.x_cstride : g.C;
    const int ycs = g.y_cstride > 0 ? g.y_cstride : g.M;
    return g.group == g.C && g.M == g.C && g.KH == 3 && g.KW == 3 && g.stride_h == g.stride_w && (g.stride_h == 1 || g.stride_h == 2) &&
           g.pad_top >= 0 && g.pad_top <= 1 && g.pad_left >= 0 && g.pad_left <= 1 && g.x_layout == CHXQ_NHWC && g.y_layout == CHXQ_NHWC &&
           g.x_dtype == CHXQ_UINT8 && x_zp == 0 && g.C % 4 == 0 && xcs % 4 == 0 && ycs % 4 == 0 && g.N <= 65535 &&
           (reinterpret_cast<uintptr_t>(x) & 3u) == 0 && (reinterpret_cast<uintptr_t>(y) & 3u) == 0 && epi.mode == kEpiRequant &&
           epi.residual == nullptr && !epi.rq.y_signed && epi.rq.round_mode == 0 && (int64_t)g.Wo * (g.C / 4) < (1ll << 31);
}

int launch_depthwise3x3(const void* x, const void* w, int w_row_stride, int w_tap_stride, int w_diag, const chxq_conv_geom& g, const EpiArgs& epi,
                        void* y, cudaStream_t s) {
    if ((int64_t)g.N * g.Ho * g.Wo == 0) return CHXQ_OK;
    Dw3Desc d;
    d.N = g.N; d.C = g.C; d.H = g.H; d.W = g.W; d.Ho = g.Ho; d.Wo = g.Wo; d.pt = g.pad_top; d.pl = g.pad_left;
    d.x_cs = g.x_cstride > 0 ? g.x_cstride : g.C;
    d.y_cs = g.y_cstride > 0 ? g.y_cstride : g.M;
    d.rows_per_strip = g.Ho >= 28 ? 14 : g.Ho;  // two more input rows per strip are read twice (out of L2)
    d.images_per_thread = g.Ho >= 28 ? 1 : (28 + g.Ho - 1) / g.Ho;
    d.w_row_stride = w_row_stride; d.w_tap_stride = w_tap_stride; d.w_diag = w_diag;
    const int words = g.Wo * (g.C / 4);
    dim3 grid((unsigned)((words + 255) / 256), (unsigned)((g.Ho + d.rows_per_strip - 1) / d.rows_per_strip),
              (unsigned)((g.N + d.images_per_thread - 1) / d.images_per_thread));
    const bool ws = g.w_dtype == CHXQ_INT8;
    const uint8_t* xb = static_cast<const uint8_t*>(x);
    const uint8_t* wb = static_cast<const uint8_t*>(w);
    uint8_t* yb = static_cast<uint8_t*>(y);
    if (g.stride_h == 1) {
        if (ws) dw3x3_rows_kernel<1, true><<<grid, 256, 0, s>>>(xb, wb, d, epi, yb);
        else dw3x3_rows_kernel<1, false><<<grid, 256, 0, s>>>(xb, wb, d, epi, yb);
    } else {
        if (ws) dw3x3_rows_kernel<2, true><<<grid, 256, 0, s>>>(xb, wb, d, epi, yb);
        else dw3x3_rows_kernel<2, false><<<grid, 256, 0, s>>>(xb, wb, d, epi, yb);
    }
    CHXQ_LAUNCH_CHECK();
    return CHXQ_OK;
}

}  // namespace chxq
