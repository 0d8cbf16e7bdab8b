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

}  // namespace chxq
