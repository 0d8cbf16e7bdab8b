// Depthwise QLinearConv (group == C == M) on NHWC u8/s8 maps: HBM-bound work, so the kernels are built around moving each byte once.
// Three kernels:
//   depthwise_kernel      any kernel size up to 5x5, strides up to 4, either operand type, zero points, residual tail.  A CTA owns an
//                         8x8 tile of output positions x 64 channels; the input halo tile is staged into shared memory with 128-bit loads
//                         (positions in the convolution's padding are filled with the activation zero point, i.e. 0 after zero-point
//                         subtraction, which is where the reference pads: runtime/ops/quantize.cc:65-72 dequantizes before
//                         chainerx::Conv zero-pads), the per-channel taps are staged as 32-bit (w - w_zp), every thread accumulates 16
//                         channels of one position in registers and stores one 128-bit word of requantized output.
//   dw3x3_rows_kernel     3x3, stride 1 or 2, uint8 map with zero point 0, symmetric weights: a row of three taps is one dp4a; plain
//                         loads (any channel count that is a multiple of four).
//   dw3x3_staged_kernel   the same arithmetic with the input rows streamed through shared memory by TMA (16-byte aligned maps); two
//                         output columns per thread at stride 1.  The one MobileNetV2's layers run on.
// All three accumulate exact int32 sums and share the requantization of every other convolution path, so their outputs are identical.
//
// The reference runs a depthwise layer as `group` separate fp32 convolutions plus a concatenate
// (runtime/chainerx_util.cc:328-339): 960 launches for one MobileNetV2 layer.
#include <algorithm>

#include "common.h"
#include "kernels.h"
#include "tc_kernel.cuh"

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

// What a thread keeps for its four channels: the taps as one word per (kernel row, channel) and the requantization per channel.
template <bool kWSigned>
struct Dw3Lane {
    uint32_t wr[3][4];
    uint32_t wr2[3][4];  // the same taps one byte up: for a window that starts at the second byte of the row words
    float ms[4], bs[4];
    int bias[4];
    float hp;
    bool fold;
    RequantParams rq;

    __device__ __forceinline__ void setup(const uint8_t* __restrict__ w, const Dw3Desc& d, const EpiArgs& epi, int c0) {
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
#pragma unroll
        for (int kh = 0; kh < 3; ++kh)
#pragma unroll
            for (int c = 0; c < 4; ++c) wr2[kh][c] = wr[kh][c] << 8;
        rq = epi.rq;
        fold = rq.fold != 0;
        hp = fold_hi_ph(rq);
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
    }

    // the four per-channel neighbour words of a row, from the words of the window's three columns
    static __device__ __forceinline__ void permute(uint32_t (&r)[4], uint32_t x0, uint32_t x1, uint32_t x2) {
        r[0] = __byte_perm(__byte_perm(x0, x1, 0x0040), x2, 0x0410);
        r[1] = __byte_perm(__byte_perm(x0, x1, 0x0051), x2, 0x0510);
        r[2] = __byte_perm(__byte_perm(x0, x1, 0x0062), x2, 0x0610);
        r[3] = __byte_perm(__byte_perm(x0, x1, 0x0073), x2, 0x0710);
    }

    // the output word of a position from the permuted words of its three input rows
    // (kFold: 1 = folded requantization, 0 = reference order, -1 = whichever the call asks for, decided per word; kShift: the window
    // starts at the second byte of the words -- the right-hand one of two columns that share their row words -- so the taps move up a byte)
    template <int kFold = -1, int kShift = 0>
    __device__ __forceinline__ uint32_t word(const uint32_t (&r0)[4], const uint32_t (&r1)[4], const uint32_t (&r2)[4]) const {
        uint32_t q[4];
        const uint32_t (&wt)[3][4] = kShift ? wr2 : wr;
        if (kFold == 1 || (kFold < 0 && fold)) {
            // the dot products start from the bits of 1.5 * 2^23: |sum| <= 9 * 255 * 255 < 2^22, so the integer sum lands in the mantissa
            // and (bits as float) - 1.5 * 2^23 IS float(sum), exactly, without a conversion; the placed integer (at most 255) is the low
            // byte of the last multiply-add's bits, which the packing permutes pick directly.  Two channels per packed-float instruction
            // where the operation has a packed form.
            const uint64_t m15 = pack2(12582912.f, 12582912.f), m23 = pack2(8388608.f, 8388608.f), hp2 = pack2(hp, hp);
#pragma unroll
            for (int c = 0; c < 4; c += 2) {
                int a0 = dot4<kWSigned>(r0[c], wt[0][c], 0x4b400000);
                int a1 = dot4<kWSigned>(r0[c + 1], wt[0][c + 1], 0x4b400000);
                a0 = dot4<kWSigned>(r1[c], wt[1][c], a0);
                a1 = dot4<kWSigned>(r1[c + 1], wt[1][c + 1], a1);
                a0 = dot4<kWSigned>(r2[c], wt[2][c], a0);
                a1 = dot4<kWSigned>(r2[c + 1], wt[2][c + 1], a1);
                const uint64_t f2 = sub_x2(pack2(__int_as_float(a0), __int_as_float(a1)), m15);
                const float t0 = fma_sat(lo_of(f2), ms[c], bs[c]), t1 = fma_sat(hi_of(f2), ms[c + 1], bs[c + 1]);
                const uint64_t q2 = fma_rm_x2(pack2(t0, t1), hp2, m23);
                q[c] = (uint32_t)q2;
                q[c + 1] = (uint32_t)(q2 >> 32);
            }
            return __byte_perm(__byte_perm(q[0], q[1], 0x0040), __byte_perm(q[2], q[3], 0x0040), 0x5410);
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            int acc = dot4<kWSigned>(r0[c], wt[0][c], 0);
            acc = dot4<kWSigned>(r1[c], wt[1][c], acc);
            acc = dot4<kWSigned>(r2[c], wt[2][c], acc);
            q[c] = requant_u8_up_fast(acc, bias[c], ms[c], false, 0u, rq);
        }
        return (q[0] & 0xffu) | ((q[1] & 0xffu) << 8) | ((q[2] & 0xffu) << 16) | (q[3] << 24);
    }
};

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
    Dw3Lane<kWSigned> ln;
    ln.setup(w, d, epi, c0);
    const int wi0 = wo * S - d.pl;
    const bool in0 = wi0 >= 0 && wi0 < d.W, in1 = wi0 + 1 >= 0 && wi0 + 1 < d.W, in2 = wi0 + 2 >= 0 && wi0 + 2 < d.W;
    const int64_t x_row = (int64_t)d.W * d.x_cs, y_row = (int64_t)d.Wo * d.y_cs;  // bytes between rows
    // small maps: a thread walks several images, so that the set-up above (weights, per-channel requantization) is paid once per ~28 rows
    for (int n = blockIdx.z * d.images_per_thread; n < min(d.N, (int)(blockIdx.z + 1) * d.images_per_thread); ++n) {
        const uint8_t* xn = x + (int64_t)n * d.H * x_row + (int64_t)wi0 * d.x_cs + c0;
        uint8_t* yp = y + ((int64_t)n * d.Ho + h_begin) * y_row + (int64_t)wo * d.y_cs + c0;
        // raw words of an input row's three columns (zeros outside the map: the padding of a zero-point-0 map); fetched one row ahead
        // of their use, so that the loads of the next row are in flight while the current one is worked on
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
        auto permute = [&](uint32_t (&r)[4], const Raw& v) { Dw3Lane<kWSigned>::permute(r, v.x0, v.x1, v.x2); };
        auto emit = [&](const uint32_t (&r0)[4], const uint32_t (&r1)[4], const uint32_t (&r2)[4]) {
            *reinterpret_cast<uint32_t*>(yp) = ln.word(r0, r1, r2);
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
                permute(rc, nx); nx = fetch(hn++); emit(ra, rb, rc); if (++ho >= h_end) break;
                permute(ra, nx); nx = fetch(hn++); emit(rb, rc, ra); if (++ho >= h_end) break;
                permute(rb, nx); nx = fetch(hn++); emit(rc, ra, rb); if (++ho >= h_end) break;
            }
        } else {
            const int base = 2 * ho - d.pt;
            Raw v = fetch(base);
            Raw p1 = fetch(base + 1), p2 = fetch(base + 2);
            permute(ra, v);
            int hn = base + 3;
            while (true) {
                permute(rb, p1); permute(rc, p2); p1 = fetch(hn); p2 = fetch(hn + 1); hn += 2; emit(ra, rb, rc); if (++ho >= h_end) break;
                permute(ra, p1); permute(rb, p2); p1 = fetch(hn); p2 = fetch(hn + 1); hn += 2; emit(rc, ra, rb); if (++ho >= h_end) break;
                permute(rc, p1); permute(ra, p2); p1 = fetch(hn); p2 = fetch(hn + 1); hn += 2; emit(rb, rc, ra); if (++ho >= h_end) break;
            }
        }
    }  // images
}

// ---- the same arithmetic, input rows staged in shared memory by TMA ----------------------------------------------------------------------
// The kernel above keeps four bytes per thread in flight (its next row's own word; the two neighbours are other threads' words), a few KB
// per SM: far too little to cover DRAM latency at HBM bandwidth.  Here a producer thread streams the input through a ring of shared-memory
// stages with TMA -- boxes of cb channel bytes x (wt - 1) * S + 3 columns x six rows, zero fill outside the map (the padding of a zero-point-0
// map) and beyond the last channel -- so tens of KB per SM are in flight and nothing but the output word lives in registers between rows.
// A CTA owns wt output columns x cb / 4 channel words (one consumer thread each) and walks the rows of images_per_cta images; six input
// rows are two periods of the three-slot row window at stride 1 and one at stride 2, so a stage is straight-line code.  Every wait is
// bounded: after wait_limit_ns without progress the thread sets the abort flag and the device status word and the CTA returns.
struct Dw3Staged {
    int N, C, H, W, Ho, Wo, pt, pl;
    int y_cs;
    int cb, wt, wbox;
    int col_tiles;
    int images_per_cta;
    int chunks;      // stages per image: ceil(((Ho - 1) * S + 3) / 6)
    int consumers;   // consumer threads: cb / 4 * wt rounded up to whole warps
    int stage_stride;
    int* status;
    unsigned long long wait_limit_ns;
};
constexpr int kDwRows = 6, kDwStages = 4;

template <int S, bool kWSigned, bool kFold, int kCols>
__global__ void __launch_bounds__(288, (kCols == 2 && kFold) ? 3 : 1) dw3x3_staged_kernel(const __grid_constant__ CUtensorMap tmX, const uint8_t* __restrict__ w, const Dw3Desc wd,
                                                           const Dw3Staged d, const EpiArgs epi, uint8_t* __restrict__ y) {
    using namespace tc;
    extern __shared__ uint8_t dw_smem_raw[];
    uint8_t* smem = dw_smem_raw + ((128u - (smem_u32(dw_smem_raw) & 127u)) & 127u);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kDwStages * d.stage_stride);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * kDwStages);
    const uint32_t bar_base = smem_u32(bars);
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (kDwStages + s); };
    const int consumer_warps = d.consumers >> 5;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kDwStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), consumer_warps);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    const int ct = blockIdx.x % d.col_tiles, cblk = blockIdx.x / d.col_tiles;
    const int n_begin = blockIdx.y * d.images_per_cta;
    const int n_end = min(d.N, n_begin + d.images_per_cta);
    const int total = (n_end - n_begin) * d.chunks;
    const uint32_t stage_bytes = (uint32_t)(kDwRows * d.wbox * d.cb);

    if ((int)threadIdx.x >= d.consumers) {
        // ---------------- producer: one lane streams the boxes ----------------
        if ((int)threadIdx.x == d.consumers) {
            const int wi0 = ct * d.wt * S - d.pl;
            int g = 0;
            for (int n = n_begin; n < n_end; ++n) {
                for (int k = 0; k < d.chunks; ++k, ++g) {
                    const int st = g % kDwStages;
                    if (g >= kDwStages && !mbar_wait(empty_bar(st), (uint32_t)(g / kDwStages - 1) & 1u, abort_flag, d.status, 31, 0, d.wait_limit_ns)) {
                        n = n_end;
                        break;
                    }
                    mbar_expect_tx(full_bar(st), stage_bytes);
                    tma_load_4d(smem_u32(smem + st * d.stage_stride), &tmX, full_bar(st), cblk * d.cb, wi0, k * kDwRows - d.pt, n);
                }
            }
            // leave only when the copies issued have landed (bounded): the CTA's shared memory must outlive them
            for (int i = max(0, g - kDwStages); i < g; ++i) {
                const uint64_t t0 = global_timer_ns();
                while (!mbar_try_wait(full_bar(i % kDwStages), (uint32_t)(i / kDwStages) & 1u))
                    if (global_timer_ns() - t0 > d.wait_limit_ns) break;
            }
        }
        return;
    }
    // ---------------- consumers ----------------
    // kCols == 2 (stride 1): a thread owns two neighbouring output columns.  The four pixel words of their windows are byte-transposed
    // into one word per channel (eight permutes for both columns instead of eight per column), which the left column multiplies by
    // (w0, w1, w2, 0) and the right one by (0, w0, w1, w2).
    static_assert(kCols == 1 || (kCols == 2 && S == 1), "two columns per thread: stride 1 only");
    const int words = d.cb >> 2;
    const int j = (int)threadIdx.x / words, cw = (int)threadIdx.x - j * words;
    const int jc = j * kCols;            // first of the thread's output columns within the tile
    const int wo = ct * d.wt + jc;
    const int c0 = cblk * d.cb + cw * 4;
    const bool active = jc < d.wt && wo < d.Wo && c0 < d.C;
    const bool second = kCols == 2 && jc + 1 < d.wt && wo + 1 < d.Wo;
    Dw3Lane<kWSigned> ln;
    if (active) ln.setup(w, wd, epi, c0);
    const int lane = threadIdx.x & 31;
    const uint32_t row_bytes = (uint32_t)(d.wbox * d.cb), cb1 = (uint32_t)d.cb, cb2 = 2u * (uint32_t)d.cb, cb3 = 3u * (uint32_t)d.cb;
    const uint32_t my_base = smem_u32(smem) + (uint32_t)((S * jc) * d.cb + cw * 4);  // shared-memory address of the window's first word in stage 0
    const int64_t y_row = (int64_t)d.Wo * d.y_cs;
    auto lds = [](uint32_t addr) {
        uint32_t v;
        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
        return v;
    };
    uint32_t r0[4], r1[4], r2[4];
    int g = 0;
    for (int n = n_begin; n < n_end; ++n) {
        uint8_t* yn = y + (int64_t)n * d.Ho * y_row + (int64_t)wo * d.y_cs + c0;
        for (int k = 0; k < d.chunks; ++k, ++g) {
            const int st = g % kDwStages;
            if (!mbar_wait(full_bar(st), (uint32_t)(g / kDwStages) & 1u, abort_flag, d.status, 32, 32, d.wait_limit_ns)) return;
            if (active) {
                uint32_t addr = my_base + (uint32_t)(st * d.stage_stride);
                auto load = [&](uint32_t (&r)[4]) {
                    if (kCols == 1) {
                        Dw3Lane<kWSigned>::permute(r, lds(addr), lds(addr + cb1), lds(addr + cb2));
                    } else {
                        const uint32_t p0 = lds(addr), p1 = lds(addr + cb1), p2 = lds(addr + cb2), p3 = lds(addr + cb3);
                        const uint32_t u0 = __byte_perm(p0, p1, 0x5140), u1 = __byte_perm(p0, p1, 0x7362);
                        const uint32_t v0 = __byte_perm(p2, p3, 0x5140), v1 = __byte_perm(p2, p3, 0x7362);
                        r[0] = __byte_perm(u0, v0, 0x5410);
                        r[1] = __byte_perm(u0, v0, 0x7632);
                        r[2] = __byte_perm(u1, v1, 0x5410);
                        r[3] = __byte_perm(u1, v1, 0x7632);
                    }
                    addr += row_bytes;
                };
                // ho: output row completed by the stage's first input row; a stage in the middle of an image stores every row it completes,
                // the first and the last ones check each row against the map
                const int ho = S == 1 ? k * kDwRows - 2 : k * 3 - 1;
                constexpr int kOut = S == 1 ? 6 : 3;
                uint8_t* yp = yn + (int64_t)ho * y_row;
                auto put = [&](bool ok, const uint32_t (&a0)[4], const uint32_t (&a1)[4], const uint32_t (&a2)[4]) {
                    if (ok) *reinterpret_cast<uint32_t*>(yp) = ln.template word<kFold ? 1 : -1, 0>(a0, a1, a2);
                    if (kCols == 2 && ok && second) *reinterpret_cast<uint32_t*>(yp + d.y_cs) = ln.template word<kFold ? 1 : -1, 1>(a0, a1, a2);
                    yp += y_row;
                };
                if (ho >= 0 && ho + kOut <= d.Ho) {
                    auto emit = [&](const uint32_t (&a0)[4], const uint32_t (&a1)[4], const uint32_t (&a2)[4]) { put(true, a0, a1, a2); };
                    if (S == 1) {
                        load(r0); emit(r1, r2, r0);
                        load(r1); emit(r2, r0, r1);
                        load(r2); emit(r0, r1, r2);
                        load(r0); emit(r1, r2, r0);
                        load(r1); emit(r2, r0, r1);
                        load(r2); emit(r0, r1, r2);
                    } else {
                        load(r0); emit(r1, r2, r0);
                        load(r1);
                        load(r2); emit(r0, r1, r2);
                        load(r0);
                        load(r1); emit(r2, r0, r1);
                        load(r2);
                    }
                } else {
                    int h = ho;
                    auto emit = [&](const uint32_t (&a0)[4], const uint32_t (&a1)[4], const uint32_t (&a2)[4]) {
                        put(h >= 0 && h < d.Ho, a0, a1, a2);
                        ++h;
                    };
                    if (S == 1) {
                        load(r0); emit(r1, r2, r0);
                        load(r1); emit(r2, r0, r1);
                        load(r2); emit(r0, r1, r2);
                        load(r0); emit(r1, r2, r0);
                        load(r1); emit(r2, r0, r1);
                        load(r2); emit(r0, r1, r2);
                    } else {
                        load(r0); emit(r1, r2, r0);
                        load(r1);
                        load(r2); emit(r0, r1, r2);
                        load(r0);
                        load(r1); emit(r2, r0, r1);
                        load(r2);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty_bar(st));
        }
    }
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

// Staged form: needs what the row kernel needs and a map TMA can describe (16-byte aligned base and pixel pitch).
bool depthwise3x3_staged_eligible(const chxq_conv_geom& g, const void* x, const void* y, int x_zp, const EpiArgs& epi) {
    const int xcs = g.x_cstride > 0 ? g.x_cstride : g.C;
    return depthwise3x3_eligible(g, x, y, x_zp, epi) && xcs % 16 == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0 && g.C >= 16;
}

int launch_depthwise3x3_staged(const void* x, const void* w, int w_row_stride, int w_tap_stride, int w_diag, const chxq_conv_geom& g,
                               const EpiArgs& epi, void* y, cudaStream_t s) {
    if ((int64_t)g.N * g.Ho * g.Wo == 0) return CHXQ_OK;
    const int S = g.stride_h;
    const int cols = (S == 1 && epi.rq.fold != 0) ? 2 : 1;  // output columns per consumer thread (two: the folded form at stride 1)
    // block shape: cb channel bytes x wt output columns, one consumer thread per (channel word, column), at most 256 of them; the best
    // product of lane use (channels and columns that exist / those the blocks cover), box reuse (columns used / columns fetched) and
    // warp fill, with a mild preference for large blocks
    int best_cb = 0, best_wt = 0;
    double best = -1.0;
    // (at least 64 channel bytes per pixel where the map has them: shorter pieces waste DRAM sectors and TMA's per-row work)
    for (int cb = std::min(64, (g.C + 15) / 16 * 16); cb <= 256 && cb < g.C + 16; cb += 16) {
        for (int wt = 1; wt <= g.Wo && (cb / 4) * ((wt + cols - 1) / cols) <= 256; ++wt) {
            const int wbox = ((wt + cols - 1) / cols * cols - 1) * S + 3;
            if (wbox > 256 || (int64_t)kDwRows * wbox * cb > 16 * 1024) continue;
            const int threads = (cb / 4) * ((wt + cols - 1) / cols), padded = (threads + 31) / 32 * 32;
            const double lanes = (double)g.C / ((g.C + cb - 1) / cb * cb) * (double)g.Wo / ((g.Wo + wt - 1) / wt * wt);
            const double reuse = (double)(wt * S) / wbox;
            const double score = lanes * (reuse < 1.0 ? reuse : 1.0) * ((double)threads / padded) * (0.75 + 0.25 * padded / 256.0);
            if (score > best) {
                best = score;
                best_cb = cb;
                best_wt = wt;
            }
        }
    }
    if (best_cb == 0) return set_error(CHXQ_ERR_UNSUPPORTED, "depthwise 3x3: no block shape for this map");
    Dw3Desc wd{};
    wd.C = g.C;
    wd.w_row_stride = w_row_stride; wd.w_tap_stride = w_tap_stride; wd.w_diag = w_diag;
    Dw3Staged d{};
    d.N = g.N; d.C = g.C; d.H = g.H; d.W = g.W; d.Ho = g.Ho; d.Wo = g.Wo; d.pt = g.pad_top; d.pl = g.pad_left;
    d.y_cs = g.y_cstride > 0 ? g.y_cstride : g.M;
    d.cb = best_cb; d.wt = best_wt; d.wbox = ((best_wt + cols - 1) / cols * cols - 1) * S + 3;
    d.col_tiles = (g.Wo + d.wt - 1) / d.wt;
    const int ch_blocks = (g.C + d.cb - 1) / d.cb;
    d.chunks = ((g.Ho - 1) * S + 3 + kDwRows - 1) / kDwRows;
    d.consumers = ((d.cb / 4) * ((d.wt + cols - 1) / cols) + 31) / 32 * 32;
    d.stage_stride = (kDwRows * d.wbox * d.cb + 127) / 128 * 128;
    const int64_t blocks_x = (int64_t)d.col_tiles * ch_blocks;
    // short maps: a CTA walks several images, so that its ring fills and a thread's set-up is paid once per ~8 stages -- as long as the
    // grid still has a few CTAs per SM slot
    const int64_t ipc_cap = std::max<int64_t>(1, (int64_t)g.N * blocks_x / 888);
    d.images_per_cta = (int)std::max<int64_t>(1, std::min<int64_t>((8 + d.chunks - 1) / d.chunks, ipc_cap));
    d.status = device_status_ptr();
    if (!d.status) return set_error(CHXQ_ERR_CUDA, "device status word is unavailable");
    d.wait_limit_ns = (unsigned long long)tc::wait_limit_ns_value();
    const int xcs = g.x_cstride > 0 ? g.x_cstride : g.C;
    alignas(64) CUtensorMap tmX;
    const int rc = tc::encode_nhwc_box_map(&tmX, x, g.C, g.W, g.H, g.N, xcs, d.cb, d.wbox, kDwRows);
    if (rc != CHXQ_OK) return rc;
    const size_t smem = 128 + (size_t)kDwStages * d.stage_stride + 2 * kDwStages * 8 + 16;
    dim3 grid((unsigned)blocks_x, (unsigned)((g.N + d.images_per_cta - 1) / d.images_per_cta));
    const unsigned block = (unsigned)d.consumers + 32u;
    const bool ws = g.w_dtype == CHXQ_INT8;
    const uint8_t* wb = static_cast<const uint8_t*>(w);
    uint8_t* yb = static_cast<uint8_t*>(y);
    auto run = [&](auto kernel) -> int {
        if (smem > 48 * 1024) CHXQ_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        kernel<<<grid, block, smem, s>>>(tmX, wb, wd, d, epi, yb);
        CHXQ_LAUNCH_CHECK();
        return CHXQ_OK;
    };
    if (epi.rq.fold != 0) {
        if (S == 1) return ws ? run(dw3x3_staged_kernel<1, true, true, 2>) : run(dw3x3_staged_kernel<1, false, true, 2>);
        return ws ? run(dw3x3_staged_kernel<2, true, true, 1>) : run(dw3x3_staged_kernel<2, false, true, 1>);
    }
    if (S == 1) return ws ? run(dw3x3_staged_kernel<1, true, false, 1>) : run(dw3x3_staged_kernel<1, false, false, 1>);
    return ws ? run(dw3x3_staged_kernel<2, true, false, 1>) : run(dw3x3_staged_kernel<2, false, false, 1>);
}

}  // namespace chxq
