// General CUDA-core kernels: any shape, layout, group count and zero-point form of MatMulInteger,
// QLinearMatMul, ConvInteger and QLinearConv, plus the small glue kernels of a quantized CNN graph.
// These are the catch-all path behind the tcgen05 kernels (tc_igemm.cu) and the on-device second
// opinion the tensor-core results are compared with; they are not the fast path.
#include "common.h"
#include "epilogue.cuh"
#include "kernels.h"

namespace chxq {
namespace {

template <bool kSigned>
__device__ __forceinline__ int ldq(const void* p, int64_t i) {
    return kSigned ? (int)static_cast<const int8_t*>(p)[i] : (int)static_cast<const uint8_t*>(p)[i];
}

__device__ __forceinline__ int ldq_rt(const void* p, int64_t i, int is_signed) {
    return is_signed ? (int)static_cast<const int8_t*>(p)[i] : (int)static_cast<const uint8_t*>(p)[i];
}

// ---------------------------------------------------------------------------------------------
// GEMM: y[b, m, n] = sum_k (a[b,m,k] - za[k]) * (b[b,k,n] - zb[n]).  32x32 output tile per block,
// zero points subtracted while staging into shared memory, int32 wrap-around accumulation.
// ---------------------------------------------------------------------------------------------
constexpr int kGT = 32;

template <bool kASigned, bool kBSigned>
__global__ void __launch_bounds__(256) gemm_simt_kernel(
        const void* __restrict__ a, const void* __restrict__ b, int64_t M, int64_t N, int64_t K, ZpSpec zas, ZpSpec zbs, EpiArgs epi,
        void* __restrict__ y) {
    __shared__ int As[kGT][kGT + 1];
    __shared__ int Bs[kGT][kGT + 1];
    const int tx = threadIdx.x, ty = threadIdx.y;  // 32 x 8
    const int64_t m0 = (int64_t)blockIdx.y * kGT, n0 = (int64_t)blockIdx.x * kGT;
    const int64_t bt = blockIdx.z;
    const int64_t a_off = bt * M * K, b_off = bt * K * N, y_off = bt * M * N;
    unsigned acc[4] = {0u, 0u, 0u, 0u};
    const int64_t n = n0 + tx;
    const void* za = zas.ptr;
    const int64_t za_len = zas.len;
    int zbn = 0;
    if (zbs.len > 0 && n < N) zbn = zbs.ptr ? ldq<kBSigned>(zbs.ptr, zbs.len == 1 ? 0 : n) : zbs.scalar;
    for (int64_t k0 = 0; k0 < K; k0 += kGT) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = ty * 4 + i;
            const int64_t m = m0 + r, k = k0 + tx;
            int v = 0;
            if (m < M && k < K) {
                v = ldq<kASigned>(a, a_off + m * K + k);
                if (za_len > 0) v -= za ? ldq<kASigned>(za, za_len == 1 ? 0 : k) : zas.scalar;
            }
            As[r][tx] = v;
            const int64_t kb = k0 + r;
            int w = 0;
            if (kb < K && n < N) w = ldq<kBSigned>(b, b_off + kb * N + n) - zbn;
            Bs[r][tx] = w;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < kGT; ++kk) {
            const unsigned bv = (unsigned)Bs[kk][tx];
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[i] += (unsigned)As[ty * 4 + i][kk] * bv;
        }
        __syncthreads();
    }
    if (n >= N) return;
    const float mult = epi.mode == kEpiRequant ? epi_mult(epi, (int)n) : 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int64_t m = m0 + ty * 4 + i;
        if (m >= M) continue;
        const int64_t o = y_off + m * N + n;
        if (epi.mode == kEpiInt32) {
            static_cast<int32_t*>(y)[o] = (int32_t)acc[i];
        } else {
            const int bias = epi.bias ? epi.bias[n] : 0;
            const int q = epi_requant(epi, (int)acc[i], mult, bias, epi.residual ? epi.residual[o] : 0);
            static_cast<uint8_t*>(y)[o] = (uint8_t)q;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Direct convolution, one thread per output element.  The output's fastest axis is the thread's
// fastest axis (channel for NHWC, column for NCHW) so stores coalesce.
// ---------------------------------------------------------------------------------------------
struct ConvDesc {
    int N, C, H, W, M, KH, KW, sh, sw, pt, pl, Ho, Wo, group;
    int x_nhwc, y_nhwc, x_cs, y_cs;  // channel strides (NHWC)
    int x_signed, w_signed;
    int has_x_zp, x_zp;
    int64_t w_zp_len;
};

// x_zp_dev != nullptr: the activation zero point is a device scalar of x's dtype (a zero point that was computed on the
// device, e.g. by the dynamic-quantization parameter kernel), read here instead of on the host.
__global__ void __launch_bounds__(256) conv_simt_kernel(
        const void* __restrict__ x, const void* __restrict__ w, const void* __restrict__ w_zp, ConvDesc d, EpiArgs epi, void* __restrict__ y,
        const void* __restrict__ x_zp_dev) {
    if (x_zp_dev != nullptr) {
        d.has_x_zp = 1;
        d.x_zp = ldq_rt(x_zp_dev, 0, d.x_signed);
    }
    const int64_t total = (int64_t)d.N * d.M * d.Ho * d.Wo;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int Cg = d.C / d.group, Mg = d.M / d.group;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        int n, m, ho, wo;
        int64_t r = idx;
        if (d.y_nhwc) {
            m = (int)(r % d.M); r /= d.M;
            wo = (int)(r % d.Wo); r /= d.Wo;
            ho = (int)(r % d.Ho); r /= d.Ho;
            n = (int)r;
        } else {
            wo = (int)(r % d.Wo); r /= d.Wo;
            ho = (int)(r % d.Ho); r /= d.Ho;
            m = (int)(r % d.M); r /= d.M;
            n = (int)r;
        }
        const int g = m / Mg;
        const int zw = d.w_zp_len == 0 ? 0 : ldq_rt(w_zp, d.w_zp_len == 1 ? 0 : m, d.w_signed);
        unsigned acc = 0u;
        for (int kh = 0; kh < d.KH; ++kh) {
            const int hi = ho * d.sh - d.pt + kh;
            if (hi < 0 || hi >= d.H) continue;
            for (int kw = 0; kw < d.KW; ++kw) {
                const int wi = wo * d.sw - d.pl + kw;
                if (wi < 0 || wi >= d.W) continue;
                for (int c = 0; c < Cg; ++c) {
                    const int ci = g * Cg + c;
                    const int64_t xo = d.x_nhwc ? (((int64_t)n * d.H + hi) * d.W + wi) * d.x_cs + ci
                                                : (((int64_t)n * d.C + ci) * d.H + hi) * d.W + wi;
                    int xv = ldq_rt(x, xo, d.x_signed);
                    if (d.has_x_zp) xv -= d.x_zp;
                    const int wv = ldq_rt(w, (((int64_t)m * Cg + c) * d.KH + kh) * d.KW + kw, d.w_signed) - zw;
                    acc += (unsigned)xv * (unsigned)wv;
                }
            }
        }
        const int64_t o = d.y_nhwc ? (((int64_t)n * d.Ho + ho) * d.Wo + wo) * d.y_cs + m : (((int64_t)n * d.M + m) * d.Ho + ho) * d.Wo + wo;
        if (epi.mode == kEpiInt32) {
            static_cast<int32_t*>(y)[o] = (int32_t)acc;
        } else {
            const float mult = epi_mult(epi, m);
            const int bias = epi.bias ? epi.bias[m] : 0;
            const int q = epi_requant(epi, (int)acc, mult, bias, epi.residual ? epi.residual[o] : 0);
            static_cast<uint8_t*>(y)[o] = (uint8_t)q;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// im2col: A[row, k] with row = (n, ho, wo), k = tap * c_pitch + c (tap = kh*KW + kw), rows k_pad
// bytes long.  Columns with c >= C or tap >= KH*KW are zero.  Positions that fall into the
// convolution's padding are written as pad_byte = x_zp, i.e. as 0 in the zero-point-subtracted
// domain, which is where the reference pads (runtime/ops/quantize.cc:123-125 subtract the zero
// point before chainerx::Conv zero-pads).  One thread writes 16 consecutive bytes of one row.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) im2col_kernel(
        const uint8_t* __restrict__ x, ConvDesc d, int c_pitch, int k_pad, int pad_byte, uint8_t* __restrict__ a) {
    const int chunks = k_pad / 16;
    const int64_t rows = (int64_t)d.N * d.Ho * d.Wo;
    const int64_t total = rows * chunks;
    const int taps = d.KH * d.KW;
    const bool fast_ok = d.x_nhwc && (d.C % 16 == 0) && (c_pitch % 16 == 0) && (d.x_cs % 16 == 0);
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const int ch = (int)(idx % chunks);
        const int64_t r = idx / chunks;
        const int wo = (int)(r % d.Wo);
        const int64_t r2 = r / d.Wo;
        const int ho = (int)(r2 % d.Ho);
        const int n = (int)(r2 / d.Ho);
        uint32_t out[4] = {0u, 0u, 0u, 0u};
        const int kbase = ch * 16;
        if (fast_ok) {
            // 16 consecutive channels of one tap.
            const int tap = kbase / c_pitch, c0 = kbase % c_pitch;
            if (tap < taps && c0 < d.C) {
                const int kh = tap / d.KW, kw = tap % d.KW;
                const int hi = ho * d.sh - d.pt + kh, wi = wo * d.sw - d.pl + kw;
                if (hi >= 0 && hi < d.H && wi >= 0 && wi < d.W) {
                    const uint4 v = *reinterpret_cast<const uint4*>(x + (((int64_t)n * d.H + hi) * d.W + wi) * d.x_cs + c0);
                    out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
                } else {
                    const uint32_t pb = (uint32_t)pad_byte * 0x01010101u;
                    out[0] = out[1] = out[2] = out[3] = pb;
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const int k = kbase + j;
                const int tap = k / c_pitch, c = k % c_pitch;
                uint32_t v = 0u;
                if (tap < taps && c < d.C) {
                    const int kh = tap / d.KW, kw = tap % d.KW;
                    const int hi = ho * d.sh - d.pt + kh, wi = wo * d.sw - d.pl + kw;
                    if (hi >= 0 && hi < d.H && wi >= 0 && wi < d.W) {
                        const int64_t xo = d.x_nhwc ? (((int64_t)n * d.H + hi) * d.W + wi) * d.x_cs + c
                                                    : (((int64_t)n * d.C + c) * d.H + hi) * d.W + wi;
                        v = x[xo];
                    } else {
                        v = (uint32_t)pad_byte;
                    }
                }
                out[j >> 2] |= v << (8 * (j & 3));
            }
        }
        *reinterpret_cast<uint4*>(a + r * k_pad + kbase) = make_uint4(out[0], out[1], out[2], out[3]);
    }
}

// im2col of an NCHW map (small channel counts: the network stem).  One block per (n, ho): the KH input rows of every
// channel are staged in shared memory (padding columns and rows filled with pad_byte), then the Wo matrix rows of this
// output row -- contiguous in A -- are written with coalesced 128-bit stores, each byte gathered through a per-k offset table.
__global__ void __launch_bounds__(256) im2col_nchw_rows_kernel(
        const uint8_t* __restrict__ x, ConvDesc d, int a_pitch, int pad_byte, int wspan, uint8_t* __restrict__ a) {
    extern __shared__ __align__(16) uint8_t sm[];
    int16_t* off = reinterpret_cast<int16_t*>(sm);                 // [a_pitch] offset of column k inside the staged rows, -1 = zero
    uint8_t* rows = sm + ((a_pitch * 2 + 15) & ~15);                // [C][KH][wspan]
    const int n = blockIdx.x / d.Ho, ho = blockIdx.x % d.Ho;
    const int K = d.KH * d.KW * d.C;
    for (int k = threadIdx.x; k < a_pitch; k += blockDim.x) {
        int o = -1;
        if (k < K) {
            const int tap = k / d.C, c = k % d.C;
            const int kh = tap / d.KW, kw = tap % d.KW;
            o = (c * d.KH + kh) * wspan + kw;
        }
        off[k] = (int16_t)o;
    }
    const int hi0 = ho * d.sh - d.pt;
    for (int i = threadIdx.x; i < d.C * d.KH * wspan; i += blockDim.x) {
        const int col = i % wspan;
        const int r = i / wspan;
        const int kh = r % d.KH, c = r / d.KH;
        const int hi = hi0 + kh, wi = col - d.pl;
        uint8_t v = (uint8_t)pad_byte;
        if (hi >= 0 && hi < d.H && wi >= 0 && wi < d.W) v = x[(((int64_t)n * d.C + c) * d.H + hi) * d.W + wi];
        rows[i] = v;
    }
    __syncthreads();
    const int cpr = a_pitch / 16;
    uint8_t* out = a + ((int64_t)n * d.Ho + ho) * d.Wo * a_pitch;
    for (int idx = threadIdx.x; idx < d.Wo * cpr; idx += blockDim.x) {
        const int wo = idx / cpr, j = idx - wo * cpr;
        const int base = wo * d.sw;
        uint32_t w4[4] = {0u, 0u, 0u, 0u};
#pragma unroll
        for (int b = 0; b < 16; ++b) {
            const int o = off[j * 16 + b];
            const uint32_t v = o >= 0 ? rows[o + base] : 0u;
            w4[b >> 2] |= v << (8 * (b & 3));
        }
        *reinterpret_cast<uint4*>(out + (int64_t)idx * 16) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
    }
}

// im2col of an NCHW map with at most 4 channels, channel pitch 4 (k = tap * 4 + c): each pixel becomes one 32-bit word, so
// a matrix row is KH*KW words gathered with 32-bit shared-memory loads.  One block per (n, ho); the staged rows hold the
// pixels of every needed input row as words (padding pixels = pad_byte in the real channels, 0 in the unused lanes).
__global__ void __launch_bounds__(256) im2col_nchw_c4_kernel(
        const uint8_t* __restrict__ x, ConvDesc d, int a_pitch, int pad_byte, int wspan, uint8_t* __restrict__ a) {
    extern __shared__ __align__(16) uint32_t srow[];  // [KH][wspan] pixels
    const int n = blockIdx.x / d.Ho, ho = blockIdx.x % d.Ho;
    const int hi0 = ho * d.sh - d.pt;
    const uint32_t lanes = d.C >= 4 ? 0x01010101u : ((1u << (8 * d.C)) - 1u) & 0x01010101u;  // only real channels carry the pad value
    const uint32_t padw = (uint32_t)(pad_byte & 0xff) * lanes;
    for (int i = threadIdx.x; i < d.KH * wspan; i += blockDim.x) {
        const int col = i % wspan, kh = i / wspan;
        const int hi = hi0 + kh, wi = col - d.pl;
        uint32_t v = padw;
        if (hi >= 0 && hi < d.H && wi >= 0 && wi < d.W) {
            v = 0u;
            for (int c = 0; c < d.C; ++c) v |= (uint32_t)x[(((int64_t)n * d.C + c) * d.H + hi) * d.W + wi] << (8 * c);
        }
        srow[i] = v;
    }
    __syncthreads();
    const int cpr = a_pitch / 16;              // 16-byte chunks (4 taps) per matrix row
    const int taps = d.KH * d.KW;
    const int groups = blockDim.x / cpr;       // rows handled per sweep
    const int j = threadIdx.x % cpr, g0 = threadIdx.x / cpr;
    if (g0 >= groups) return;
    int off[4];
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        const int t = j * 4 + b;
        off[b] = t < taps ? (t / d.KW) * wspan + (t % d.KW) : -1;
    }
    uint8_t* out = a + ((int64_t)n * d.Ho + ho) * d.Wo * a_pitch;
    for (int wo = g0; wo < d.Wo; wo += groups) {
        const int base = wo * d.sw;
        uint4 v;
        v.x = off[0] >= 0 ? srow[off[0] + base] : 0u;
        v.y = off[1] >= 0 ? srow[off[1] + base] : 0u;
        v.z = off[2] >= 0 ? srow[off[2] + base] : 0u;
        v.w = off[3] >= 0 ? srow[off[3] + base] : 0u;
        *reinterpret_cast<uint4*>(out + ((int64_t)wo * cpr + j) * 16) = v;
    }
}

// ---------------------------------------------------------------------------------------------
// Glue kernels (NHWC u8 maps, 16 channels = one 128-bit word per thread where channels allow).
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t vmax_u8x4(uint32_t a, uint32_t b) {
    return __vmaxu4(a, b);
}

// Running maximum of packed bytes kept as two words of 16-bit lanes (even bytes, odd bytes): the byte-wise maximum has no
// native instruction, the 16-bit-pair maximum has.
struct MaxU8x4 {
    uint32_t even, odd;
    __device__ __forceinline__ void init() { even = odd = 0u; }
    __device__ __forceinline__ void update(uint32_t w) {
        even = __vmaxu2(even, w & 0x00ff00ffu);
        odd = __vmaxu2(odd, (w >> 8) & 0x00ff00ffu);
    }
    __device__ __forceinline__ uint32_t value() const { return even | (odd << 8); }
};

__global__ void __launch_bounds__(256) maxpool_u8_nhwc_kernel(
        const uint8_t* __restrict__ x, int N, int H, int W, int C, int k, int s, int p, int Ho, int Wo, uint8_t* __restrict__ y) {
    const int cv = C / 16;
    const int64_t total = (int64_t)N * Ho * Wo * cv;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        int c16, wo, ho, n;
        if (total < (1ll << 31)) {  // 32-bit index arithmetic: a 64-bit division costs an order of magnitude more instructions
            unsigned r = (unsigned)idx;
            c16 = (int)(r % (unsigned)cv); r /= (unsigned)cv;
            wo = (int)(r % (unsigned)Wo); r /= (unsigned)Wo;
            ho = (int)(r % (unsigned)Ho);
            n = (int)(r / (unsigned)Ho);
        } else {
            c16 = (int)(idx % cv);
            int64_t r = idx / cv;
            wo = (int)(r % Wo); r /= Wo;
            ho = (int)(r % Ho);
            n = (int)(r / Ho);
        }
        MaxU8x4 b0, b1, b2, b3;
        b0.init(); b1.init(); b2.init(); b3.init();
        for (int kh = 0; kh < k; ++kh) {
            const int hi = ho * s - p + kh;
            if (hi < 0 || hi >= H) continue;
            for (int kw = 0; kw < k; ++kw) {
                const int wi = wo * s - p + kw;
                if (wi < 0 || wi >= W) continue;
                const uint4 v = *reinterpret_cast<const uint4*>(x + (((int64_t)n * H + hi) * W + wi) * C + c16 * 16);
                b0.update(v.x); b1.update(v.y); b2.update(v.z); b3.update(v.w);
            }
        }
        *reinterpret_cast<uint4*>(y + (((int64_t)n * Ho + ho) * Wo + wo) * C + c16 * 16) = make_uint4(b0.value(), b1.value(), b2.value(), b3.value());
    }
}

__global__ void __launch_bounds__(256) maxpool_u8_nhwc_scalar_kernel(
        const uint8_t* __restrict__ x, int N, int H, int W, int C, int k, int s, int p, int Ho, int Wo, uint8_t* __restrict__ y) {
    const int64_t total = (int64_t)N * Ho * Wo * C;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const int c = (int)(idx % C);
        int64_t r = idx / C;
        const int wo = (int)(r % Wo); r /= Wo;
        const int ho = (int)(r % Ho);
        const int n = (int)(r / Ho);
        int best = 0;
        for (int kh = 0; kh < k; ++kh) {
            const int hi = ho * s - p + kh;
            if (hi < 0 || hi >= H) continue;
            for (int kw = 0; kw < k; ++kw) {
                const int wi = wo * s - p + kw;
                if (wi < 0 || wi >= W) continue;
                best = max(best, (int)x[(((int64_t)n * H + hi) * W + wi) * C + c]);
            }
        }
        y[idx] = (uint8_t)best;
    }
}

// y[n, c] = (float(sum_i (x[n,i,c] - zp)) / float(HW)) * scale.  One thread per (n, c); threads of
// a warp read consecutive channels, so every load instruction is a coalesced row segment.
__global__ void __launch_bounds__(256) global_avgpool_dq_kernel(
        const uint8_t* __restrict__ x, int N, int HW, int C, float scale, int zp, float* __restrict__ y) {
    const int64_t total = (int64_t)N * C;
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int c = (int)(idx % C);
    const int n = (int)(idx / C);
    int s = 0;
    const uint8_t* p = x + (int64_t)n * HW * C + c;
    for (int i = 0; i < HW; ++i) s += (int)p[(int64_t)i * C] - zp;
    y[idx] = __fmul_rn(__fdiv_rn((float)s, (float)HW), scale);
}

// fp32 Linear: y[n,o] = fma chain over k ascending of x[n,k] * w[o,k], then + b[o].  Every output is accumulated by one
// thread in k order (no split-K), so the result does not depend on the tiling.  32 x 64 output tile per block of 128
// threads; a thread owns rows {4 tn .. 4 tn + 3} and columns {to + 16 j}.  A 128-bit shared-memory load costs four cycles
// of the SM's load unit whatever it broadcasts; the 4 x 4 register tile needs eight of them per 64 fused multiply-adds.  The
// price of the sequential chains is parallelism: 256 x 1000 outputs are 3.5 warps per SM, about one per scheduler (measured:
// 63 us for [256, 2048] x [1000, 2048]^T, a quarter of the fp32 rate).  With K-major tiles of pitch 36 floats the loads along k are
// conflict-free (the eight lanes of a quarter warp read eight different rows whose starts are 36 floats apart, or all the
// same row).  The next K slice is fetched into registers while the current one is consumed, and shared memory is
// double-buffered, so there is one barrier per slice.
constexpr int kLinKS = 32;     // K slice
constexpr int kLinPitch = 36;  // floats
constexpr int kLinThreads = 128;

__global__ void __launch_bounds__(kLinThreads) linear_f32_kernel(
        const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b, int N, int K, int O, float* __restrict__ y) {
    __shared__ __align__(16) float Xs[2][32][kLinPitch];
    __shared__ __align__(16) float Ws[2][64][kLinPitch];
    const int tid = threadIdx.x;
    const int tn = tid / 16, to = tid % 16;
    const int n0 = blockIdx.y * 32, o0 = blockIdx.x * 64;
    const bool vec = (K % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15u) == 0) && ((reinterpret_cast<uintptr_t>(w) & 15u) == 0);
    // staging assignment: float4 number f = tid + 128 i of a tile covers row f / 8, k offset 4 (f % 8): two of X, four of W
    const int sr = tid / 8, sk = (tid % 8) * 4;
    auto fetch = [&](const float* base, int row, int rows, int k0) -> float4 {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (row < rows) {
            const float* p = base + (int64_t)row * K + k0 + sk;
            if (vec && k0 + sk + 4 <= K) {
                v = *reinterpret_cast<const float4*>(p);
            } else {
                if (k0 + sk + 0 < K) v.x = p[0];
                if (k0 + sk + 1 < K) v.y = p[1];
                if (k0 + sk + 2 < K) v.z = p[2];
                if (k0 + sk + 3 < K) v.w = p[3];
            }
        }
        return v;
    };
    float acc[4][4] = {};
    float4 px[2], pw[4];
#pragma unroll
    for (int i = 0; i < 2; ++i) px[i] = fetch(x, n0 + sr + 16 * i, N, 0);
#pragma unroll
    for (int i = 0; i < 4; ++i) pw[i] = fetch(w, o0 + sr + 16 * i, O, 0);
    int buf = 0;
    for (int k0 = 0; k0 < K; k0 += kLinKS, buf ^= 1) {
#pragma unroll
        for (int i = 0; i < 2; ++i) *reinterpret_cast<float4*>(&Xs[buf][sr + 16 * i][sk]) = px[i];
#pragma unroll
        for (int i = 0; i < 4; ++i) *reinterpret_cast<float4*>(&Ws[buf][sr + 16 * i][sk]) = pw[i];
        __syncthreads();
        if (k0 + kLinKS < K) {
#pragma unroll
            for (int i = 0; i < 2; ++i) px[i] = fetch(x, n0 + sr + 16 * i, N, k0 + kLinKS);
#pragma unroll
            for (int i = 0; i < 4; ++i) pw[i] = fetch(w, o0 + sr + 16 * i, O, k0 + kLinKS);
        }
        // Elements past K are zero in both operands; fma(0, 0, acc) leaves acc as it is, so the slice is always run in full.
#pragma unroll
        for (int k4 = 0; k4 < kLinKS; k4 += 4) {
            float4 xv[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) xv[i] = *reinterpret_cast<const float4*>(&Xs[buf][tn * 4 + i][k4]);
#pragma unroll
            for (int j = 0; j < 4; ++j) wv[j] = *reinterpret_cast<const float4*>(&Ws[buf][to + 16 * j][k4]);
            // k ascending per accumulator; the sixteen accumulators advance together, so that a fused multiply-add never waits
            // for the one before it (there is only one warp per scheduler to hide that latency)
            const float xa[4][4] = {{xv[0].x, xv[0].y, xv[0].z, xv[0].w}, {xv[1].x, xv[1].y, xv[1].z, xv[1].w},
                                    {xv[2].x, xv[2].y, xv[2].z, xv[2].w}, {xv[3].x, xv[3].y, xv[3].z, xv[3].w}};
            const float wa[4][4] = {{wv[0].x, wv[0].y, wv[0].z, wv[0].w}, {wv[1].x, wv[1].y, wv[1].z, wv[1].w},
                                    {wv[2].x, wv[2].y, wv[2].z, wv[2].w}, {wv[3].x, wv[3].y, wv[3].z, wv[3].w}};
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[i][j] = __fmaf_rn(xa[i][kk], wa[j][kk], acc[i][j]);
        }
        // the buffer written next iteration is the other one; its readers finished before this iteration's barrier
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int n = n0 + tn * 4 + i;
        if (n >= N) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int o = o0 + to + 16 * j;
            if (o < O) y[(int64_t)n * O + o] = __fadd_rn(acc[i][j], b ? b[o] : 0.f);
        }
    }
}

// NCHW <-> NHWC transposes through a 32x32 shared tile over the (C, H*W) plane.
template <typename T>
__global__ void __launch_bounds__(256) transpose_chw_kernel(const T* __restrict__ x, int C, int HW, int in_ld, int out_ld, int to_nhwc, T* __restrict__ y) {
    // to_nhwc: x is [N][C][HW] -> y [N][HW][out_ld];  else x is [N][HW][in_ld] -> y [N][C][HW]
    __shared__ T tile[32][33];
    const int n = blockIdx.z;
    const int tx = threadIdx.x, ty = threadIdx.y;  // 32 x 8
    const int rows = to_nhwc ? C : HW, cols = to_nhwc ? HW : C;  // input is [rows][cols(+ld)]
    const int64_t in_row_ld = to_nhwc ? HW : in_ld;
    const int64_t out_row_ld = to_nhwc ? out_ld : HW;
    const int64_t in_base = (int64_t)n * rows * in_row_ld;
    const int64_t out_base = (int64_t)n * cols * out_row_ld;
    const int r0 = blockIdx.y * 32, c0 = blockIdx.x * 32;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = r0 + ty * 4 + i, c = c0 + tx;
        if (r < rows && c < cols) tile[ty * 4 + i][tx] = x[in_base + (int64_t)r * in_row_ld + c];
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int c = c0 + ty * 4 + i, r = r0 + tx;
        if (r < rows && c < cols) y[out_base + (int64_t)c * out_row_ld + r] = tile[tx][ty * 4 + i];
    }
}

// NCHW <-> NHWC transposes of 1-byte maps, 64 channels x 64 positions per block of 256 threads.  The NCHW side moves as 32-bit
// words (four positions of one channel), the NHWC side as 128-bit words (sixteen channels of one position); in between, every
// thread transposes a 4 x 4 block of bytes in registers (eight byte permutes) and the tile crosses shared memory as words
// [position][channel / 4] with a pitch of 17 words, which keeps the word accesses of both phases (nearly) conflict-free.
// Channels beyond C up to the NHWC pitch are written as zeros (to_nhwc) or ignored.
constexpr int kTrC = 64, kTrP = 64, kTrPitchW = 17;

__device__ __forceinline__ void transpose4x4_bytes(uint32_t (&r)[4]) {
    const uint32_t t0 = __byte_perm(r[0], r[1], 0x5140), t1 = __byte_perm(r[0], r[1], 0x7362);
    const uint32_t t2 = __byte_perm(r[2], r[3], 0x5140), t3 = __byte_perm(r[2], r[3], 0x7362);
    r[0] = __byte_perm(t0, t2, 0x5410);
    r[1] = __byte_perm(t0, t2, 0x7632);
    r[2] = __byte_perm(t1, t3, 0x5410);
    r[3] = __byte_perm(t1, t3, 0x7632);
}

template <bool kToNhwc>
__global__ void __launch_bounds__(256) transpose_u8_tile_kernel(const uint8_t* __restrict__ x, int C, int HW, int ld, uint8_t* __restrict__ y) {
    __shared__ uint32_t tw[kTrP][kTrPitchW];
    const int n = blockIdx.z, c0 = blockIdx.y * kTrC, p0 = blockIdx.x * kTrP, tid = threadIdx.x;
    const uint8_t* nchw_in = x + (int64_t)n * C * HW;
    uint8_t* nchw_out = y + (int64_t)n * C * HW;
    const uint8_t* nhwc_in = x + (int64_t)n * HW * ld;
    uint8_t* nhwc_out = y + (int64_t)n * HW * ld;
    const bool words_ok = (HW % 4 == 0) && ((reinterpret_cast<uintptr_t>(kToNhwc ? x : y) & 3u) == 0);
    const bool quads_ok = (ld % 16 == 0) && ((reinterpret_cast<uintptr_t>(kToNhwc ? y : x) & 15u) == 0);
    const int a = tid / 16, b = tid % 16;   // NCHW side: channels 4a .. 4a+3, positions 4b .. 4b+3
    const int pos = tid / 4, q = tid % 4;   // NHWC side: position pos, channels 16q .. 16q+15
    if (kToNhwc) {
        uint32_t r[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int c = c0 + 4 * a + i, p = p0 + 4 * b;
            uint32_t v = 0u;
            if (c < C && p < HW) {
                const uint8_t* src = nchw_in + (int64_t)c * HW + p;
                if (words_ok && p + 4 <= HW) {
                    v = *reinterpret_cast<const uint32_t*>(src);
                } else {
                    for (int j = 0; j < 4 && p + j < HW; ++j) v |= (uint32_t)src[j] << (8 * j);
                }
            }
            r[i] = v;
        }
        transpose4x4_bytes(r);  // r[j] = channels 4a .. 4a+3 of position 4b + j
#pragma unroll
        for (int j = 0; j < 4; ++j) tw[4 * b + j][a] = r[j];
        __syncthreads();
        const int p = p0 + pos, c = c0 + 16 * q;
        if (p < HW && c < ld) {
            const uint32_t w4[4] = {tw[pos][4 * q], tw[pos][4 * q + 1], tw[pos][4 * q + 2], tw[pos][4 * q + 3]};
            uint8_t* dst = nhwc_out + (int64_t)p * ld + c;
            if (quads_ok && c + 16 <= ld) {
                *reinterpret_cast<uint4*>(dst) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
            } else {
                for (int j = 0; j < 16 && c + j < ld; ++j) dst[j] = (uint8_t)(w4[j >> 2] >> (8 * (j & 3)));
            }
        }
    } else {
        const int p = p0 + pos, c = c0 + 16 * q;
        uint32_t w4[4] = {0u, 0u, 0u, 0u};
        if (p < HW && c < C) {
            const uint8_t* src = nhwc_in + (int64_t)p * ld + c;
            if (quads_ok && c + 16 <= ld) {
                const uint4 v = *reinterpret_cast<const uint4*>(src);
                w4[0] = v.x; w4[1] = v.y; w4[2] = v.z; w4[3] = v.w;
            } else {
                for (int j = 0; j < 16 && c + j < C; ++j) w4[j >> 2] |= (uint32_t)src[j] << (8 * (j & 3));
            }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) tw[pos][4 * q + k] = w4[k];
        __syncthreads();
        uint32_t r[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) r[j] = tw[4 * b + j][a];  // channels 4a .. 4a+3 of position 4b + j
        transpose4x4_bytes(r);                                // r[i] = positions 4b .. 4b+3 of channel 4a + i
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int cc = c0 + 4 * a + i, pp = p0 + 4 * b;
            if (cc >= C || pp >= HW) continue;
            uint8_t* dst = nchw_out + (int64_t)cc * HW + pp;
            if (words_ok && pp + 4 <= HW) {
                *reinterpret_cast<uint32_t*>(dst) = r[i];
            } else {
                for (int j = 0; j < 4 && pp + j < HW; ++j) dst[j] = (uint8_t)(r[i] >> (8 * j));
            }
        }
    }
}

inline int grid_1d(int64_t total, int threads = 256, int per_sm = 16) {
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int64_t blocks = (total + threads - 1) / threads;
    const int64_t cap = (int64_t)sms * per_sm;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

}  // namespace

int launch_gemm_simt(
        const void* a, bool a_signed, const void* b, bool b_signed, int64_t batch, int64_t M, int64_t N, int64_t K, const ZpSpec& za,
        const ZpSpec& zb, const EpiArgs& epi, void* y, cudaStream_t s) {
    if (M == 0 || N == 0 || batch == 0) return CHXQ_OK;
    if ((M + kGT - 1) / kGT > 65535 || batch > 65535) return set_error(CHXQ_ERR_UNSUPPORTED, "SIMT GEMM: M or batch too large for the grid");
    dim3 grid((unsigned)((N + kGT - 1) / kGT), (unsigned)((M + kGT - 1) / kGT), (unsigned)batch), block(32, 8);
    if (a_signed) {
        if (b_signed)
            gemm_simt_kernel<true, true><<<grid, block, 0, s>>>(a, b, M, N, K, za, zb, epi, y);
        else
            gemm_simt_kernel<true, false><<<grid, block, 0, s>>>(a, b, M, N, K, za, zb, epi, y);
    } else {
        if (b_signed)
            gemm_simt_kernel<false, true><<<grid, block, 0, s>>>(a, b, M, N, K, za, zb, epi, y);
        else
            gemm_simt_kernel<false, false><<<grid, block, 0, s>>>(a, b, M, N, K, za, zb, epi, y);
    }
    CHXQ_LAUNCH_CHECK();
    return CHXQ_OK;
}

static ConvDesc make_desc(const chxq_conv_geom& g, int has_x_zp, int x_zp, int64_t w_zp_len) {
    ConvDesc d;
    d.N = g.N; d.C = g.C; d.H = g.H; d.W = g.W; d.M = g.M; d.KH = g.KH; d.KW = g.KW;
    d.sh = g.stride_h; d.sw = g.stride_w; d.pt = g.pad_top; d.pl = g.pad_left; d.Ho = g.Ho; d.Wo = g.Wo; d.group = g.group;
    d.x_nhwc = g.x_layout == CHXQ_NHWC;
    d.y_nhwc = g.y_layout == CHXQ_NHWC;
    d.x_cs = g.x_cstride > 0 ? g.x_cstride : g.C;
    d.y_cs = g.y_cstride > 0 ? g.y_cstride : g.M;
    d.x_signed = g.x_dtype == CHXQ_INT8;
    d.w_signed = g.w_dtype == CHXQ_INT8;
    d.has_x_zp = has_x_zp;
    d.x_zp = x_zp;
    d.w_zp_len = w_zp_len;
    return d;
}

int launch_conv_simt(
        const void* x, const void* w, const chxq_conv_geom& g, int has_x_zp, int x_zp, const void* w_zp, int64_t w_zp_len, const EpiArgs& epi,
        void* y, cudaStream_t s, const void* x_zp_dev) {
    const int64_t total = (int64_t)g.N * g.M * g.Ho * g.Wo;
    if (total == 0) return CHXQ_OK;
    ConvDesc d = make_desc(g, has_x_zp, x_zp, w_zp_len);
    conv_simt_kernel<<<grid_1d(total, 256, 32), 256, 0, s>>>(x, w, w_zp, d, epi, y, x_zp_dev);
    CHXQ_LAUNCH_CHECK();
    return CHXQ_OK;
}

int launch_im2col(const void* x, const chxq_conv_geom& g, int c_pitch, int k_pad, int pad_byte, void* a, cudaStream_t s) {
    ConvDesc d = make_desc(g, 0, 0, 0);
    const int64_t total = (int64_t)g.N * g.Ho * g.Wo * (k_pad / 16);
    if (total == 0) return CHXQ_OK;
    if (!d.x_nhwc && c_pitch == 4 && g.C <= 4 && k_pad / 16 <= 256) {
        const int wspan = (g.Wo - 1) * g.stride_w + g.KW;
        const size_t smem = (size_t)g.KH * wspan * 4;
        if (smem <= 48 * 1024 && (int64_t)g.N * g.Ho < (1ll << 31)) {
            im2col_nchw_c4_kernel<<<(unsigned)(g.N * g.Ho), 256, smem, s>>>(static_cast<const uint8_t*>(x), d, k_pad, pad_byte, wspan,
                                                                        static_cast<uint8_t*>(a));
            CHXQ_LAUNCH_CHECK();
            return CHXQ_OK;
        }
    }
    if (!d.x_nhwc && c_pitch == g.C && k_pad < 32768) {
        // NCHW input with dense K: stage whole input rows per (n, ho).
        const int wspan = (g.Wo - 1) * g.stride_w + g.KW;
        const size_t smem = ((size_t)(k_pad * 2 + 15) & ~(size_t)15) + (size_t)g.C * g.KH * wspan;
        if (smem <= 48 * 1024 && (int64_t)g.C * g.KH * wspan < 32768 && (int64_t)g.N * g.Ho < (1ll << 31)) {
            im2col_nchw_rows_kernel<<<(unsigned)(g.N * g.Ho), 256, smem, s>>>(static_cast<const uint8_t*>(x), d, k_pad, pad_byte, wspan,
                                                                          static_cast<uint8_t*>(a));
            CHXQ_LAUNCH_CHECK();
            return CHXQ_OK;
        }
    }
    im2col_kernel<<<grid_1d(total, 256, 32), 256, 0, s>>>(static_cast<const uint8_t*>(x), d, c_pitch, k_pad, pad_byte, static_cast<uint8_t*>(a));
    CHXQ_LAUNCH_CHECK();
    return CHXQ_OK;
}

}  // namespace chxq

using namespace chxq;

extern "C" int chxq_maxpool_u8_nhwc(
        const uint8_t* x, int32_t N, int32_t H, int32_t W, int32_t C, int32_t k, int32_t stride, int32_t pad, int32_t Ho, int32_t Wo, uint8_t* y,
        void* stream) {
    CHXQ_CHECK_ARG(x && y, "MaxPool: null buffer");
    CHXQ_CHECK_ARG(N > 0 && H > 0 && W > 0 && C > 0 && k > 0 && stride > 0 && pad >= 0 && Ho > 0 && Wo > 0, "MaxPool: bad geometry");
    CHXQ_CHECK_ARG((Ho - 1) * stride - pad < H && (Wo - 1) * stride - pad < W, "MaxPool: output window starts outside the input");
    cudaStream_t s = as_stream(stream);
    const bool vec = (C % 16 == 0) && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15u) == 0;
    if (vec)
        maxpool_u8_nhwc_kernel<<<grid_1d((int64_t)N * Ho * Wo * (C / 16)), 256, 0, s>>>(x, N, H, W, C, k, stride, pad, Ho, Wo, y);
    else
        maxpool_u8_nhwc_scalar_kernel<<<grid_1d((int64_t)N * Ho * Wo * C), 256, 0, s>>>(x, N, H, W, C, k, stride, pad, Ho, Wo, y);
    CHXQ_LAUNCH_CHECK();
    return CHXQ_OK;
}

extern "C" int chxq_global_avgpool_dq_nhwc(const uint8_t* x, int32_t N, int32_t HW, int32_t C, float scale, int32_t zp, float* y, void* stream) {
    CHXQ_CHECK_ARG(x && y && N > 0 && HW > 0 && C > 0, "AveragePool: bad arguments");
    const int64_t total = (int64_t)N * C;
    global_avgpool_dq_kernel<<<(unsigned)((total + 255) / 256), 256, 0, as_stream(stream)>>>(x, N, HW, C, scale, zp, y);
    CHXQ_LAUNCH_CHECK();
    return CHXQ_OK;
}

extern "C" int chxq_linear_f32(const float* x, const float* w, const float* b, int32_t N, int32_t K, int32_t O, float* y, void* stream) {
    CHXQ_CHECK_ARG(x && w && y && N > 0 && K > 0 && O > 0, "Linear: bad arguments");
    dim3 grid((O + 63) / 64, (N + 31) / 32);
    linear_f32_kernel<<<grid, kLinThreads, 0, as_stream(stream)>>>(x, w, b, N, K, O, y);
    CHXQ_LAUNCH_CHECK();
    return CHXQ_OK;
}

static int transpose_dispatch(const void* x, int elem_bytes, int N, int C, int H, int W, int c_stride, void* y, int to_nhwc, void* stream) {
    CHXQ_CHECK_ARG(x && y && N > 0 && C > 0 && H > 0 && W > 0, "layout transform: bad arguments");
    CHXQ_CHECK_ARG(elem_bytes == 1 || elem_bytes == 4, "layout transform: element size must be 1 or 4 bytes");
    const int ld = c_stride > 0 ? c_stride : C;
    CHXQ_CHECK_ARG(ld >= C, "layout transform: channel stride smaller than C");
    CHXQ_CHECK_ARG(N <= 65535, "layout transform: batch too large for the grid");
    const int HW = H * W;
    const int rows = to_nhwc ? C : HW, cols = to_nhwc ? HW : C;
    dim3 grid((cols + 31) / 32, (rows + 31) / 32, N), block(32, 8);
    CHXQ_CHECK_ARG(grid.y <= 65535, "layout transform: map too large for the grid");
    cudaStream_t s = as_stream(stream);
    if (elem_bytes == 1) {
        // 1-byte maps: the tiled kernel (32-bit words on the NCHW side, 128-bit words on the NHWC side)
        dim3 tgrid((HW + kTrP - 1) / kTrP, ((to_nhwc ? ld : C) + kTrC - 1) / kTrC, N);
        CHXQ_CHECK_ARG(tgrid.y <= 65535, "layout transform: too many channels for the grid");
        if (to_nhwc)
            transpose_u8_tile_kernel<true><<<tgrid, 256, 0, s>>>(static_cast<const uint8_t*>(x), C, HW, ld, static_cast<uint8_t*>(y));
        else
            transpose_u8_tile_kernel<false><<<tgrid, 256, 0, s>>>(static_cast<const uint8_t*>(x), C, HW, ld, static_cast<uint8_t*>(y));
    } else
        transpose_chw_kernel<uint32_t><<<grid, block, 0, s>>>(static_cast<const uint32_t*>(x), C, HW, ld, ld, to_nhwc, static_cast<uint32_t*>(y));
    CHXQ_LAUNCH_CHECK();
    return CHXQ_OK;
}

extern "C" int chxq_nchw_to_nhwc(const void* x, int32_t elem_bytes, int32_t N, int32_t C, int32_t H, int32_t W, int32_t c_stride, void* y, void* stream) {
    return transpose_dispatch(x, elem_bytes, N, C, H, W, c_stride, y, 1, stream);
}

extern "C" int chxq_nhwc_to_nchw(const void* x, int32_t elem_bytes, int32_t N, int32_t C, int32_t H, int32_t W, int32_t c_stride, void* y, void* stream) {
    return transpose_dispatch(x, elem_bytes, N, C, H, W, c_stride, y, 0, stream);
}
