// C-ABI entry points of the contraction ops (MatMulInteger, QLinearMatMul, ConvInteger, QLinearConv):
// argument validation, convolution geometry, path selection, workspace carving, and the small
// pre-pass kernels that feed the tensor-core kernel (operand repacking and zero-point terms).
#include <string.h>

#include <atomic>

#include "common.h"
#include "kernels.h"

namespace chxq {
namespace {

inline size_t align_up(size_t v, size_t a) {
    return (v + a - 1) / a * a;
}

template <bool kSigned>
__device__ __forceinline__ int ldq(const void* p, int64_t i) {
    return kSigned ? (int)static_cast<const int8_t*>(p)[i] : (int)static_cast<const uint8_t*>(p)[i];
}
__device__ __forceinline__ int ldq_rt(const void* p, int64_t i, int is_signed) {
    return is_signed ? (int)static_cast<const int8_t*>(p)[i] : (int)static_cast<const uint8_t*>(p)[i];
}
__device__ __forceinline__ int zp_at(const ZpSpec& z, int64_t i, int is_signed) {
    if (z.len == 0) return 0;
    if (z.ptr == nullptr) return z.scalar;
    return ldq_rt(z.ptr, z.len == 1 ? 0 : i, is_signed);
}

// B[K, N] (row-major) -> Bt[N, k_pad] (K-major rows, zero padded) and, in the same pass, the column terms of the activation zero
// point, T[n] += sum_k za[k] * b[k, n] (T zeroed beforehand; integer atomics, so the sum is exact whatever the order).
// 64 x 64 bytes per block of 256 threads: 32-bit loads along N, a 4 x 4 byte transpose in registers, the tile through shared
// memory as words with a pitch of 17 (conflict-free), 128-bit stores along K.
__device__ __forceinline__ void transpose4x4(uint32_t (&r)[4]) {
    const uint32_t t0 = __byte_perm(r[0], r[1], 0x5140), t1 = __byte_perm(r[0], r[1], 0x7362);
    const uint32_t t2 = __byte_perm(r[2], r[3], 0x5140), t3 = __byte_perm(r[2], r[3], 0x7362);
    r[0] = __byte_perm(t0, t2, 0x5410);
    r[1] = __byte_perm(t0, t2, 0x7632);
    r[2] = __byte_perm(t1, t3, 0x5410);
    r[3] = __byte_perm(t1, t3, 0x7632);
}

__global__ void __launch_bounds__(256) transpose_b_terms_kernel(
        const uint8_t* __restrict__ b, int64_t K, int64_t N, int64_t k_pad, uint8_t* __restrict__ bt, ZpSpec za, int a_signed, int b_signed,
        int32_t* __restrict__ T) {
    __shared__ uint32_t tw[64][17];
    __shared__ int colsum[64];
    const int tid = threadIdx.x;
    const int64_t k0 = (int64_t)blockIdx.y * 64, n0 = (int64_t)blockIdx.x * 64;
    const int a = tid / 16, bq = tid % 16;  // load side: rows k0 + 4a .. +3, columns n0 + 4bq .. +3
    const bool words_ok = (N % 4 == 0) && ((reinterpret_cast<uintptr_t>(b) & 3u) == 0);
    if (tid < 64) colsum[tid] = 0;
    uint32_t r[4];
    int part[4] = {0, 0, 0, 0};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int64_t k = k0 + 4 * a + i, n = n0 + 4 * bq;
        uint32_t v = 0u;
        if (k < K && n < N) {
            const uint8_t* src = b + k * N + n;
            if (words_ok && n + 4 <= N) {
                v = *reinterpret_cast<const uint32_t*>(src);
            } else {
                for (int j = 0; j < 4 && n + j < N; ++j) v |= (uint32_t)src[j] << (8 * j);
            }
            if (T != nullptr) {
                const int z = zp_at(za, k, a_signed);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint32_t byte = (v >> (8 * j)) & 0xffu;
                    part[j] += z * (b_signed ? (int)(int8_t)byte : (int)byte);
                }
            }
        }
        r[i] = v;
    }
    transpose4x4(r);  // r[j] = rows 4a .. 4a+3 of column 4bq + j
    __syncthreads();   // colsum is zero
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        tw[4 * bq + j][a] = r[j];
        if (T != nullptr && part[j] != 0) atomicAdd(&colsum[4 * bq + j], part[j]);
    }
    __syncthreads();
    const int col = tid / 4, q = tid % 4;  // store side: column n0 + col, rows k0 + 16q .. +15
    const int64_t n = n0 + col, k = k0 + 16 * q;
    if (n < N && k < k_pad) {
        const uint32_t w4[4] = {tw[col][4 * q], tw[col][4 * q + 1], tw[col][4 * q + 2], tw[col][4 * q + 3]};
        uint8_t* dst = bt + n * k_pad + k;
        if (k + 16 <= k_pad && ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0)) {
            *reinterpret_cast<uint4*>(dst) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
        } else {
            for (int j = 0; j < 16 && k + j < k_pad; ++j) dst[j] = (uint8_t)(w4[j >> 2] >> (8 * (j & 3)));
        }
    }
    if (T != nullptr && tid < 64 && n0 + tid < N && colsum[tid] != 0) atomicAdd(&T[n0 + tid], colsum[tid]);
}

// zbn[n] = zb[n] widened.  One thread per column.
__global__ void __launch_bounds__(256) gemm_zb_kernel(int b_signed, int64_t N, ZpSpec zb, int32_t* __restrict__ zbn) {
    const int64_t n = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (n < N) zbn[n] = zp_at(zb, n, b_signed);
}

// R[m] = sum_k (a[m, k] - za[k]).  One warp per row.
__global__ void __launch_bounds__(256) gemm_row_terms_kernel(const void* __restrict__ a, int a_signed, int64_t M, int64_t K, ZpSpec za, int32_t* __restrict__ R) {
    const int64_t m = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (m >= M) return;
    int s = 0;
    for (int64_t k = lane; k < K; k += 32) s += ldq_rt(a, m * K + k, a_signed) - zp_at(za, k, a_signed);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) R[m] = s;
}

// OIHW weights -> K-major rows [M][tap * c_pitch + c], zero padded to k_total.  One thread per output byte.
__global__ void __launch_bounds__(256) pack_weights_kernel(
        const uint8_t* __restrict__ w, int M, int C, int taps, int c_pitch, int k_total, uint8_t* __restrict__ out) {
    const int64_t total = (int64_t)M * k_total;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int k = (int)(i % k_total);
        const int m = (int)(i / k_total);
        const int tap = k / c_pitch, c = k % c_pitch;
        uint8_t v = 0;
        if (tap < taps && c < C) v = w[((int64_t)m * C + c) * taps + tap];
        out[i] = v;
    }
}

// wsum[m] = sum of the raw quantized weights of output channel m; zw32[m] = widened zero point;
// *any_nonzero |= (zw[m] != 0).  One warp per channel.
__global__ void __launch_bounds__(256) weight_terms_kernel(
        const void* __restrict__ w, int w_signed, int M, int inner, ZpSpec zw, int32_t* __restrict__ wsum, int32_t* __restrict__ zw32,
        int32_t* __restrict__ any_nonzero) {
    const int m = (int)(((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5);
    const int lane = threadIdx.x & 31;
    if (m >= M) return;
    int s = 0;
    for (int i = lane; i < inner; i += 32) s += ldq_rt(w, (int64_t)m * inner + i, w_signed);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) {
        wsum[m] = s;
        const int z = zp_at(zw, m, w_signed);
        zw32[m] = z;
        if (z != 0) atomicOr(any_nonzero, 1);
    }
}

// Row sums of an explicit im2col matrix: R[r] = sum_{k < k_real...} A[r, k] - k_real * x_zp
// (padded columns are zero, so summing the whole row is the same).  One warp per row, 16 bytes per lane.
__global__ void __launch_bounds__(256) rowsum_matrix_kernel(const uint8_t* __restrict__ a, int a_signed, int64_t rows, int k_pad, int sub, int32_t* __restrict__ R) {
    const int64_t r = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (r >= rows) return;
    int s = 0;
    const uint4* p = reinterpret_cast<const uint4*>(a + r * k_pad);
    for (int i = lane; i < k_pad / 16; i += 32) {
        const uint4 v = p[i];
        if (a_signed) {
            s = __dp4a((int)v.x, 0x01010101, s); s = __dp4a((int)v.y, 0x01010101, s);
            s = __dp4a((int)v.z, 0x01010101, s); s = __dp4a((int)v.w, 0x01010101, s);
        } else {
            unsigned u = (unsigned)s;
            u = __dp4a(v.x, 0x01010101u, u); u = __dp4a(v.y, 0x01010101u, u);
            u = __dp4a(v.z, 0x01010101u, u); u = __dp4a(v.w, 0x01010101u, u);
            s = (int)u;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) R[r] = s - sub;
}

// Receptive-field sums of a map addressed by element strides (es_n, es_c, es_h, es_w):
// S[pos] = sum over taps inside the map and channels of (x - x_zp).  One thread per output position.
__global__ void __launch_bounds__(256) conv_possum_kernel(
        const uint8_t* __restrict__ x, int x_signed, int N, int H, int W, int C, int64_t es_n, int64_t es_c, int64_t es_h, int64_t es_w, int KH,
        int KW, int sh, int sw, int pt, int pl, int Ho, int Wo, int x_zp, int32_t* __restrict__ S) {
    const int64_t total = (int64_t)N * Ho * Wo;
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int wo = (int)(idx % Wo);
    const int64_t r = idx / Wo;
    const int ho = (int)(r % Ho);
    const int n = (int)(r / Ho);
    int s = 0;
    for (int kh = 0; kh < KH; ++kh) {
        const int hi = ho * sh - pt + kh;
        if (hi < 0 || hi >= H) continue;
        for (int kw = 0; kw < KW; ++kw) {
            const int wi = wo * sw - pl + kw;
            if (wi < 0 || wi >= W) continue;
            const uint8_t* p = x + (int64_t)n * es_n + (int64_t)hi * es_h + (int64_t)wi * es_w;
            for (int c = 0; c < C; ++c) s += (x_signed ? (int)(int8_t)p[c * es_c] : (int)p[c * es_c]) - x_zp;
        }
    }
    S[idx] = s;
}

// Space-to-depth repack for the stride-2 small-channel path: block (n, r, b) of the output holds the 2x2 pixels
// (2 (r + t0h) + dy, 2 (b + t0w) + dx), channel-minor, as 16 bytes [(dy*2+dx)*C + c]; pixels outside the map hold the
// activation zero point, unused bytes hold zero (their weights are zero).
// kQuant: the input is the fp32 tensor in front of a QuantizeLinear (scale qs, zero point qzp, reference rounding) that is
// applied on the fly, with the arithmetic of quantize_one, so that the uint8 map never exists in memory.
// Fused max pooling (kernel 3, stride 2, no padding) of a convolution's uint8 output: extents of the pooled map.
struct PoolSpec {
    int ho, wo;
};
struct S2dQuant {
    float scale, zp_f;
    int has_zp, round_mode;
    QDiv dv;  // constant-divisor form of scale (fast path of the QuantizeLinear kernels)
};
template <bool kQuant, int kC = 0>  // kC: the channel count when known at compile time (3: the byte positions of a block become constants)
__global__ void __launch_bounds__(256) s2d_repack_kernel(
        const void* __restrict__ xv, int N, int C_rt, int H, int W, int64_t es_n, int64_t es_c, int64_t es_h, int64_t es_w, int t0h, int t0w,
        int rows2, int cols2, uint32_t pad_byte, S2dQuant qz, uint4* __restrict__ out) {
    // One thread per PAIR of horizontally adjacent blocks: their four input pixels per (row, channel) are contiguous in a
    // W-contiguous map and come in as one 32-bit (uint8) or 128-bit (fp32) load away from the borders.
    const int C = kC > 0 ? kC : C_rt;
    const uint8_t* x = static_cast<const uint8_t*>(xv);
    const float* xf = static_cast<const float*>(xv);
    // (pairs start at an odd block where the first input column of block 0 is not a multiple of four pixels from the row start -- an odd
    // first tap offset -- so that the pair's four pixels stay one aligned load; the block in front of the row is not stored)
    const int shift = t0w & 1;
    const int pairs = (cols2 + shift + 1) / 2;
    const int64_t total = (int64_t)N * rows2 * pairs;
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    int b0, r, n;
    if (total < (1ll << 31)) {  // 32-bit index arithmetic where it fits: 64-bit divisions are an order of magnitude dearer
        unsigned q = (unsigned)idx;
        b0 = 2 * (int)(q % (unsigned)pairs) - shift; q /= (unsigned)pairs;
        r = (int)(q % (unsigned)rows2);
        n = (int)(q / (unsigned)rows2);
    } else {
        b0 = 2 * (int)(idx % pairs) - shift;
        const int64_t q = idx / pairs;
        r = (int)(q % rows2);
        n = (int)(q / rows2);
    }
    const bool base_ok = (reinterpret_cast<uintptr_t>(xv) & 15u) == 0;
    uint32_t word[2][4] = {{0u, 0u, 0u, 0u}, {0u, 0u, 0u, 0u}};
    const int xx0 = 2 * (b0 + t0w);
    if (kQuant && kC == 3) {
        // Three fp32 planes, away from the borders, reference rounding: six 128-bit loads, each quantized to one word of four pixels, and
        // the twelve bytes of a block (row, column, channel order) gathered from those words with seven byte permutes per block.
        const int yy0 = 2 * (r + t0h);
        const int64_t off0 = (int64_t)n * es_n + (int64_t)yy0 * es_h + (int64_t)xx0;
        if (es_w == 1 && base_ok && qz.dv.fast && qz.round_mode == 0 && yy0 >= 0 && yy0 + 1 < H && xx0 >= 0 && xx0 + 3 < W &&
            ((off0 | es_h | es_c) & 3) == 0) {
            const QDiv8 d8 = make_qdiv8(qz.dv, qz.zp_f);
            float4 f[2][3];
#pragma unroll
            for (int dy = 0; dy < 2; ++dy)
#pragma unroll
                for (int c = 0; c < 3; ++c) f[dy][c] = __ldcs(reinterpret_cast<const float4*>(xf + off0 + dy * es_h + c * es_c));
            bool general = false;
            uint32_t P[2][3];
#pragma unroll
            for (int dy = 0; dy < 2; ++dy)
#pragma unroll
                for (int c = 0; c < 3; ++c) P[dy][c] = quantize4_u8_up(f[dy][c], d8, &general);
            if (!general) {
                const int64_t o = ((int64_t)n * rows2 + r) * cols2 + b0;
                uint4 a, b;
                a.x = __byte_perm(__byte_perm(P[0][0], P[0][1], 0x1040), P[0][2], 0x3410);
                a.y = __byte_perm(__byte_perm(P[0][1], P[0][2], 0x0051), __byte_perm(P[1][0], P[1][1], 0x0040), 0x5410);
                a.z = __byte_perm(__byte_perm(P[1][0], P[1][1], 0x0510), P[1][2], 0x5214);
                a.w = 0u;
                b.x = __byte_perm(__byte_perm(P[0][0], P[0][1], 0x3062), P[0][2], 0x3610);
                b.y = __byte_perm(__byte_perm(P[0][1], P[0][2], 0x0073), __byte_perm(P[1][0], P[1][1], 0x0062), 0x5410);
                b.z = __byte_perm(__byte_perm(P[1][0], P[1][1], 0x0730), P[1][2], 0x7216);
                b.w = 0u;
                if (b0 >= 0) out[o] = a;
                if (b0 + 1 < cols2) out[o + 1] = b;
                return;
            }
        }
    }
#pragma unroll
    for (int dy = 0; dy < 2; ++dy) {
        const int yy = 2 * (r + t0h) + dy;
        const bool row_in = yy >= 0 && yy < H;
#pragma unroll
        for (int c = 0; c < 4; ++c) {  // at most four channels on this path; unrolled so that the loads of all channels are in flight together
            if (c >= C) break;
            uint32_t px[4] = {pad_byte, pad_byte, pad_byte, pad_byte};
            if (row_in) {
                const int64_t off = (int64_t)n * es_n + (int64_t)yy * es_h + (int64_t)c * es_c + (int64_t)xx0 * es_w;
                if (es_w == 1 && xx0 >= 0 && xx0 + 3 < W && (off & 3) == 0 && base_ok) {
                    if (kQuant) {
                        const float4 f = __ldcs(reinterpret_cast<const float4*>(xf + off));
                        bool general = !qz.dv.fast;  // same arithmetic as quantize_vec16_kernel: division by a constant, add-based rounding
                        if (!general) {
                            if (qz.round_mode == 0) {
                                const uint32_t packed = quantize4_u8_up(f, make_qdiv8(qz.dv, qz.zp_f), &general);
                                px[0] = packed & 0xffu; px[1] = (packed >> 8) & 0xffu; px[2] = (packed >> 16) & 0xffu; px[3] = packed >> 24;
                            } else {
                                const float t0 = qdiv_unguarded(f.x, qz.dv, &general), t1 = qdiv_unguarded(f.y, qz.dv, &general);
                                const float t2 = qdiv_unguarded(f.z, qz.dv, &general), t3 = qdiv_unguarded(f.w, qz.dv, &general);
                                px[0] = quantize_u8_rne_bits(t0, qz.zp_f); px[1] = quantize_u8_rne_bits(t1, qz.zp_f);
                                px[2] = quantize_u8_rne_bits(t2, qz.zp_f); px[3] = quantize_u8_rne_bits(t3, qz.zp_f);
                            }
                        }
                        if (general) {
                            px[0] = (uint32_t)quantize_one<false>(f.x, qz.scale, qz.zp_f, qz.has_zp != 0, qz.round_mode);
                            px[1] = (uint32_t)quantize_one<false>(f.y, qz.scale, qz.zp_f, qz.has_zp != 0, qz.round_mode);
                            px[2] = (uint32_t)quantize_one<false>(f.z, qz.scale, qz.zp_f, qz.has_zp != 0, qz.round_mode);
                            px[3] = (uint32_t)quantize_one<false>(f.w, qz.scale, qz.zp_f, qz.has_zp != 0, qz.round_mode);
                        }
                    } else {
                        const uint32_t w4 = *reinterpret_cast<const uint32_t*>(x + off);
                        px[0] = w4 & 0xffu; px[1] = (w4 >> 8) & 0xffu; px[2] = (w4 >> 16) & 0xffu; px[3] = w4 >> 24;
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int xx = xx0 + i;
                        if (xx >= 0 && xx < W)
                            px[i] = kQuant ? (uint32_t)quantize_one<false>(xf[off + i * es_w], qz.scale, qz.zp_f, qz.has_zp != 0, qz.round_mode)
                                           : (uint32_t)x[off + i * es_w];
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int pos = (dy * 2 + (i & 1)) * C + c;
                word[i >> 1][pos >> 2] |= px[i] << (8 * (pos & 3));
            }
        }
    }
    const int64_t o = ((int64_t)n * rows2 + r) * cols2 + b0;
    if (b0 >= 0) out[o] = make_uint4(word[0][0], word[0][1], word[0][2], word[0][3]);
    if (b0 + 1 < cols2) out[o + 1] = make_uint4(word[1][0], word[1][1], word[1][2], word[1][3]);
}

// OIHW weights -> the K layout of the space-to-depth path: row m, K index t * bk + u * 16 + (dy*2+dx) * C + c holds
// w[m][c][kh][kw] with kh = 2 (t + t0h) + dy + pad_top, kw = 2 (u + t0w) + dx + pad_left, zero where no such tap exists.
__global__ void __launch_bounds__(256) pack_weights_s2d_kernel(
        const uint8_t* __restrict__ w, int M, int C, int KH, int KW, int pt, int pl, int t0h, int t0w, int kw2, int bk, int k_total,
        uint8_t* __restrict__ out) {
    const int64_t total = (int64_t)M * k_total;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int k = (int)(i % k_total);
        const int m = (int)(i / k_total);
        const int t = k / bk, within = k % bk;
        const int u = within / 16, e = within % 16;
        uint8_t v = 0;
        if (u < kw2 && e < 4 * C) {
            const int d = e / C, c = e % C;
            const int kh = 2 * (t + t0h) + (d >> 1) + pt, kw = 2 * (u + t0w) + (d & 1) + pl;
            if (kh >= 0 && kh < KH && kw >= 0 && kw < KW) v = w[(((int64_t)m * C + c) * KH + kh) * KW + kw];
        }
        out[i] = v;
    }
}

// Depthwise OIHW weights [M][1][taps] -> dense diagonal blocks: row m, K index tap * 64 + (m % 64) holds w[m][tap], the
// other 63 entries of each tap are zero.
__global__ void __launch_bounds__(256) pack_weights_diag_kernel(const uint8_t* __restrict__ w, int M, int taps, uint8_t* __restrict__ out) {
    const int64_t total = (int64_t)M * taps * 64;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int j = (int)(i % 64);
        const int64_t r = i / 64;
        const int tap = (int)(r % taps);
        const int m = (int)(r / taps);
        out[i] = j == (m & 63) ? w[(int64_t)m * taps + tap] : (uint8_t)0;
    }
}

inline int blocks_for(int64_t threads_needed, int block = 256) {
    int64_t b = (threads_needed + block - 1) / block;
    if (b < 1) b = 1;
    if (b > 2147483647ll) b = 2147483647ll;
    return (int)b;
}

// ---------------------------------------------------------------------------------------------
// GEMM dispatch shared by MatMulInteger and QLinearMatMul.
// ---------------------------------------------------------------------------------------------
struct GemmWs {
    size_t bt_off, t_off, zbn_off, r_off, total;
    int bk;
    int64_t k_pad;
};

GemmWs gemm_ws_layout(int64_t M, int64_t N, int64_t K) {
    GemmWs w;
    w.bk = choose_bk((int)(K > (1 << 20) ? 128 : K));
    w.k_pad = (K + w.bk - 1) / w.bk * w.bk;
    size_t off = 0;
    w.bt_off = off; off += align_up((size_t)N * (size_t)w.k_pad, 256);
    w.t_off = off; off += align_up((size_t)N * 4, 256);
    w.zbn_off = off; off += align_up((size_t)N * 4, 256);
    w.r_off = off; off += align_up((size_t)M * 4, 256);
    w.total = off;
    return w;
}

bool gemm_tc_eligible(const void* a, int64_t M, int64_t N, int64_t K) {
    return K % 16 == 0 && K >= 16 && (reinterpret_cast<uintptr_t>(a) & 15u) == 0 && M >= 1 && N >= 1 && M < (1ll << 31) && N < (1ll << 31) &&
           K < (1ll << 31);
}

int gemm_dispatch(
        const char* op, const void* a, bool a_signed, const void* b, bool b_signed, int64_t batch, int64_t M, int64_t N, int64_t K,
        const ZpSpec& za, const ZpSpec& zb, const EpiArgs& epi, void* y, size_t y_elem, void* workspace, size_t workspace_bytes, int path,
        cudaStream_t s) {
    if (batch == 0 || M == 0 || N == 0) return CHXQ_OK;
    const bool tc_ok = gemm_tc_eligible(a, M, N, K) && ((M * K) % 16 == 0 || batch == 1);
    bool use_tc = path == CHXQ_PATH_TENSOR || (path == CHXQ_PATH_AUTO && tc_ok);
    if (path == CHXQ_PATH_TENSOR && !tc_ok)
        return set_error(CHXQ_ERR_UNSUPPORTED, "%s: tensor-core path needs K %% 16 == 0 and a 16-byte aligned A (M=%lld N=%lld K=%lld)", op,
                         (long long)M, (long long)N, (long long)K);
    if (use_tc) {
        const GemmWs ws = gemm_ws_layout(M, N, K);
        if (workspace == nullptr || workspace_bytes < ws.total || (reinterpret_cast<uintptr_t>(workspace) & 255u)) {
            if (path == CHXQ_PATH_TENSOR)
                return set_error(CHXQ_ERR_WORKSPACE, "%s: tensor-core path needs %zu bytes of 256-byte aligned workspace (got %zu)", op, ws.total,
                                 workspace_bytes);
            use_tc = false;
        }
    }
    if (!use_tc) return launch_gemm_simt(a, a_signed, b, b_signed, batch, M, N, K, za, zb, epi, y, s);

    const GemmWs ws = gemm_ws_layout(M, N, K);
    uint8_t* wsp = static_cast<uint8_t*>(workspace);
    uint8_t* bt = wsp + ws.bt_off;
    int32_t* T = reinterpret_cast<int32_t*>(wsp + ws.t_off);
    int32_t* zbn = reinterpret_cast<int32_t*>(wsp + ws.zbn_off);
    int32_t* R = reinterpret_cast<int32_t*>(wsp + ws.r_off);
    for (int64_t bi = 0; bi < batch; ++bi) {
        const uint8_t* ab = static_cast<const uint8_t*>(a) + bi * M * K;
        const uint8_t* bb = static_cast<const uint8_t*>(b) + bi * K * N;
        dim3 tgrid((unsigned)((N + 63) / 64), (unsigned)((ws.k_pad + 63) / 64));
        if (tgrid.y > 65535) return set_error(CHXQ_ERR_UNSUPPORTED, "%s: K too large for the repacking grid", op);
        // one pass over B: the K-major copy and, when a has a zero point, its column terms
        if (za.len > 0) CHXQ_CUDA(cudaMemsetAsync(T, 0, (size_t)N * 4, s));
        transpose_b_terms_kernel<<<tgrid, 256, 0, s>>>(bb, K, N, ws.k_pad, bt, za, a_signed ? 1 : 0, b_signed ? 1 : 0, za.len > 0 ? T : nullptr);
        if (zb.len > 0) {
            gemm_zb_kernel<<<blocks_for(N), 256, 0, s>>>(b_signed ? 1 : 0, N, zb, zbn);
            gemm_row_terms_kernel<<<blocks_for(M * 32), 256, 0, s>>>(ab, a_signed, M, K, za, R);
            count_launch(2);
        }
        CHXQ_LAUNCH_CHECK();
        TcProblem p{};
        p.a = ab; p.a_signed = a_signed; p.C = (int)K; p.a_cs = K; p.W = (int)M; p.H = 1; p.N = 1;
        p.b = bt; p.b_signed = b_signed; p.cols = (int)N; p.c_pad = (int)ws.k_pad; p.bk = ws.bk;
        p.KH = 1; p.KW = 1; p.pad_top = 0; p.pad_left = 0;
        p.Wo = (int)M; p.Ho = 1; p.No = 1; p.Wb = 128; p.Hb = 1; p.Nb = 1; p.bn = 0;
        p.y = static_cast<uint8_t*>(y) + (size_t)bi * M * N * y_elem;
        p.ldc = N;
        p.col_corr = za.len > 0 ? T : nullptr;
        p.col_scale = 1;
        p.col_mul = zb.len > 0 ? zbn : nullptr;
        p.row_corr = zb.len > 0 ? R : nullptr;
        p.epi = epi;
        p.alg_macs = (double)M * (double)N * (double)K;
        if (epi.residual) p.epi.residual = epi.residual + (size_t)bi * M * N;
        const int rc = launch_tc_igemm(p, s);
        if (rc != CHXQ_OK) return rc;
    }
    return CHXQ_OK;
}

int check_zp_len(const char* op, const char* which, const void* ptr, int64_t len, int64_t axis_len) {
    if (len == 0) return CHXQ_OK;
    if (ptr == nullptr) return set_error(CHXQ_ERR_INVALID_ARGUMENT, "%s: %s has length %lld but a null pointer", op, which, (long long)len);
    if (len != 1 && len != axis_len)
        return set_error(CHXQ_ERR_INVALID_ARGUMENT, "%s: %s has %lld elements; expected 1 or %lld", op, which, (long long)len, (long long)axis_len);
    return CHXQ_OK;
}

// ---------------------------------------------------------------------------------------------
// Convolution dispatch shared by ConvInteger and QLinearConv.
// ---------------------------------------------------------------------------------------------
int validate_geom(const char* op, const chxq_conv_geom* g) {
    CHXQ_CHECK_ARG(g != nullptr, "%s: null geometry", op);
    CHXQ_CHECK_ARG(g->N >= 0 && g->C > 0 && g->H > 0 && g->W > 0 && g->M > 0 && g->KH > 0 && g->KW > 0, "%s: bad tensor extents", op);
    CHXQ_CHECK_ARG(g->group >= 1 && g->C % g->group == 0 && g->M % g->group == 0, "%s: channels (%d, %d) not divisible by group %d", op, g->C,
                   g->M, g->group);
    CHXQ_CHECK_ARG(g->stride_h >= 1 && g->stride_w >= 1, "%s: strides must be positive", op);
    CHXQ_CHECK_ARG(is_q8(g->x_dtype) && is_q8(g->w_dtype), "%s: x and w must be uint8 or int8", op);
    CHXQ_CHECK_ARG((g->x_layout == CHXQ_NCHW || g->x_layout == CHXQ_NHWC) && (g->y_layout == CHXQ_NCHW || g->y_layout == CHXQ_NHWC),
                   "%s: unknown layout", op);
    const int Ho = (g->H + g->pad_top + g->pad_bottom - g->KH) / g->stride_h + 1;
    const int Wo = (g->W + g->pad_left + g->pad_right - g->KW) / g->stride_w + 1;
    CHXQ_CHECK_ARG(g->H + g->pad_top + g->pad_bottom >= g->KH && g->W + g->pad_left + g->pad_right >= g->KW, "%s: kernel larger than padded input",
                   op);
    CHXQ_CHECK_ARG(Ho == g->Ho && Wo == g->Wo, "%s: output extent (%d, %d) does not match the geometry (%d, %d)", op, g->Ho, g->Wo, Ho, Wo);
    CHXQ_CHECK_ARG(g->x_cstride == 0 || (g->x_layout == CHXQ_NHWC && g->x_cstride >= g->C), "%s: bad x channel stride", op);
    CHXQ_CHECK_ARG(g->y_cstride == 0 || (g->y_layout == CHXQ_NHWC && g->y_cstride >= g->M), "%s: bad y channel stride", op);
    return CHXQ_OK;
}

struct ConvWs {
    size_t pack_off, wsum_off, zw_off, flag_off, dw_off, pack_total;  // packed-weight blob (dw_off: depthwise 3x3 only, [M][12] raw taps)
    size_t im2col_bytes, rowsum_bytes;
};

ConvWs conv_ws_layout(const chxq_conv_geom& g, const TcConvPlan& pl) {
    ConvWs w{};
    size_t off = 0;
    w.pack_off = off; off += align_up((size_t)g.M * (size_t)pl.k_total, 1024);
    w.wsum_off = off; off += align_up((size_t)g.M * 4, 256);
    w.zw_off = off; off += align_up((size_t)g.M * 4, 256);
    w.flag_off = off; off += 256;
    w.dw_off = off;
    if (pl.diag && g.KH == 3 && g.KW == 3) off += align_up((size_t)g.M * 12, 256);  // the nine taps of a channel, 12 bytes apart (row-dp4a kernel)
    w.pack_total = off;
    const size_t rows = (size_t)g.N * g.Ho * g.Wo;
    w.im2col_bytes = pl.path == kTcS2d ? align_up((size_t)g.N * pl.rows2 * pl.cols2 * 16 + 256, 1024) : align_up(rows * (size_t)pl.a_pitch, 1024);
    w.rowsum_bytes = align_up(rows * 4, 256);
    return w;
}

bool needs_im2col(const chxq_conv_geom& g, const TcConvPlan& pl, int x_zp) {
    if (pl.path == kTcIm2col || pl.path == kTcS2d) return true;  // S2d: the repacked map lives in the same scratch
    const bool padded = g.pad_top || g.pad_left || g.pad_bottom || g.pad_right;
    return pl.path == kTcDirect && padded && x_zp != 0;
}

int pack_weights(const void* w, const chxq_conv_geom& g, const TcConvPlan& pl, const ZpSpec& zw, uint8_t* blob, cudaStream_t s) {
    const ConvWs L = conv_ws_layout(g, pl);
    const int taps = g.KH * g.KW;
    int32_t* flag = reinterpret_cast<int32_t*>(blob + L.flag_off);
    CHXQ_CUDA(cudaMemsetAsync(flag, 0, 4, s));
    const int cg = g.C / g.group;
    if (pl.diag) {
        pack_weights_diag_kernel<<<blocks_for((int64_t)g.M * pl.k_total), 256, 0, s>>>(static_cast<const uint8_t*>(w), g.M, taps, blob + L.pack_off);
        if (g.KH == 3 && g.KW == 3)  // [M][9] -> [M][12]
            CHXQ_CUDA(cudaMemcpy2DAsync(blob + L.dw_off, 12, w, 9, 9, (size_t)g.M, cudaMemcpyDeviceToDevice, s));
    }
    else if (pl.path == kTcS2d)
        pack_weights_s2d_kernel<<<blocks_for((int64_t)g.M * pl.k_total), 256, 0, s>>>(static_cast<const uint8_t*>(w), g.M, g.C, g.KH, g.KW, g.pad_top,
                                                                                      g.pad_left, pl.t0h, pl.t0w, pl.kw2, pl.bk, pl.k_total,
                                                                                      blob + L.pack_off);
    else
        pack_weights_kernel<<<blocks_for((int64_t)g.M * pl.k_total), 256, 0, s>>>(static_cast<const uint8_t*>(w), g.M, cg, taps, pl.c_pitch,
                                                                                  pl.k_total, blob + L.pack_off);
    weight_terms_kernel<<<blocks_for((int64_t)g.M * 32), 256, 0, s>>>(w, g.w_dtype == CHXQ_INT8, g.M, cg * taps, zw,
                                                                     reinterpret_cast<int32_t*>(blob + L.wsum_off),
                                                                     reinterpret_cast<int32_t*>(blob + L.zw_off), flag);
    count_launch(1);
    CHXQ_LAUNCH_CHECK();
    return CHXQ_OK;
}

// Runs a planned convolution on the tensor-core kernel from a packed weight blob.
int conv_tc_run(
        const void* x, const uint8_t* blob, const chxq_conv_geom& g, const TcConvPlan& pl, int x_zp, bool zw_zero, const EpiArgs& epi, void* y,
        uint8_t* scratch, size_t scratch_bytes, cudaStream_t s, const S2dQuant* quant_in = nullptr, const PoolSpec* pool = nullptr,
        TcProblem* plan_only = nullptr) {
    const ConvWs L = conv_ws_layout(g, pl);
    const int taps = g.KH * g.KW;
    const int64_t rows = (int64_t)g.N * g.Ho * g.Wo;
    if (rows == 0 && !plan_only) return CHXQ_OK;
    const bool im2col = needs_im2col(g, pl, x_zp);
    // Depthwise 3x3 over a zero-point-0 uint8 map: the CUDA-core row-dp4a kernel with TMA-staged rows (raw taps kept beside the
    // diagonal-block pack) moves each byte once instead of paying 64x the multiply-accumulates on the tensor pipe; measured at batch 512
    // it is 1.1x (7 x 7 maps) to 3.8x (112 x 112) faster.  chxq_tc_variant 1 also takes the plain-load row kernel for maps TMA cannot
    // describe, 2..5 keep the diagonal blocks.
    const int variant = tc_variant_value();
    if (pl.diag && zw_zero && !plan_only && !quant_in && !pool && !(variant >= 2 && variant <= 5) && depthwise3x3_eligible(g, x, y, x_zp, epi)) {
        if (depthwise3x3_staged_eligible(g, x, y, x_zp, epi)) return launch_depthwise3x3_staged(x, blob + L.dw_off, 12, 1, 0, g, epi, y, s);
        if (variant == 1) return launch_depthwise3x3(x, blob + L.dw_off, 12, 1, 0, g, epi, y, s);
    }
    // plan_only: describe the problem without launching anything -- only for layers that need no pass in front of the kernel
    if (plan_only && (pl.path != kTcDirect || im2col || !zw_zero || rows == 0))
        return set_error(CHXQ_ERR_UNSUPPORTED, "convolution: this layer needs a pass in front of the tensor-core kernel");
    if (g.group > 1 && (im2col || !zw_zero))
        return set_error(CHXQ_ERR_UNSUPPORTED,
                         "grouped convolution on the tensor-core path needs zero weight zero points and, with padding, a zero activation zero point");
    const size_t need = (im2col ? L.im2col_bytes : 0) + (zw_zero ? 0 : L.rowsum_bytes);
    if (need > 0 && (scratch == nullptr || scratch_bytes < need || (reinterpret_cast<uintptr_t>(scratch) & 255u)))
        return set_error(CHXQ_ERR_WORKSPACE, "convolution: tensor-core path needs %zu bytes of 256-byte aligned workspace (got %zu)", need,
                         scratch_bytes);
    const int64_t xcs = g.x_cstride > 0 ? g.x_cstride : g.C;
    const int64_t ycs = g.y_cstride > 0 ? g.y_cstride : g.M;
    const bool x_signed = g.x_dtype == CHXQ_INT8;
    TcProblem p{};
    int32_t* rowsum = nullptr;
    // element strides of the input map
    const bool nhwc = g.x_layout == CHXQ_NHWC;
    const int64_t es_c = nhwc ? 1 : (int64_t)g.H * g.W, es_w = nhwc ? xcs : 1, es_h = nhwc ? xcs * g.W : g.W,
                  es_n = nhwc ? xcs * g.W * g.H : (int64_t)g.C * g.H * g.W;
    if (pl.path == kTcS2d) {
        uint8_t* A = scratch;
        if (quant_in && !zw_zero) return set_error(CHXQ_ERR_UNSUPPORTED, "fused QuantizeLinear + QLinearConv needs zero weight zero points");
        if (quant_in && g.C == 3)
            s2d_repack_kernel<true, 3><<<blocks_for((int64_t)g.N * pl.rows2 * ((pl.cols2 + (pl.t0w & 1) + 1) / 2)), 256, 0, s>>>(
                    x, g.N, g.C, g.H, g.W, es_n, es_c, es_h, es_w, pl.t0h, pl.t0w, pl.rows2, pl.cols2, (uint32_t)(x_zp & 0xff), *quant_in,
                    reinterpret_cast<uint4*>(A));
        else if (quant_in)
            s2d_repack_kernel<true><<<blocks_for((int64_t)g.N * pl.rows2 * ((pl.cols2 + (pl.t0w & 1) + 1) / 2)), 256, 0, s>>>(
                    x, g.N, g.C, g.H, g.W, es_n, es_c, es_h, es_w, pl.t0h, pl.t0w, pl.rows2, pl.cols2, (uint32_t)(x_zp & 0xff), *quant_in,
                    reinterpret_cast<uint4*>(A));
        else
            s2d_repack_kernel<false><<<blocks_for((int64_t)g.N * pl.rows2 * ((pl.cols2 + (pl.t0w & 1) + 1) / 2)), 256, 0, s>>>(
                    x, g.N, g.C, g.H, g.W, es_n, es_c, es_h, es_w, pl.t0h, pl.t0w, pl.rows2, pl.cols2, (uint32_t)(x_zp & 0xff), S2dQuant{}, reinterpret_cast<uint4*>(A));
        CHXQ_LAUNCH_CHECK();
        if (!zw_zero) {
            rowsum = reinterpret_cast<int32_t*>(scratch + L.im2col_bytes);
            conv_possum_kernel<<<blocks_for(rows), 256, 0, s>>>(static_cast<const uint8_t*>(x), x_signed, g.N, g.H, g.W, g.C, es_n, es_c, es_h, es_w,
                                                              g.KH, g.KW, g.stride_h, g.stride_w, g.pad_top, g.pad_left, g.Ho, g.Wo, x_zp, rowsum);
            CHXQ_LAUNCH_CHECK();
        }
        // Overlapping rows: output column wo reads the bk bytes that start 16 wo bytes into block row (ho + t).
        p.a = A; p.C = pl.bk; p.a_cs = 16; p.W = g.Wo; p.H = pl.rows2; p.N = g.N;
        p.c_pad = pl.bk; p.KH = pl.kh2; p.KW = 1; p.pad_top = 0; p.pad_left = 0; p.sw = 1; p.sh = 1;
        p.a_row_bytes = (int64_t)pl.cols2 * 16;
        p.Wo = g.Wo; p.Ho = g.Ho; p.No = g.N; p.Wb = pl.Wb; p.Hb = pl.Hb; p.Nb = pl.Nb;
    } else if (im2col) {
        uint8_t* A = scratch;
        int rc = launch_im2col(x, g, pl.c_pitch, pl.a_pitch, x_zp & 0xff, A, s);
        if (rc != CHXQ_OK) return rc;
        if (!zw_zero) {
            rowsum = reinterpret_cast<int32_t*>(scratch + L.im2col_bytes);
            rowsum_matrix_kernel<<<blocks_for(rows * 32), 256, 0, s>>>(A, x_signed, rows, pl.a_pitch, taps * g.C * x_zp, rowsum);
            CHXQ_LAUNCH_CHECK();
        }
        if (rows >= (1ll << 31)) return set_error(CHXQ_ERR_UNSUPPORTED, "convolution: too many output positions");
        p.a = A; p.C = pl.a_pitch; p.a_cs = pl.a_pitch; p.W = (int)rows; p.H = 1; p.N = 1;
        p.c_pad = pl.k_total; p.KH = 1; p.KW = 1; p.pad_top = 0; p.pad_left = 0;
        p.Wo = (int)rows; p.Ho = 1; p.No = 1; p.Wb = 128; p.Hb = 1; p.Nb = 1;
    } else {
        if (!zw_zero) {
            rowsum = reinterpret_cast<int32_t*>(scratch);
            conv_possum_kernel<<<blocks_for(rows), 256, 0, s>>>(static_cast<const uint8_t*>(x), x_signed, g.N, g.H, g.W, g.C, es_n, es_c, es_h, es_w,
                                                              g.KH, g.KW, g.stride_h, g.stride_w, g.pad_top, g.pad_left, g.Ho, g.Wo, x_zp, rowsum);
            CHXQ_LAUNCH_CHECK();
        }
        p.a = x; p.C = g.C; p.a_cs = xcs;
        if (pl.Wb == 128 && taps == 1 && !pool) {  // a 1x1 convolution over the flattened map (the pooling form needs the image structure)
            p.W = (int)((int64_t)g.N * g.H * g.W); p.H = 1; p.N = 1;
            p.Wo = (int)rows; p.Ho = 1; p.No = 1;
        } else {
            p.W = g.W; p.H = g.H; p.N = g.N;
            p.Wo = g.Wo; p.Ho = g.Ho; p.No = g.N;
        }
        p.c_pad = pl.c_pitch; p.KH = g.KH; p.KW = g.KW; p.pad_top = g.pad_top; p.pad_left = g.pad_left;
        p.sw = g.stride_w; p.sh = g.stride_h;
        p.group_cols = pl.group_cols; p.group_cin = pl.group_cin;
        p.Wb = pl.Wb; p.Hb = pl.Hb; p.Nb = pl.Nb;
    }
    p.a_signed = x_signed;
    p.b = blob + L.pack_off; p.b_signed = g.w_dtype == CHXQ_INT8; p.cols = g.M; p.bk = pl.bk; p.bn = 0;
    p.y = y; p.ldc = ycs;
    p.col_corr = x_zp != 0 ? reinterpret_cast<const int32_t*>(blob + L.wsum_off) : nullptr;
    p.col_scale = x_zp;
    p.col_mul = zw_zero ? nullptr : reinterpret_cast<const int32_t*>(blob + L.zw_off);
    p.row_corr = zw_zero ? nullptr : rowsum;
    p.epi = epi;
    p.alg_macs = (double)rows * g.M * (g.C / g.group) * taps;
    if (pool) {
        if (!(pl.path == kTcS2d || (pl.path == kTcDirect && !im2col)) || p.No != g.N || epi.mode != kEpiRequant)
            return set_error(CHXQ_ERR_UNSUPPORTED, "fused max pooling: the convolution must run on the direct or space-to-depth tensor-core path");
        p.Wb = 16; p.Hb = 8; p.Nb = 1;  // the pooling form's tiles, whatever the output extents (edges are masked)
        p.pool_ho = pool->ho; p.pool_wo = pool->wo;
    }
    if (plan_only) {
        *plan_only = p;
        return CHXQ_OK;
    }
    return launch_tc_igemm(p, s);
}

// The reference's own signature is NCHW in, NCHW out (runtime/chxvm_defs.py:457-461, 466-469).  The tensor-core kernels read and
// write NHWC, so an NCHW call is run as: transpose x into scratch (skipped for maps of at most four channels, which the stem
// paths read as NCHW themselves), the NHWC convolution into scratch, transpose y back.  The two transposes move every activation
// byte once more; a caller that keeps its maps NHWC (chxq_conv_geom layouts) avoids them.
struct NchwPlan {
    chxq_conv_geom g2;   // the NHWC problem that actually runs
    bool x_transposed;
    size_t x_bytes, y_bytes, y_elem;
};

bool nchw_plan(const chxq_conv_geom& g, size_t y_elem, NchwPlan* out) {
    if (g.x_layout != CHXQ_NCHW || g.y_layout != CHXQ_NCHW || g.N > 65535) return false;
    NchwPlan pl{};
    pl.g2 = g;
    pl.y_elem = y_elem;
    pl.x_transposed = g.C > 4;
    if (pl.x_transposed) {
        pl.g2.x_layout = CHXQ_NHWC;
        pl.g2.x_cstride = (g.C + 15) / 16 * 16;
        pl.x_bytes = align_up((size_t)g.N * g.H * g.W * pl.g2.x_cstride, 1024);
    }
    pl.g2.y_layout = CHXQ_NHWC;
    pl.g2.y_cstride = (g.M + 15) / 16 * 16;
    pl.y_bytes = align_up((size_t)g.N * g.Ho * g.Wo * pl.g2.y_cstride * y_elem, 1024);
    if (plan_tc_conv(pl.g2).path == kTcNone) return false;
    *out = pl;
    return true;
}

size_t inner_conv_workspace(const chxq_conv_geom& g2) {
    const TcConvPlan pl = plan_tc_conv(g2);
    if (pl.path == kTcNone) return 0;
    const ConvWs L = conv_ws_layout(g2, pl);
    const bool padded = g2.pad_top || g2.pad_left || g2.pad_bottom || g2.pad_right;
    const size_t im2col = (pl.path == kTcIm2col || pl.path == kTcS2d || padded) ? L.im2col_bytes : 0;
    return L.pack_total + im2col + L.rowsum_bytes;
}

int conv_dispatch(
        const char* op, const void* x, const void* w, const chxq_conv_geom* g, int has_x_zp, int x_zp, const ZpSpec& zw, const EpiArgs& epi,
        void* y, void* workspace, size_t workspace_bytes, int path, cudaStream_t s) {
    int rc = validate_geom(op, g);
    if (rc != CHXQ_OK) return rc;
    if ((int64_t)g->N * g->M * g->Ho * g->Wo == 0) return CHXQ_OK;  // empty batch: nothing to compute
    CHXQ_CHECK_ARG(x && w && y, "%s: null buffer", op);
    CHXQ_CHECK_ARG(path == CHXQ_PATH_AUTO || path == CHXQ_PATH_SIMT || path == CHXQ_PATH_TENSOR, "%s: bad path", op);
    const int xz = has_x_zp ? x_zp : 0;
    // 3x3 depthwise with symmetric weights (a null zero-point array) over a zero-point-0 map: the row-dp4a kernel
    if (path == CHXQ_PATH_AUTO && g->group > 1 && zw.ptr == nullptr && depthwise3x3_eligible(*g, x, y, xz, epi)) {
        if (depthwise3x3_staged_eligible(*g, x, y, xz, epi)) return launch_depthwise3x3_staged(x, w, g->KH * g->KW, 1, 0, *g, epi, y, s);
        return launch_depthwise3x3(x, w, g->KH * g->KW, 1, 0, *g, epi, y, s);
    }
    if (path == CHXQ_PATH_AUTO && g->group > 1 && epi.mode == kEpiRequant && depthwise_eligible(*g, x, y, epi.residual))
        return launch_depthwise(x, w, *g, xz, zw.ptr, zw.len, epi, y, s);
    // NCHW in, NCHW out (the reference's signature): NHWC inside, transposes around it, when the caller's workspace has room.
    NchwPlan np;
    if (path != CHXQ_PATH_SIMT && epi.residual == nullptr && nchw_plan(*g, epi.mode == kEpiInt32 ? 4 : 1, &np)) {
        const size_t need = np.x_bytes + np.y_bytes + inner_conv_workspace(np.g2);
        const bool aligned_io = (reinterpret_cast<uintptr_t>(x) & 3u) == 0 && (reinterpret_cast<uintptr_t>(y) & 3u) == 0;
        if (workspace != nullptr && workspace_bytes >= need && (reinterpret_cast<uintptr_t>(workspace) & 255u) == 0 && aligned_io) {
            uint8_t* wsp = static_cast<uint8_t*>(workspace);
            const void* x2 = x;
            if (np.x_transposed) {
                rc = chxq_nchw_to_nhwc(x, 1, g->N, g->C, g->H, g->W, np.g2.x_cstride, wsp, s);
                if (rc != CHXQ_OK) return rc;
                x2 = wsp;
            }
            void* y2 = wsp + np.x_bytes;
            rc = conv_dispatch(op, x2, w, &np.g2, has_x_zp, x_zp, zw, epi, y2, wsp + np.x_bytes + np.y_bytes, workspace_bytes - np.x_bytes - np.y_bytes,
                               CHXQ_PATH_TENSOR, s);
            if (rc == CHXQ_OK) return chxq_nhwc_to_nchw(y2, (int)np.y_elem, g->N, g->M, g->Ho, g->Wo, np.g2.y_cstride, y, s);
            if (!(rc == CHXQ_ERR_UNSUPPORTED && path == CHXQ_PATH_AUTO)) return rc;
            // zero points or an epilogue the tensor-core kernels do not take: the general kernel reads NCHW directly
            return launch_conv_simt(x, w, *g, has_x_zp, x_zp, zw.ptr, zw.len, epi, y, s);
        }
        if (path == CHXQ_PATH_TENSOR)
            return set_error(CHXQ_ERR_WORKSPACE, "%s: the tensor-core path behind NCHW tensors needs %zu bytes of 256-byte aligned workspace (got %zu)", op,
                             need, workspace_bytes);
    }
    const TcConvPlan pl = plan_tc_conv(*g);
    const bool aligned = (reinterpret_cast<uintptr_t>(x) & 15u) == 0;
    bool use_tc = path != CHXQ_PATH_SIMT && pl.path != kTcNone && aligned;
    if (g->group > 1 && use_tc) {
        // the grouped tensor-core path covers uint8 round-half-up epilogues (and raw accumulators) with absent weight zero points
        const bool padded = g->pad_top || g->pad_left || g->pad_bottom || g->pad_right;
        const bool epi_ok = epi.mode != kEpiRequant || (!epi.rq.y_signed && epi.rq.round_mode == 0);
        if (zw.len != 0 || (padded && xz != 0) || !epi_ok) use_tc = false;
    }
    if (path == CHXQ_PATH_TENSOR && !use_tc)
        return set_error(CHXQ_ERR_UNSUPPORTED, "%s: the tensor-core path needs group == 1, NHWC output and a 16-byte aligned input", op);
    if (use_tc) {
        const ConvWs L = conv_ws_layout(*g, pl);
        const bool zw_zero = zw.len == 0;  // a zero point that is present is not read back: treat it as non-zero
        const size_t need = L.pack_total + (needs_im2col(*g, pl, xz) ? L.im2col_bytes : 0) + (zw_zero ? 0 : L.rowsum_bytes);
        if (workspace == nullptr || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255u)) {
            if (path == CHXQ_PATH_TENSOR)
                return set_error(CHXQ_ERR_WORKSPACE, "%s: tensor-core path needs %zu bytes of 256-byte aligned workspace (got %zu)", op, need,
                                 workspace_bytes);
            use_tc = false;
        } else {
            uint8_t* blob = static_cast<uint8_t*>(workspace);
            rc = pack_weights(w, *g, pl, zw, blob, s);
            if (rc != CHXQ_OK) return rc;
            return conv_tc_run(x, blob, *g, pl, xz, zw_zero, epi, y, blob + L.pack_total, workspace_bytes - L.pack_total, s);
        }
    }
    return launch_conv_simt(x, w, *g, has_x_zp, x_zp, zw.ptr, zw.len, epi, y, s);
}

int fill_requant(const char* op, const chxq_qconv_params* p, const chxq_conv_geom* g, EpiArgs* e) {
    CHXQ_CHECK_ARG(p != nullptr, "%s: null parameters", op);
    CHXQ_CHECK_ARG(is_q8(p->y_dtype), "%s: y_zero_point dtype must be uint8 or int8", op);
    const bool ys = p->y_dtype == CHXQ_INT8;
    CHXQ_CHECK_ARG(p->y_zero_point >= (ys ? -128 : 0) && p->y_zero_point <= (ys ? 127 : 255), "%s: y zero point %d out of range", op,
                   p->y_zero_point);
    const bool xs = g->x_dtype == CHXQ_INT8;
    CHXQ_CHECK_ARG(p->x_zero_point >= (xs ? -128 : 0) && p->x_zero_point <= (xs ? 127 : 255), "%s: x zero point %d out of range", op,
                   p->x_zero_point);
    // runtime/ops/quantize.cc:76-88: per-channel needs one scale and zero point per output channel, else both are 0-d.
    CHXQ_CHECK_ARG(p->w_params_len == 1 || p->w_params_len == g->M, "%s: w_scale / w_zero_point must have 1 or M=%d elements (got %lld)", op,
                   g->M, (long long)p->w_params_len);
    CHXQ_CHECK_ARG(p->w_scale != nullptr, "%s: null weight scale", op);  // a null w_zero_point says "every zero point is zero"
    CHXQ_CHECK_ARG(p->round_mode == CHXQ_ROUND_REF_HALF_UP || p->round_mode == CHXQ_ROUND_RNE, "%s: bad round_mode", op);
    CHXQ_CHECK_ARG(p->residual == nullptr || p->y_dtype == CHXQ_UINT8, "%s: the residual tail needs a uint8 output", op);
    memset(e, 0, sizeof(*e));
    e->mode = kEpiRequant;
    e->x_scale = p->x_scale;
    e->w_scale = p->w_scale;
    e->w_per_channel = p->w_params_len != 1;
    e->bias = p->bias;
    e->rq.y_scale = p->y_scale;
    e->rq.y_zp_f = (float)p->y_zero_point;
    e->rq.y_has_zp = p->y_zero_point != 0;
    e->rq.y_signed = ys;
    e->rq.round_mode = p->round_mode;
    e->rq.clamp_hi_q = p->clamp_hi_q;
    e->residual = static_cast<const uint8_t*>(p->residual);
    e->rq.res_scale = p->res_scale;
    e->rq.res_zp_f = (float)p->res_zero_point;
    e->rq.res_has_zp = p->res_zero_point != 0;
    e->rq.res_relu = p->res_relu;
    e->rq.out_scale = p->out_scale;
    e->rq.out_zp_f = (float)p->out_zero_point;
    e->rq.out_has_zp = p->out_zero_point != 0;
    finish_requant_params(&e->rq);
    if (p->fold_scales) {
        CHXQ_CHECK_ARG(p->y_dtype == CHXQ_UINT8, "%s: folded requantization needs a uint8 output", op);
        e->rq.fold = 1;
        e->rq.y_over_out = p->residual ? p->y_scale / p->out_scale : 0.f;
        e->rq.res_over_out = p->residual ? p->res_scale / p->out_scale : 0.f;
        finish_fold_params(&e->rq);
    }
    return CHXQ_OK;
}

}  // namespace
}  // namespace chxq

using namespace chxq;

extern "C" size_t chxq_matmul_integer_workspace(int64_t batch, int64_t M, int64_t N, int64_t K) {
    (void)batch;
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    return gemm_ws_layout(M, N, K).total;
}

extern "C" int chxq_matmul_integer(
        const void* a, int32_t a_dtype, const void* b, int32_t b_dtype, int64_t batch, int64_t M, int64_t N, int64_t K, const void* a_zero_point,
        int64_t a_zp_len, const void* b_zero_point, int64_t b_zp_len, int32_t* y, void* workspace, size_t workspace_bytes, int32_t path,
        void* stream) {
    CHXQ_CHECK_ARG(is_q8(a_dtype) && is_q8(b_dtype), "MatMulInteger: operands must be uint8 or int8 (got %d, %d)", a_dtype, b_dtype);
    CHXQ_CHECK_ARG(batch >= 0 && M >= 0 && N >= 0 && K >= 0, "MatMulInteger: negative extent");
    CHXQ_CHECK_ARG(path == CHXQ_PATH_AUTO || path == CHXQ_PATH_SIMT || path == CHXQ_PATH_TENSOR, "MatMulInteger: bad path");
    int rc = check_zp_len("MatMulInteger", "a_zero_point", a_zero_point, a_zp_len, K);
    if (rc != CHXQ_OK) return rc;
    rc = check_zp_len("MatMulInteger", "b_zero_point", b_zero_point, b_zp_len, N);
    if (rc != CHXQ_OK) return rc;
    if (batch * M * N == 0) return CHXQ_OK;
    CHXQ_CHECK_ARG(y != nullptr && (K == 0 || (a && b)), "MatMulInteger: null buffer");
    cudaStream_t s = as_stream(stream);
    if (K == 0) {
        CHXQ_CUDA(cudaMemsetAsync(y, 0, (size_t)batch * M * N * 4, s));
        return CHXQ_OK;
    }
    EpiArgs epi{};
    epi.mode = kEpiInt32;
    const ZpSpec za{a_zero_point, a_zp_len, 0}, zb{b_zero_point, b_zp_len, 0};
    return gemm_dispatch("MatMulInteger", a, a_dtype == CHXQ_INT8, b, b_dtype == CHXQ_INT8, batch, M, N, K, za, zb, epi, y, 4, workspace,
                         workspace_bytes, path, s);
}

// ---------------------------------------------------------------------------------------------
// MatMulInteger without any allocation: the scratch of the tensor-core path lives in a fixed device array.
// ---------------------------------------------------------------------------------------------
namespace chxq {
namespace {

// Scratch of chxq_matmul_integer_noalloc: transposed B, the two zero-point vectors and the row sums.  Every GPU that loads
// this library holds these bytes until the process exits.
static __device__ __align__(256) unsigned char g_noalloc_scratch[CHXQ_NOALLOC_SCRATCH_BYTES];

// In host code the array's name is only a stand-in for the symbol, not a device address: the address a kernel can use
// comes from cudaGetSymbolAddress, asked once per device with that device current.
int noalloc_scratch_ptr(void** out, cudaStream_t s) {
    static std::atomic<void*> cache[64] = {};  // two host threads may make the first call together: both store the same address
    int dev = 0;
    CHXQ_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return set_error(CHXQ_ERR_UNSUPPORTED, "MatMulInteger(noalloc): device ordinal %d out of range", dev);
    void* ptr = cache[dev].load(std::memory_order_acquire);
    if (ptr == nullptr) {
        // The lookup is not a stream operation and fails with an opaque error inside a capture: say what to do instead.
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(s, &cap) == cudaSuccess && cap != cudaStreamCaptureStatusNone)
            return set_error(CHXQ_ERR_UNSUPPORTED,
                             "MatMulInteger(noalloc): the first call on a device looks up the scratch array's address and cannot run "
                             "inside a stream capture; make one call on this device before capturing");
        cudaGetLastError();
        CHXQ_CUDA(cudaGetSymbolAddress(&ptr, g_noalloc_scratch));
        if (ptr == nullptr) return set_error(CHXQ_ERR_CUDA, "MatMulInteger(noalloc): the scratch symbol has no device address");
        cache[dev].store(ptr, std::memory_order_release);
    }
    *out = ptr;
    return CHXQ_OK;
}

}  // namespace
}  // namespace chxq

extern "C" int chxq_matmul_integer_noalloc(
        const void* a, int32_t a_dtype, const void* b, int32_t b_dtype, int64_t M, int64_t N, int64_t K, const void* a_zero_point,
        int64_t a_zp_len, const void* b_zero_point, int64_t b_zp_len, int32_t* y, void* stream) {
    CHXQ_CHECK_ARG(is_q8(a_dtype) && is_q8(b_dtype), "MatMulInteger(noalloc): operands must be uint8 or int8 (got %d, %d)", a_dtype, b_dtype);
    CHXQ_CHECK_ARG(M >= 0 && N >= 0 && K >= 0, "MatMulInteger(noalloc): negative extent");
    int rc = check_zp_len("MatMulInteger(noalloc)", "a_zero_point", a_zero_point, a_zp_len, K);
    if (rc != CHXQ_OK) return rc;
    rc = check_zp_len("MatMulInteger(noalloc)", "b_zero_point", b_zero_point, b_zp_len, N);
    if (rc != CHXQ_OK) return rc;
    if (M * N == 0) return CHXQ_OK;
    CHXQ_CHECK_ARG(y != nullptr && (K == 0 || (a && b)), "MatMulInteger(noalloc): null buffer");
    cudaStream_t s = as_stream(stream);
    if (K == 0) {
        CHXQ_CUDA(cudaMemsetAsync(y, 0, (size_t)M * N * 4, s));
        return CHXQ_OK;
    }
    EpiArgs epi{};
    epi.mode = kEpiInt32;
    const ZpSpec za{a_zero_point, a_zp_len, 0}, zb{b_zero_point, b_zp_len, 0};
    if (!gemm_tc_eligible(a, M, N, K)) {
        // shapes the tensor-core kernel does not take run on the CUDA-core kernel, which needs no scratch at all
        return launch_gemm_simt(a, a_dtype == CHXQ_INT8, b, b_dtype == CHXQ_INT8, 1, M, N, K, za, zb, epi, y, s);
    }
    const size_t need = gemm_ws_layout(M, N, K).total;
    if (need > (size_t)CHXQ_NOALLOC_SCRATCH_BYTES)
        return set_error(CHXQ_ERR_WORKSPACE,
                         "MatMulInteger(noalloc): M=%lld N=%lld K=%lld needs %zu bytes of scratch, the fixed array holds %d; use "
                         "chxq_matmul_integer with a caller-provided workspace",
                         (long long)M, (long long)N, (long long)K, need, (int)CHXQ_NOALLOC_SCRATCH_BYTES);
    void* scratch = nullptr;
    rc = noalloc_scratch_ptr(&scratch, s);
    if (rc != CHXQ_OK) return rc;
    return gemm_dispatch("MatMulInteger(noalloc)", a, a_dtype == CHXQ_INT8, b, b_dtype == CHXQ_INT8, 1, M, N, K, za, zb, epi, y, 4, scratch,
                         (size_t)CHXQ_NOALLOC_SCRATCH_BYTES, CHXQ_PATH_TENSOR, s);
}

extern "C" int chxq_qlinear_matmul(
        const void* a, int32_t a_dtype, float a_scale, int32_t a_zero_point, const void* b, int32_t b_dtype, float b_scale, int32_t b_zero_point,
        float y_scale, int32_t y_zero_point, int32_t y_dtype, int64_t M, int64_t N, int64_t K, int32_t round_mode, void* y, void* workspace,
        size_t workspace_bytes, int32_t path, void* stream) {
    CHXQ_CHECK_ARG(is_q8(a_dtype) && is_q8(b_dtype) && is_q8(y_dtype), "QLinearMatMul: a, b and y must be uint8 or int8");
    CHXQ_CHECK_ARG(M >= 0 && N >= 0 && K > 0, "QLinearMatMul: bad extents");
    CHXQ_CHECK_ARG(path == CHXQ_PATH_AUTO || path == CHXQ_PATH_SIMT || path == CHXQ_PATH_TENSOR, "QLinearMatMul: bad path");
    CHXQ_CHECK_ARG(round_mode == CHXQ_ROUND_REF_HALF_UP || round_mode == CHXQ_ROUND_RNE, "QLinearMatMul: bad round_mode");
    const bool ys = y_dtype == CHXQ_INT8;
    CHXQ_CHECK_ARG(y_zero_point >= (ys ? -128 : 0) && y_zero_point <= (ys ? 127 : 255), "QLinearMatMul: y zero point %d out of range", y_zero_point);
    if (M * N == 0) return CHXQ_OK;
    CHXQ_CHECK_ARG(a && b && y, "QLinearMatMul: null buffer");
    EpiArgs epi{};
    epi.mode = kEpiRequant;
    epi.w_scale = nullptr;
    epi.mult_scalar = a_scale * b_scale;  // fp32 product, as dequantized operands carry it
    epi.rq.y_scale = y_scale;
    epi.rq.y_zp_f = (float)y_zero_point;
    epi.rq.y_has_zp = y_zero_point != 0;
    epi.rq.y_signed = ys;
    epi.rq.round_mode = round_mode;
    epi.rq.clamp_hi_q = -1;
    finish_requant_params(&epi.rq);
    const ZpSpec za{nullptr, a_zero_point != 0 ? 1 : 0, a_zero_point}, zb{nullptr, b_zero_point != 0 ? 1 : 0, b_zero_point};
    return gemm_dispatch("QLinearMatMul", a, a_dtype == CHXQ_INT8, b, b_dtype == CHXQ_INT8, 1, M, N, K, za, zb, epi, y, 1, workspace,
                         workspace_bytes, path, as_stream(stream));
}

extern "C" int chxq_conv_resolve_geometry(
        int32_t N, int32_t C, int32_t H, int32_t W, int32_t M, int32_t Cg, int32_t KH, int32_t KW, const int64_t* strides, int32_t n_strides,
        const int64_t* pads, int32_t n_pads, int32_t group, const char* auto_pad, chxq_conv_geom* out) {
    CHXQ_CHECK_ARG(out != nullptr, "conv geometry: null output");
    CHXQ_CHECK_ARG(group >= 1 && (int64_t)Cg * group == C, "conv geometry: weight has %d input channels per group, input has %d channels in %d groups",
                   Cg, C, group);
    CHXQ_CHECK_ARG(n_strides == 0 || n_strides == 2, "conv geometry: strides must be empty or have one value per spatial dim");
    CHXQ_CHECK_ARG(n_pads == 0 || n_pads == 2, "conv geometry: pads must be empty or have one value per spatial dim (begin == end)");
    memset(out, 0, sizeof(*out));
    // ComplementStride / ComplementPad (runtime/chainerx_util.cc:180-200): empty -> 1 / 0.
    const int64_t sh = n_strides ? strides[0] : 1, sw = n_strides ? strides[1] : 1;
    int64_t pt = n_pads ? pads[0] : 0, pl = n_pads ? pads[1] : 0;
    int64_t pb = pt, pr = pl;
    CHXQ_CHECK_ARG(sh >= 1 && sw >= 1, "conv geometry: strides must be positive");
    if (auto_pad && auto_pad[0] && strcmp(auto_pad, "NOTSET") != 0) {
        // CalculateAutoPad (runtime/chainerx_util.cc:276-311) knows SAME_UPPER only.
        CHXQ_CHECK_ARG(strcmp(auto_pad, "SAME_UPPER") == 0, "conv geometry: auto_pad '%s' is not supported (SAME_UPPER only)", auto_pad);
        const int64_t th = (H + sh - 1) / sh, tw = (W + sw - 1) / sw;
        const int64_t nh = (th - 1) * sh + KH - H, nw = (tw - 1) * sw + KW - W;
        pt = nh / 2; pb = nh - pt;
        pl = nw / 2; pr = nw - pl;
        if (!(pb > 0 || pr > 0)) {  // no end padding is materialised: begin pads apply to both sides
            pb = pt;
            pr = pl;
        }
    }
    CHXQ_CHECK_ARG(H + pt + pb >= KH && W + pl + pr >= KW, "conv geometry: kernel larger than padded input");
    out->N = N; out->C = C; out->H = H; out->W = W; out->M = M; out->KH = KH; out->KW = KW;
    out->stride_h = (int32_t)sh; out->stride_w = (int32_t)sw;
    out->pad_top = (int32_t)pt; out->pad_left = (int32_t)pl; out->pad_bottom = (int32_t)pb; out->pad_right = (int32_t)pr;
    out->group = group;
    out->Ho = (int32_t)((H + pt + pb - KH) / sh + 1);
    out->Wo = (int32_t)((W + pl + pr - KW) / sw + 1);
    out->x_dtype = CHXQ_UINT8; out->w_dtype = CHXQ_INT8;
    out->x_layout = CHXQ_NCHW; out->y_layout = CHXQ_NCHW;
    return CHXQ_OK;
}

extern "C" size_t chxq_conv_workspace(const chxq_conv_geom* g) {
    if (!g || validate_geom("conv workspace", g) != CHXQ_OK) return 0;
    NchwPlan np;
    if (nchw_plan(*g, 4, &np)) return np.x_bytes + np.y_bytes + inner_conv_workspace(np.g2);  // sized for int32 outputs (ConvInteger), the larger case
    const TcConvPlan pl = plan_tc_conv(*g);
    if (pl.path == kTcNone) return 0;
    const ConvWs L = conv_ws_layout(*g, pl);
    const bool padded = g->pad_top || g->pad_left || g->pad_bottom || g->pad_right;
    // Worst case over zero points: an explicit im2col matrix when the direct path cannot express the
    // padding value, and per-position sums when the weight zero point is non-zero.
    const size_t im2col = (pl.path == kTcIm2col || pl.path == kTcS2d || padded) ? L.im2col_bytes : 0;
    return L.pack_total + im2col + L.rowsum_bytes;
}

extern "C" size_t chxq_conv_packed_workspace(const chxq_conv_geom* g, int32_t x_zero_point, int32_t packed_flags) {
    if (!g || validate_geom("conv workspace", g) != CHXQ_OK) return 0;
    const TcConvPlan pl = plan_tc_conv(*g);
    if (pl.path == kTcNone) return 0;
    const ConvWs L = conv_ws_layout(*g, pl);
    return (needs_im2col(*g, pl, x_zero_point) ? L.im2col_bytes : 0) + ((packed_flags & 2) ? 0 : L.rowsum_bytes);
}

extern "C" int chxq_conv_integer(
        const void* x, const void* w, const chxq_conv_geom* g, int32_t has_x_zp, int32_t x_zero_point, const void* w_zero_point,
        int64_t w_zp_len, int32_t* y, void* workspace, size_t workspace_bytes, int32_t path, void* stream) {
    int rc = validate_geom("ConvInteger", g);
    if (rc != CHXQ_OK) return rc;
    rc = check_zp_len("ConvInteger", "w_zero_point", w_zero_point, w_zp_len, g->M);
    if (rc != CHXQ_OK) return rc;
    EpiArgs epi{};
    epi.mode = kEpiInt32;
    const ZpSpec zw{w_zero_point, w_zp_len, 0};
    return conv_dispatch("ConvInteger", x, w, g, has_x_zp, x_zero_point, zw, epi, y, workspace, workspace_bytes, path, as_stream(stream));
}

extern "C" int chxq_conv_integer_dev(
        const void* x, const void* w, const chxq_conv_geom* g, const void* x_zero_point, const void* w_zero_point, int64_t w_zp_len, int32_t* y,
        void* stream) {
    int rc = validate_geom("ConvInteger", g);
    if (rc != CHXQ_OK) return rc;
    rc = check_zp_len("ConvInteger", "w_zero_point", w_zero_point, w_zp_len, g->M);
    if (rc != CHXQ_OK) return rc;
    if ((int64_t)g->N * g->M * g->Ho * g->Wo == 0) return CHXQ_OK;
    CHXQ_CHECK_ARG(x && w && y && x_zero_point, "ConvInteger: null buffer");
    EpiArgs epi{};
    epi.mode = kEpiInt32;
    return launch_conv_simt(x, w, *g, 1, 0, w_zero_point, w_zp_len, epi, y, as_stream(stream), x_zero_point);
}

extern "C" int chxq_qlinear_conv(
        const void* x, const void* w, const chxq_conv_geom* g, const chxq_qconv_params* p, void* y, void* workspace, size_t workspace_bytes,
        int32_t path, void* stream) {
    int rc = validate_geom("QLinearConv", g);
    if (rc != CHXQ_OK) return rc;
    EpiArgs epi;
    rc = fill_requant("QLinearConv", p, g, &epi);
    if (rc != CHXQ_OK) return rc;
    const ZpSpec zw{p->w_zero_point, p->w_zero_point ? p->w_params_len : 0, 0};
    return conv_dispatch("QLinearConv", x, w, g, 1, p->x_zero_point, zw, epi, y, workspace, workspace_bytes, path, as_stream(stream));
}

extern "C" size_t chxq_conv_prepack_bytes(const chxq_conv_geom* g) {
    if (!g || validate_geom("conv prepack", g) != CHXQ_OK) return 0;
    const TcConvPlan pl = plan_tc_conv(*g);
    if (pl.path == kTcNone) return 0;
    return conv_ws_layout(*g, pl).pack_total;
}

extern "C" int chxq_conv_prepack(
        const void* w, const chxq_conv_geom* g, const void* w_zero_point, int64_t w_zp_len, void* packed, size_t packed_bytes, int32_t* eligible,
        void* stream) {
    int rc = validate_geom("conv prepack", g);
    if (rc != CHXQ_OK) return rc;
    CHXQ_CHECK_ARG(eligible != nullptr, "conv prepack: null eligible pointer");
    *eligible = 0;
    rc = check_zp_len("conv prepack", "w_zero_point", w_zero_point, w_zp_len, g->M);
    if (rc != CHXQ_OK) return rc;
    const TcConvPlan pl = plan_tc_conv(*g);
    if (pl.path == kTcNone) return CHXQ_OK;
    const ConvWs L = conv_ws_layout(*g, pl);
    CHXQ_CHECK_ARG(w && packed && packed_bytes >= L.pack_total && (reinterpret_cast<uintptr_t>(packed) & 255u) == 0,
                   "conv prepack: need %zu bytes of 256-byte aligned memory", L.pack_total);
    cudaStream_t s = as_stream(stream);
    uint8_t* blob = static_cast<uint8_t*>(packed);
    const ZpSpec zw{w_zero_point, w_zp_len, 0};
    rc = pack_weights(w, *g, pl, zw, blob, s);
    if (rc != CHXQ_OK) return rc;
    int32_t flag = 0;
    CHXQ_CUDA(cudaMemcpyAsync(&flag, blob + L.flag_off, 4, cudaMemcpyDeviceToHost, s));
    CHXQ_CUDA(cudaStreamSynchronize(s));
    *eligible = 1 | (flag == 0 ? 2 : 0);
    return CHXQ_OK;
}

static int packed_common(const char* op, const void* x, const void* packed, const chxq_conv_geom* g, int32_t packed_flags, TcConvPlan* pl) {
    int rc = validate_geom(op, g);
    if (rc != CHXQ_OK) return rc;
    CHXQ_CHECK_ARG(x && packed, "%s: null buffer", op);
    CHXQ_CHECK_ARG((packed_flags & 1) != 0, "%s: these weights were not packed for the tensor-core path", op);
    *pl = plan_tc_conv(*g);
    if (pl->path == kTcNone || (reinterpret_cast<uintptr_t>(x) & 15u))
        return set_error(CHXQ_ERR_UNSUPPORTED, "%s: geometry or input alignment is not eligible for the tensor-core path", op);
    return CHXQ_OK;
}

extern "C" int chxq_qlinear_conv_packed(
        const void* x, const void* packed, const chxq_conv_geom* g, const chxq_qconv_params* p, int32_t packed_flags, void* y, void* workspace,
        size_t workspace_bytes, void* stream) {
    TcConvPlan pl;
    int rc = packed_common("QLinearConv(packed)", x, packed, g, packed_flags, &pl);
    if (rc != CHXQ_OK) return rc;
    CHXQ_CHECK_ARG(y != nullptr, "QLinearConv(packed): null output");
    EpiArgs epi;
    rc = fill_requant("QLinearConv(packed)", p, g, &epi);
    if (rc != CHXQ_OK) return rc;
    return conv_tc_run(x, static_cast<const uint8_t*>(packed), *g, pl, p->x_zero_point, (packed_flags & 2) != 0, epi, y,
                       static_cast<uint8_t*>(workspace), workspace_bytes, as_stream(stream));
}

// QLinearConv (g1, p1) followed by the 1x1 / stride-1 QLinearConv (g2, p2) that is its only reader, as one kernel: the map between
// them is requantized tile by tile into shared memory and never written.
extern "C" int chxq_qlinear_conv_chain_packed(
        const void* x, const void* packed1, const chxq_conv_geom* g1, const chxq_qconv_params* p1, int32_t packed_flags1, const void* packed2,
        const chxq_conv_geom* g2, const chxq_qconv_params* p2, int32_t packed_flags2, void* y, void* stream) {
    const char* op = "QLinearConv+QLinearConv(packed)";
    TcConvPlan pl1, pl2;
    int rc = packed_common(op, x, packed1, g1, packed_flags1, &pl1);
    if (rc != CHXQ_OK) return rc;
    rc = packed_common(op, x, packed2, g2, packed_flags2, &pl2);
    if (rc != CHXQ_OK) return rc;
    CHXQ_CHECK_ARG(y != nullptr && p1 != nullptr && p2 != nullptr, "%s: null argument", op);
    CHXQ_CHECK_ARG(g2->KH == 1 && g2->KW == 1 && g2->stride_h == 1 && g2->stride_w == 1 && g2->pad_top == 0 && g2->pad_left == 0 &&
                           g2->pad_bottom == 0 && g2->pad_right == 0 && g2->group == 1,
                   "%s: the second convolution must be 1x1, stride 1, without padding or groups", op);
    CHXQ_CHECK_ARG(g2->N == g1->N && g2->C == g1->M && g2->H == g1->Ho && g2->W == g1->Wo, "%s: the second convolution does not read the first one's output", op);
    CHXQ_CHECK_ARG(g2->x_dtype == CHXQ_UINT8 && p1->y_dtype == CHXQ_UINT8, "%s: the map between the convolutions must be uint8", op);
    CHXQ_CHECK_ARG(p2->x_scale == p1->y_scale && p2->x_zero_point == p1->y_zero_point,
                   "%s: the second convolution's input scale and zero point must be the first one's output scale and zero point", op);
    CHXQ_CHECK_ARG(p1->residual == nullptr, "%s: only the second convolution may carry a residual tail", op);
    if (g1->x_layout != CHXQ_NHWC || g2->y_layout != CHXQ_NHWC || (packed_flags1 & 2) == 0 || (packed_flags2 & 2) == 0 || p1->x_zero_point != 0 ||
        p2->x_zero_point != 0 || !p1->fold_scales || !p2->fold_scales)
        return set_error(CHXQ_ERR_UNSUPPORTED, "%s: needs NHWC maps, zero weight and activation zero points and folded requantizations", op);
    EpiArgs e1, e2;
    rc = fill_requant(op, p1, g1, &e1);
    if (rc != CHXQ_OK) return rc;
    rc = fill_requant(op, p2, g2, &e2);
    if (rc != CHXQ_OK) return rc;
    TcProblem q1, q2;
    rc = conv_tc_run(x, static_cast<const uint8_t*>(packed1), *g1, pl1, 0, true, e1, /*y=*/y, nullptr, 0, as_stream(stream), nullptr, nullptr, &q1);
    if (rc != CHXQ_OK) return rc;
    rc = conv_tc_run(x, static_cast<const uint8_t*>(packed2), *g2, pl2, 0, true, e2, y, nullptr, 0, as_stream(stream), nullptr, nullptr, &q2);
    if (rc != CHXQ_OK) return rc;
    return launch_tc_chain_igemm(q1, q2, as_stream(stream));
}

// QuantizeLinear(x; p->x_scale, p->x_zero_point, uint8, reference rounding or round-half-to-even) fused into the packed
// QLinearConv that consumes it: for stride-2 stems (the space-to-depth path), whose repack pass quantizes on the fly.
extern "C" int chxq_quantize_qlinear_conv_packed(
        const float* x, int32_t quant_round_mode, const void* packed, const chxq_conv_geom* g, const chxq_qconv_params* p, int32_t packed_flags, void* y,
        void* workspace, size_t workspace_bytes, void* stream) {
    TcConvPlan pl;
    int rc = packed_common("QuantizeLinear+QLinearConv(packed)", x, packed, g, packed_flags, &pl);
    if (rc != CHXQ_OK) return rc;
    CHXQ_CHECK_ARG(y != nullptr, "QuantizeLinear+QLinearConv(packed): null output");
    CHXQ_CHECK_ARG(g->x_dtype == CHXQ_UINT8, "QuantizeLinear+QLinearConv(packed): the quantized activation type must be uint8");
    CHXQ_CHECK_ARG(quant_round_mode == CHXQ_ROUND_REF_HALF_UP || quant_round_mode == CHXQ_ROUND_RNE, "QuantizeLinear+QLinearConv(packed): bad rounding mode");
    if (pl.path != kTcS2d)
        return set_error(CHXQ_ERR_UNSUPPORTED, "QuantizeLinear+QLinearConv(packed): only stride-2 convolutions over at most 4 channels fuse their QuantizeLinear");
    EpiArgs epi;
    rc = fill_requant("QuantizeLinear+QLinearConv(packed)", p, g, &epi);
    if (rc != CHXQ_OK) return rc;
    CHXQ_CHECK_ARG(p->x_zero_point >= 0 && p->x_zero_point <= 255 && p->x_scale > 0.f, "QuantizeLinear+QLinearConv(packed): bad activation scale / zero point");
    const S2dQuant qz{p->x_scale, (float)p->x_zero_point, p->x_zero_point != 0, quant_round_mode, make_qdiv(p->x_scale)};
    return conv_tc_run(x, static_cast<const uint8_t*>(packed), *g, pl, p->x_zero_point, (packed_flags & 2) != 0, epi, y,
                       static_cast<uint8_t*>(workspace), workspace_bytes, as_stream(stream), &qz);
}

// QLinearConv (with its QuantizeLinear in front when x_is_f32) followed by MaxPool(kernel 3, stride 2, pad 0) as one kernel.
extern "C" int chxq_qlinear_conv_maxpool_packed(
        const void* x, int32_t x_is_f32, int32_t quant_round_mode, const void* packed, const chxq_conv_geom* g, const chxq_qconv_params* p,
        int32_t packed_flags, int32_t pool_kernel, int32_t pool_stride, int32_t pool_pad, int32_t cover_all, void* y, void* workspace,
        size_t workspace_bytes, void* stream) {
    const char* op = "QLinearConv+MaxPool(packed)";
    TcConvPlan pl;
    int rc = packed_common(op, x, packed, g, packed_flags, &pl);
    if (rc != CHXQ_OK) return rc;
    CHXQ_CHECK_ARG(y != nullptr, "%s: null output", op);
    if (pool_kernel != 3 || pool_stride != 2 || pool_pad != 0)
        return set_error(CHXQ_ERR_UNSUPPORTED, "%s: only kernel 3, stride 2, pad 0 pooling is fused", op);
    EpiArgs epi;
    rc = fill_requant(op, p, g, &epi);
    if (rc != CHXQ_OK) return rc;
    if (epi.residual != nullptr || epi.rq.y_signed) return set_error(CHXQ_ERR_UNSUPPORTED, "%s: uint8 output without a residual only", op);
    const int extra = cover_all ? 1 : 0;
    if (g->Ho < 3 || g->Wo < 3) return set_error(CHXQ_ERR_UNSUPPORTED, "%s: the convolution's output is smaller than the pooling window", op);
    const PoolSpec pool{(g->Ho - 3 + extra) / 2 + 1, (g->Wo - 3 + extra) / 2 + 1};
    if (x_is_f32) {
        CHXQ_CHECK_ARG(g->x_dtype == CHXQ_UINT8, "%s: the quantized activation type must be uint8", op);
        CHXQ_CHECK_ARG(quant_round_mode == CHXQ_ROUND_REF_HALF_UP || quant_round_mode == CHXQ_ROUND_RNE, "%s: bad rounding mode", op);
        if (pl.path != kTcS2d)
            return set_error(CHXQ_ERR_UNSUPPORTED, "%s: only stride-2 convolutions over at most 4 channels fuse their QuantizeLinear", op);
        CHXQ_CHECK_ARG(p->x_zero_point >= 0 && p->x_zero_point <= 255 && p->x_scale > 0.f, "%s: bad activation scale / zero point", op);
        const S2dQuant qz{p->x_scale, (float)p->x_zero_point, p->x_zero_point != 0, quant_round_mode, make_qdiv(p->x_scale)};
        return conv_tc_run(x, static_cast<const uint8_t*>(packed), *g, pl, p->x_zero_point, (packed_flags & 2) != 0, epi, y,
                           static_cast<uint8_t*>(workspace), workspace_bytes, as_stream(stream), &qz, &pool);
    }
    return conv_tc_run(x, static_cast<const uint8_t*>(packed), *g, pl, p->x_zero_point, (packed_flags & 2) != 0, epi, y,
                       static_cast<uint8_t*>(workspace), workspace_bytes, as_stream(stream), nullptr, &pool);
}

extern "C" int chxq_conv_integer_packed(
        const void* x, const void* packed, const chxq_conv_geom* g, int32_t has_x_zp, int32_t x_zero_point, int32_t packed_flags, int32_t* y,
        void* workspace, size_t workspace_bytes, void* stream) {
    TcConvPlan pl;
    int rc = packed_common("ConvInteger(packed)", x, packed, g, packed_flags, &pl);
    if (rc != CHXQ_OK) return rc;
    CHXQ_CHECK_ARG(y != nullptr, "ConvInteger(packed): null output");
    EpiArgs epi{};
    epi.mode = kEpiInt32;
    return conv_tc_run(x, static_cast<const uint8_t*>(packed), *g, pl, has_x_zp ? x_zero_point : 0, (packed_flags & 2) != 0, epi, y,
                       static_cast<uint8_t*>(workspace), workspace_bytes, as_stream(stream));
}
