// Model preparation on the device: Conv + BatchNormalization folding (compiler/merge.cc:142-215) and the weight quantizer
// (compiler/quantize.cc:70-129) as one pass over the fp32 weights.  Every arithmetic step is the single-rounded fp32
// operation the host implementations perform (no fused multiply-add, IEEE division and square root), so the quantized weights,
// scales, zero points and folded biases are bit-identical to chxq_quantize_weights_host and to a NumPy evaluation of the merge.
//
// Layout: w is [M, inner] row-major (OIHW with inner = C/g * KH * KW); one block of 256 threads per output channel.
//   pass 1: s[m] = gamma[m] / sqrt(var[m] + eps); w'[m, :] = w[m, :] * s[m]; per-channel min / max of w' (both widened to
//           include 0, compiler/quantize.cc:71-72); b'[m] = (b[m] - mean[m]) * s[m] + beta[m].
//   pass 2: (rmin, rmax) = the channel's own pair, or the reduction over all channels for per-tensor quantization; scale,
//           zero point and the rounded quotients.
// Algorithmic traffic: 4 B read per weight in each pass (the second read is served from L2 for every layer of the networks
// measured here) + 1 B written; HBM-bound, but run once per model, not per inference.
#include <math.h>

#include "common.h"

namespace chxq {
namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float bn_factor(const float* gamma, const float* var, float eps, int m) {
    return gamma ? __fdiv_rn(gamma[m], __fsqrt_rn(__fadd_rn(var[m], eps))) : 1.0f;
}

__device__ __forceinline__ void block_minmax(float& mn, float& mx) {
    __shared__ float smn[kThreads / 32], smx[kThreads / 32];
    for (int o = 16; o > 0; o >>= 1) {
        mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();  // the shared arrays may still be read by a previous call
    if (lane == 0) {
        smn[warp] = mn;
        smx[warp] = mx;
    }
    __syncthreads();
    mn = smn[0];
    mx = smx[0];
#pragma unroll
    for (int i = 1; i < kThreads / 32; ++i) {
        mn = fminf(mn, smn[i]);
        mx = fmaxf(mx, smx[i]);
    }
}

__global__ void __launch_bounds__(kThreads) fold_minmax_kernel(
        const float* __restrict__ w, int64_t inner, const float* __restrict__ gamma, const float* __restrict__ beta, const float* __restrict__ mean,
        const float* __restrict__ var, float eps, const float* __restrict__ conv_bias, float* __restrict__ folded_w, float* __restrict__ folded_bias,
        float* __restrict__ cmin, float* __restrict__ cmax) {
    const int m = blockIdx.x;
    const float s = bn_factor(gamma, var, eps, m);
    const float* row = w + (int64_t)m * inner;
    float mn = 0.f, mx = 0.f;
    for (int64_t i = threadIdx.x; i < inner; i += kThreads) {
        const float v = gamma ? __fmul_rn(row[i], s) : row[i];
        if (folded_w) folded_w[(int64_t)m * inner + i] = v;
        mn = v < mn ? v : mn;  // the host's comparisons: a NaN weight never replaces the running value
        mx = v > mx ? v : mx;
    }
    block_minmax(mn, mx);
    if (threadIdx.x == 0) {
        cmin[m] = mn;
        cmax[m] = mx;
        if (folded_bias && gamma) {
            const float b = conv_bias ? conv_bias[m] : 0.f;
            folded_bias[m] = __fadd_rn(__fmul_rn(__fsub_rn(b, mean[m]), s), beta[m]);
        }
    }
}

template <bool kInt8>
__global__ void __launch_bounds__(kThreads) quantize_weights_kernel(
        const float* __restrict__ w, int M, int64_t inner, const float* __restrict__ gamma, const float* __restrict__ var, float eps,
        const float* __restrict__ cmin, const float* __restrict__ cmax, int per_channel, void* __restrict__ q, float* __restrict__ scales,
        int32_t* __restrict__ zero_points) {
    const int m = blockIdx.x;
    float rmin, rmax;
    if (per_channel) {
        rmin = cmin[m];
        rmax = cmax[m];
    } else {
        rmin = 0.f;
        rmax = 0.f;
        for (int i = threadIdx.x; i < M; i += kThreads) {
            rmin = fminf(rmin, cmin[i]);
            rmax = fmaxf(rmax, cmax[i]);
        }
        block_minmax(rmin, rmax);
    }
    const float s = bn_factor(gamma, var, eps, m);
    const float* row = w + (int64_t)m * inner;
    float scale;
    int32_t zp = 0;
    if (kInt8) {
        scale = __fdiv_rn(__fmul_rn(fmaxf(fabsf(rmin), fabsf(rmax)), 2.0f), 254.f);
    } else {
        scale = rmin != rmax ? __fdiv_rn(__fsub_rn(rmax, rmin), 255.f) : 1.f;
        zp = (int32_t)rintf(__fdiv_rn(__fsub_rn(0.f, rmin), scale));
    }
    const float zpf = (float)zp;
    for (int64_t i = threadIdx.x; i < inner; i += kThreads) {
        const float v = gamma ? __fmul_rn(row[i], s) : row[i];
        // SlowRound (runtime/chainerx_util.cc:397-410): fp32 quotient rounded to nearest even (the double rint of a float is rintf)
        const float r = rintf(__fdiv_rn(v, scale));
        // the conversions keep the low eight bits of the truncated integer, which is what the host's casts produce
        if (kInt8)
            static_cast<int8_t*>(q)[(int64_t)m * inner + i] = (int8_t)(__float2int_rz(r) & 0xff);
        else
            static_cast<uint8_t*>(q)[(int64_t)m * inner + i] = (uint8_t)(__float2int_rz(__fadd_rn(r, zpf)) & 0xff);
    }
    if (threadIdx.x == 0 && (per_channel || m == 0)) {
        scales[per_channel ? m : 0] = scale;
        zero_points[per_channel ? m : 0] = zp;
    }
}

}  // namespace
}  // namespace chxq

using namespace chxq;

extern "C" size_t chxq_prepare_weights_workspace(int64_t M) {
    return M > 0 ? (size_t)M * 2 * sizeof(float) : 0;
}

extern "C" int chxq_prepare_weights(
        const float* w, int64_t M, int64_t inner, const float* bn_scale, const float* bn_bias, const float* bn_mean, const float* bn_var, float epsilon,
        const float* conv_bias, int32_t to_int8, int32_t per_channel, void* q, float* scales, int32_t* zero_points, float* folded_w,
        float* folded_bias, void* workspace, size_t workspace_bytes, void* stream) {
    CHXQ_CHECK_ARG(w && q && scales && zero_points && M > 0 && inner > 0, "prepare_weights: bad arguments");
    CHXQ_CHECK_ARG(M < (1ll << 31), "prepare_weights: too many output channels for the grid");
    const bool bn = bn_scale != nullptr;
    CHXQ_CHECK_ARG(!bn || (bn_bias && bn_mean && bn_var), "prepare_weights: batch normalization needs scale, bias, mean and variance");
    CHXQ_CHECK_ARG(bn || (!bn_bias && !bn_mean && !bn_var && !conv_bias), "prepare_weights: bias / mean / variance given without a batch-norm scale");
    CHXQ_CHECK_ARG(!bn || folded_bias, "prepare_weights: folding a batch normalization produces a bias: give folded_bias");
    CHXQ_CHECK_ARG(workspace && workspace_bytes >= chxq_prepare_weights_workspace(M), "prepare_weights: workspace smaller than chxq_prepare_weights_workspace(M)");
    float* cmin = static_cast<float*>(workspace);
    float* cmax = cmin + M;
    cudaStream_t s = as_stream(stream);
    fold_minmax_kernel<<<(unsigned)M, kThreads, 0, s>>>(w, inner, bn_scale, bn_bias, bn_mean, bn_var, epsilon, conv_bias, folded_w, folded_bias, cmin, cmax);
    CHXQ_LAUNCH_CHECK();
    if (to_int8)
        quantize_weights_kernel<true><<<(unsigned)M, kThreads, 0, s>>>(w, (int)M, inner, bn_scale, bn_var, epsilon, cmin, cmax, per_channel, q, scales, zero_points);
    else
        quantize_weights_kernel<false><<<(unsigned)M, kThreads, 0, s>>>(w, (int)M, inner, bn_scale, bn_var, epsilon, cmin, cmax, per_channel, q, scales, zero_points);
    CHXQ_LAUNCH_CHECK();
    return CHXQ_OK;
}
