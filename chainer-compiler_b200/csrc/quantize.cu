// QuantizeLinear / DequantizeLinear and the other single-pass, HBM-bound elementwise kernels.
//
// Every kernel here moves each byte once: 128-bit loads and stores, 16 elements per thread per
// step, enough independent loads in flight per thread to cover HBM latency.  The reference runs
// QuantizeLinear as five or six separate full-tensor ChainerX passes (runtime/ops/quantize.cc:29-34)
// and DequantizeLinear as two or three (:37-44).
#include <stdarg.h>

#include <atomic>

#include "common.h"
#include "qmath.cuh"

namespace chxq {

static thread_local char g_err[1024] = "";

int set_error(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

__device__ int g_device_status = 0;

static std::atomic<long long> g_launches{0};
void count_launch(int n) {
    g_launches.fetch_add(n, std::memory_order_relaxed);
}

int* device_status_ptr() {
    // Resolved once per device (symbol lookup is not something to repeat inside a stream capture).
    // Host threads driving different GPUs may get here at the same time: the slots are atomics (every writer stores the same value).
    static std::atomic<int*> cache[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    int* p = cache[dev].load(std::memory_order_acquire);
    if (p == nullptr) {
        if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_device_status) != cudaSuccess) return nullptr;
        cache[dev].store(p, std::memory_order_release);
    }
    return p;
}

namespace {

constexpr int kThreads = 256;

// 16 elements per thread per step as four 128-bit loads and four 32-bit stores; lane i of a warp touches the i-th
// 16 bytes (load) / 4 bytes (store) of a contiguous span, so every memory instruction is fully coalesced.
// kMode: 0 = uint8 round-half-up through the constant-divisor division and add-based rounding (no conversion or
// reciprocal instruction per element); 2 = the same for round-half-to-even; 1 = general (int8 outputs, unusual scales).
template <bool kSigned, int kMode>
__global__ void __launch_bounds__(kThreads) quantize_vec16_kernel(
        const float4* __restrict__ x, int64_t n4, float scale, QDiv dv, float zp_f, int has_zp, int round_mode, uint32_t* __restrict__ y) {
    const int64_t step = (int64_t)gridDim.x * blockDim.x * 4;
    const QDiv8 dv8 = make_qdiv8(dv, zp_f);
    for (int64_t base = (int64_t)blockIdx.x * blockDim.x * 4 + threadIdx.x; base < n4; base += step) {
        float4 v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t g = base + (int64_t)j * blockDim.x;
            v[j] = g < n4 ? __ldcs(x + g) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t g = base + (int64_t)j * blockDim.x;
            uint32_t q0, q1, q2, q3;
            if (kMode == 0) {
                bool general = false;  // one magnitude test for the four quotients; the rare group that fails is redone
                const uint32_t packed = quantize4_u8_up(v[j], dv8, &general);
                if (!general) {
                    if (g < n4) __stcs(y + g, packed);
                    continue;
                }
                q0 = (uint32_t)quantize_one<false>(v[j].x, scale, zp_f, has_zp != 0, round_mode);
                q1 = (uint32_t)quantize_one<false>(v[j].y, scale, zp_f, has_zp != 0, round_mode);
                q2 = (uint32_t)quantize_one<false>(v[j].z, scale, zp_f, has_zp != 0, round_mode);
                q3 = (uint32_t)quantize_one<false>(v[j].w, scale, zp_f, has_zp != 0, round_mode);
            } else if (kMode == 2) {
                bool general = false;
                const float t0 = qdiv_unguarded(v[j].x, dv, &general), t1 = qdiv_unguarded(v[j].y, dv, &general);
                const float t2 = qdiv_unguarded(v[j].z, dv, &general), t3 = qdiv_unguarded(v[j].w, dv, &general);
                q0 = quantize_u8_rne_bits(t0, zp_f); q1 = quantize_u8_rne_bits(t1, zp_f);
                q2 = quantize_u8_rne_bits(t2, zp_f); q3 = quantize_u8_rne_bits(t3, zp_f);
                if (general) {
                    q0 = (uint32_t)quantize_one<false>(v[j].x, scale, zp_f, has_zp != 0, round_mode);
                    q1 = (uint32_t)quantize_one<false>(v[j].y, scale, zp_f, has_zp != 0, round_mode);
                    q2 = (uint32_t)quantize_one<false>(v[j].z, scale, zp_f, has_zp != 0, round_mode);
                    q3 = (uint32_t)quantize_one<false>(v[j].w, scale, zp_f, has_zp != 0, round_mode);
                }
            } else {
                q0 = (uint32_t)quantize_one<kSigned>(v[j].x, scale, zp_f, has_zp != 0, round_mode) & 0xffu;
                q1 = (uint32_t)quantize_one<kSigned>(v[j].y, scale, zp_f, has_zp != 0, round_mode) & 0xffu;
                q2 = (uint32_t)quantize_one<kSigned>(v[j].z, scale, zp_f, has_zp != 0, round_mode) & 0xffu;
                q3 = (uint32_t)quantize_one<kSigned>(v[j].w, scale, zp_f, has_zp != 0, round_mode) & 0xffu;
            }
            if (g < n4) __stcs(y + g, q0 | (q1 << 8) | (q2 << 16) | (q3 << 24));
        }
    }
}

template <bool kSigned>
__global__ void __launch_bounds__(kThreads) quantize_scalar_kernel(
        const float* __restrict__ x, int64_t begin, int64_t n, float scale, float zp_f, int has_zp, int round_mode, uint8_t* __restrict__ y) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = begin + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        y[i] = (uint8_t)quantize_one<kSigned>(x[i], scale, zp_f, has_zp != 0, round_mode);
    }
}

// 16 elements per thread per step as four 32-bit loads and four 128-bit stores, coalesced like the quantize kernel.
template <bool kSigned>
__global__ void __launch_bounds__(kThreads) dequantize_vec16_kernel(
        const uint32_t* __restrict__ x, int64_t n4, float scale, float zp_f, int has_zp, float4* __restrict__ y) {
    const int64_t step = (int64_t)gridDim.x * blockDim.x * 4;
    for (int64_t base = (int64_t)blockIdx.x * blockDim.x * 4 + threadIdx.x; base < n4; base += step) {
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t g = base + (int64_t)j * blockDim.x;
            w[j] = g < n4 ? __ldcs(x + g) : 0u;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t g = base + (int64_t)j * blockDim.x;
            float4 o;
            if (kSigned) {
                o.x = dequantize_one((int)(int8_t)(w[j] & 0xffu), scale, zp_f, has_zp != 0);
                o.y = dequantize_one((int)(int8_t)((w[j] >> 8) & 0xffu), scale, zp_f, has_zp != 0);
                o.z = dequantize_one((int)(int8_t)((w[j] >> 16) & 0xffu), scale, zp_f, has_zp != 0);
                o.w = dequantize_one((int)(int8_t)(w[j] >> 24), scale, zp_f, has_zp != 0);
            } else {
                // byte -> float without a conversion instruction: 2^23 + b as a bit pattern, minus (2^23 + zp), exactly b - zp
                const float c = __fadd_rn(8388608.f, zp_f);
                o.x = __fmul_rn(__fsub_rn(byte_to_magic(w[j], 0), c), scale);
                o.y = __fmul_rn(__fsub_rn(byte_to_magic(w[j], 1), c), scale);
                o.z = __fmul_rn(__fsub_rn(byte_to_magic(w[j], 2), c), scale);
                o.w = __fmul_rn(__fsub_rn(byte_to_magic(w[j], 3), c), scale);
            }
            if (g < n4) __stcs(y + g, o);
        }
    }
}

template <bool kSigned>
__global__ void __launch_bounds__(kThreads) dequantize_scalar_kernel(
        const uint8_t* __restrict__ x, int64_t begin, int64_t n, float scale, float zp_f, int has_zp, float* __restrict__ y) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = begin + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const int q = kSigned ? (int)(int8_t)x[i] : (int)x[i];
        y[i] = dequantize_one(q, scale, zp_f, has_zp != 0);
    }
}

__global__ void __launch_bounds__(kThreads) qadd_u8_kernel(
        const uint8_t* __restrict__ a, const uint8_t* __restrict__ b, int64_t n, RequantParams p, uint8_t* __restrict__ y, int vec_ok) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t n16 = vec_ok ? n / 16 : 0;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += stride) {
        const uint4 qa = __ldcs(reinterpret_cast<const uint4*>(a) + i);
        const uint4 qb = __ldcs(reinterpret_cast<const uint4*>(b) + i);
        const uint32_t wa[4] = {qa.x, qa.y, qa.z, qa.w}, wb[4] = {qb.x, qb.y, qb.z, qb.w};
        uint32_t wo[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint32_t o = 0;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int va = (wa[j] >> (8 * k)) & 0xff, vb = (wb[j] >> (8 * k)) & 0xff;
                o |= ((uint32_t)residual_one(va, vb, p) & 0xffu) << (8 * k);
            }
            wo[j] = o;
        }
        reinterpret_cast<uint4*>(y)[i] = make_uint4(wo[0], wo[1], wo[2], wo[3]);
    }
    for (int64_t i = n16 * 16 + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        y[i] = (uint8_t)residual_one(a[i], b[i], p);
    }
}

// One pass min/max: per-thread float4 loads, warp shuffles, one atomic pair per block on
// order-preserving integer keys.
__device__ __forceinline__ unsigned f2key(float f) {
    unsigned u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key2f(unsigned k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

__global__ void minmax_init_kernel(unsigned* keys) {
    keys[0] = 0xffffffffu;  // min key
    keys[1] = 0u;           // max key
}

__global__ void __launch_bounds__(kThreads) minmax_kernel(const float* __restrict__ x, int64_t n, unsigned* keys, int vec_ok) {
    float mn = INFINITY, mx = -INFINITY;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t n4 = vec_ok ? n / 4 : 0;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        const float4 v = __ldcs(reinterpret_cast<const float4*>(x) + i);
        mn = fminf(fminf(mn, v.x), fminf(v.y, fminf(v.z, v.w)));
        mx = fmaxf(fmaxf(mx, v.x), fmaxf(v.y, fmaxf(v.z, v.w)));
    }
    for (int64_t i = n4 * 4 + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        mn = fminf(mn, x[i]);
        mx = fmaxf(mx, x[i]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    if ((threadIdx.x & 31) == 0) {
        atomicMin(&keys[0], f2key(mn));
        atomicMax(&keys[1], f2key(mx));
    }
}

__global__ void minmax_finish_kernel(const unsigned* keys, float* out2) {
    out2[0] = key2f(keys[0]);
    out2[1] = key2f(keys[1]);
}

inline int grid_for(int64_t work_items, int per_sm = 8) {
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int64_t blocks = (work_items + kThreads - 1) / kThreads;
    int64_t cap = (int64_t)sms * per_sm;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

inline bool aligned16(const void* p) {
    return (reinterpret_cast<uintptr_t>(p) & 15u) == 0;
}

}  // namespace
}  // namespace chxq

using namespace chxq;

extern "C" const char* chxq_last_error(void) {
    return chxq::g_err;
}

extern "C" int chxq_version(void) {
    return 100;
}

extern "C" int64_t chxq_launch_count(void) {
    return (int64_t)chxq::g_launches.load(std::memory_order_relaxed);
}

extern "C" int chxq_device_status(void* stream) {
    CHXQ_CUDA(cudaStreamSynchronize(as_stream(stream)));
    int* dptr = device_status_ptr();
    if (!dptr) return set_error(CHXQ_ERR_CUDA, "device status word is unavailable");
    int h = 0;
    CHXQ_CUDA(cudaMemcpy(&h, dptr, sizeof(int), cudaMemcpyDeviceToHost));
    if (h != 0) {
        int zero = 0;
        CHXQ_CUDA(cudaMemcpy(dptr, &zero, sizeof(int), cudaMemcpyHostToDevice));
        return set_error(CHXQ_ERR_DEVICE_TIMEOUT, "a bounded device-side wait expired (code %d)", h);
    }
    return CHXQ_OK;
}

extern "C" int chxq_quantize_linear(
        const float* x, int64_t n, float y_scale, int32_t y_zero_point, int32_t y_dtype, int32_t round_mode, void* y, void* stream) {
    CHXQ_CHECK_ARG(n >= 0, "QuantizeLinear: negative element count");
    CHXQ_CHECK_ARG(is_q8(y_dtype), "QuantizeLinear: y_zero_point dtype must be uint8 or int8 (got %d)", y_dtype);
    const bool sgn = y_dtype == CHXQ_INT8;
    // runtime/ops/quantize.cc:26-27: the zero point must lie inside the output range.
    CHXQ_CHECK_ARG(y_zero_point >= (sgn ? -128 : 0) && y_zero_point <= (sgn ? 127 : 255), "QuantizeLinear: zero point %d out of range",
                   y_zero_point);
    CHXQ_CHECK_ARG(round_mode == CHXQ_ROUND_REF_HALF_UP || round_mode == CHXQ_ROUND_RNE, "QuantizeLinear: bad round_mode");
    if (n == 0) return CHXQ_OK;
    CHXQ_CHECK_ARG(x && y, "QuantizeLinear: null buffer");
    cudaStream_t s = as_stream(stream);
    const float zp_f = (float)y_zero_point;
    const int has_zp = y_zero_point != 0;
    int64_t done = 0;
    if (aligned16(x) && (reinterpret_cast<uintptr_t>(y) & 3u) == 0 && n >= 4) {
        const int64_t n4 = n / 4;
        const int grid = grid_for((n4 + 3) / 4, 32);
        const QDiv dv = make_qdiv(y_scale);
        const float4* x4 = reinterpret_cast<const float4*>(x);
        uint32_t* y32 = reinterpret_cast<uint32_t*>(y);
        if (sgn)
            quantize_vec16_kernel<true, 1><<<grid, kThreads, 0, s>>>(x4, n4, y_scale, dv, zp_f, has_zp, round_mode, y32);
        else if (round_mode == CHXQ_ROUND_REF_HALF_UP && dv.fast)
            quantize_vec16_kernel<false, 0><<<grid, kThreads, 0, s>>>(x4, n4, y_scale, dv, zp_f, has_zp, round_mode, y32);
        else if (dv.fast)
            quantize_vec16_kernel<false, 2><<<grid, kThreads, 0, s>>>(x4, n4, y_scale, dv, zp_f, has_zp, round_mode, y32);
        else
            quantize_vec16_kernel<false, 1><<<grid, kThreads, 0, s>>>(x4, n4, y_scale, dv, zp_f, has_zp, round_mode, y32);
        CHXQ_LAUNCH_CHECK();
        done = n4 * 4;
    }
    if (done < n) {
        const int grid = grid_for(n - done, 8);
        if (sgn)
            quantize_scalar_kernel<true><<<grid, kThreads, 0, s>>>(x, done, n, y_scale, zp_f, has_zp, round_mode, static_cast<uint8_t*>(y));
        else
            quantize_scalar_kernel<false><<<grid, kThreads, 0, s>>>(x, done, n, y_scale, zp_f, has_zp, round_mode, static_cast<uint8_t*>(y));
        CHXQ_LAUNCH_CHECK();
    }
    return CHXQ_OK;
}

extern "C" int chxq_dequantize_linear(
        const void* x, int32_t x_dtype, int64_t n, float x_scale, int32_t x_zero_point, float* y, void* stream) {
    CHXQ_CHECK_ARG(n >= 0, "DequantizeLinear: negative element count");
    CHXQ_CHECK_ARG(is_q8(x_dtype), "DequantizeLinear: x must be uint8 or int8 (got dtype %d)", x_dtype);
    if (n == 0) return CHXQ_OK;
    CHXQ_CHECK_ARG(x && y, "DequantizeLinear: null buffer");
    cudaStream_t s = as_stream(stream);
    const bool sgn = x_dtype == CHXQ_INT8;
    const float zp_f = (float)x_zero_point;
    const int has_zp = x_zero_point != 0;
    int64_t done = 0;
    if ((reinterpret_cast<uintptr_t>(x) & 3u) == 0 && aligned16(y) && n >= 4) {
        const int64_t n4 = n / 4;
        const int grid = grid_for((n4 + 3) / 4, 1 << 20);
        if (sgn)
            dequantize_vec16_kernel<true><<<grid, kThreads, 0, s>>>(reinterpret_cast<const uint32_t*>(x), n4, x_scale, zp_f, has_zp,
                                                                    reinterpret_cast<float4*>(y));
        else
            dequantize_vec16_kernel<false><<<grid, kThreads, 0, s>>>(reinterpret_cast<const uint32_t*>(x), n4, x_scale, zp_f, has_zp,
                                                                     reinterpret_cast<float4*>(y));
        CHXQ_LAUNCH_CHECK();
        done = n4 * 4;
    }
    if (done < n) {
        const int grid = grid_for(n - done, 8);
        if (sgn)
            dequantize_scalar_kernel<true><<<grid, kThreads, 0, s>>>(static_cast<const uint8_t*>(x), done, n, x_scale, zp_f, has_zp, y);
        else
            dequantize_scalar_kernel<false><<<grid, kThreads, 0, s>>>(static_cast<const uint8_t*>(x), done, n, x_scale, zp_f, has_zp, y);
        CHXQ_LAUNCH_CHECK();
    }
    return CHXQ_OK;
}

extern "C" int chxq_qadd_u8(
        const uint8_t* a, float a_scale, int32_t a_zp, const uint8_t* b, float b_scale, int32_t b_zp, int64_t n, float y_scale, int32_t y_zp,
        int32_t relu, int32_t round_mode, uint8_t* y, void* stream) {
    CHXQ_CHECK_ARG(n >= 0, "qadd: negative element count");
    if (n == 0) return CHXQ_OK;
    CHXQ_CHECK_ARG(a && b && y, "qadd: null buffer");
    RequantParams p{};
    p.y_scale = a_scale;
    p.y_zp_f = (float)a_zp;
    p.y_has_zp = a_zp != 0;
    p.res_scale = b_scale;
    p.res_zp_f = (float)b_zp;
    p.res_has_zp = b_zp != 0;
    p.res_relu = relu;
    p.out_scale = y_scale;
    p.out_zp_f = (float)y_zp;
    p.out_has_zp = y_zp != 0;
    p.round_mode = round_mode;
    finish_requant_params(&p);
    const int vec_ok = aligned16(a) && aligned16(b) && aligned16(y);
    qadd_u8_kernel<<<grid_for((n + 15) / 16, 8), kThreads, 0, as_stream(stream)>>>(a, b, n, p, y, vec_ok);
    CHXQ_LAUNCH_CHECK();
    return CHXQ_OK;
}

namespace chxq {
namespace {

// scale = (rmax - rmin) / 255 (1 when the range is empty); zero point = uint8(floor((0 - rmin) / scale)), in the fp32 operations
// of the Sub / Div / Floor / Cast nodes the quantizer emits (compiler/quantize.cc:196-207).  The range is not widened to
// include zero, as in the reference, so an all-positive input gives floor(-rmin / scale) < 0; the Cast of a negative float to
// uint8 is undefined in C++, here it saturates to 0 (and to 255 above), which is what the host-side helper of run_onnx does.
__global__ void dynamic_params_u8_kernel(const float* __restrict__ rmin, const float* __restrict__ rmax, float* __restrict__ scale, uint8_t* __restrict__ zp) {
    const float lo = *rmin, hi = *rmax;
    const float sc = hi != lo ? __fdiv_rn(__fsub_rn(hi, lo), 255.0f) : 1.0f;
    float z = floorf(__fdiv_rn(__fsub_rn(0.0f, lo), sc));
    z = fminf(fmaxf(z, 0.0f), 255.0f);
    *scale = sc;
    *zp = (uint8_t)(z != z ? 0.f : z);
}

// QuantizeLinear whose scale and zero point are device scalars: same element arithmetic as quantize_one (true division).
template <bool kSigned>
__global__ void __launch_bounds__(kThreads) quantize_dev_kernel(
        const float* __restrict__ x, int64_t n, const float* __restrict__ scale_p, const void* __restrict__ zp_p, int round_mode, uint8_t* __restrict__ y,
        int vec_ok) {
    const float scale = *scale_p;
    const int zp = zp_p == nullptr ? 0 : (kSigned ? (int)*static_cast<const int8_t*>(zp_p) : (int)*static_cast<const uint8_t*>(zp_p));
    const float zp_f = (float)zp;
    const bool has_zp = zp != 0;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t n4 = vec_ok ? n / 4 : 0;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        const float4 v = __ldcs(reinterpret_cast<const float4*>(x) + i);
        const uint32_t q0 = (uint32_t)quantize_one<kSigned>(v.x, scale, zp_f, has_zp, round_mode) & 0xffu;
        const uint32_t q1 = (uint32_t)quantize_one<kSigned>(v.y, scale, zp_f, has_zp, round_mode) & 0xffu;
        const uint32_t q2 = (uint32_t)quantize_one<kSigned>(v.z, scale, zp_f, has_zp, round_mode) & 0xffu;
        const uint32_t q3 = (uint32_t)quantize_one<kSigned>(v.w, scale, zp_f, has_zp, round_mode) & 0xffu;
        reinterpret_cast<uint32_t*>(y)[i] = q0 | (q1 << 8) | (q2 << 16) | (q3 << 24);
    }
    for (int64_t i = n4 * 4 + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        y[i] = (uint8_t)quantize_one<kSigned>(x[i], scale, zp_f, has_zp, round_mode);
}

}  // namespace
}  // namespace chxq

extern "C" int chxq_dynamic_quant_params_u8(const float* rmin, const float* rmax, float* scale, uint8_t* zero_point, void* stream) {
    CHXQ_CHECK_ARG(rmin && rmax && scale && zero_point, "dynamic quantization parameters: null pointer");
    dynamic_params_u8_kernel<<<1, 1, 0, as_stream(stream)>>>(rmin, rmax, scale, zero_point);
    CHXQ_LAUNCH_CHECK();
    return CHXQ_OK;
}

extern "C" int chxq_quantize_linear_dev(
        const float* x, int64_t n, const float* y_scale, const void* y_zero_point, int32_t y_dtype, int32_t round_mode, void* y, void* stream) {
    CHXQ_CHECK_ARG(n >= 0, "QuantizeLinear: negative element count");
    CHXQ_CHECK_ARG(is_q8(y_dtype), "QuantizeLinear: y_zero_point dtype must be uint8 or int8 (got %d)", y_dtype);
    CHXQ_CHECK_ARG(round_mode == CHXQ_ROUND_REF_HALF_UP || round_mode == CHXQ_ROUND_RNE, "QuantizeLinear: bad round_mode");
    if (n == 0) return CHXQ_OK;
    CHXQ_CHECK_ARG(x && y && y_scale, "QuantizeLinear: null buffer");
    const int vec_ok = aligned16(x) && (reinterpret_cast<uintptr_t>(y) & 3u) == 0;
    const int grid = grid_for((n + 3) / 4, 16);
    if (y_dtype == CHXQ_INT8)
        quantize_dev_kernel<true><<<grid, kThreads, 0, as_stream(stream)>>>(x, n, y_scale, y_zero_point, round_mode, static_cast<uint8_t*>(y), vec_ok);
    else
        quantize_dev_kernel<false><<<grid, kThreads, 0, as_stream(stream)>>>(x, n, y_scale, y_zero_point, round_mode, static_cast<uint8_t*>(y), vec_ok);
    CHXQ_LAUNCH_CHECK();
    return CHXQ_OK;
}

extern "C" int chxq_minmax_f32(const float* x, int64_t n, float* out2, void* stream) {
    CHXQ_CHECK_ARG(n > 0 && x && out2, "minmax: empty input or null buffer");
    cudaStream_t s = as_stream(stream);
    // out2 doubles as the key scratch (two 32-bit words), converted in place at the end.
    unsigned* keys = reinterpret_cast<unsigned*>(out2);
    minmax_init_kernel<<<1, 1, 0, s>>>(keys);
    minmax_kernel<<<grid_for((n + 3) / 4, 4), kThreads, 0, s>>>(x, n, keys, aligned16(x));
    minmax_finish_kernel<<<1, 1, 0, s>>>(keys, out2);
    count_launch(2);
    CHXQ_LAUNCH_CHECK();
    return CHXQ_OK;
}
