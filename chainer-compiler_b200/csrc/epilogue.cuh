// Epilogue description shared by the CUDA-core and tensor-core contraction kernels.
#pragma once

#include "qmath.cuh"

namespace chxq {

enum EpiMode : int {
    kEpiInt32 = 0,   // MatMulInteger / ConvInteger: store the exact accumulator
    kEpiRequant = 1  // QLinearMatMul / QLinearConv: requantize to u8 / i8 (optionally + residual tail)
};

struct EpiArgs {
    int mode;
    // mult[m] = x_scale * w_scale[m] (w_scale != nullptr) or mult_scalar
    float x_scale;
    const float* w_scale;
    int w_per_channel;  // 1: index by channel, 0: w_scale[0]
    float mult_scalar;
    const int32_t* bias;  // per output channel, may be null
    RequantParams rq;
    const uint8_t* residual;  // same indexing as the output, may be null
};

__device__ __forceinline__ float epi_mult(const EpiArgs& e, int ch) {
    if (e.w_scale == nullptr) return e.mult_scalar;
    return __fmul_rn(e.x_scale, e.w_scale[e.w_per_channel ? ch : 0]);
}

// Final value of one output element whose accumulator is `acc` (zero-point terms already applied).
// For kEpiRequant returns the quantized byte (as int); residual, when present, is the byte at the same
// output position.
__device__ __forceinline__ int epi_requant(const EpiArgs& e, int acc, float mult, int bias, int res_byte) {
    if (e.rq.fold) {  // uint8 only (checked on the host)
        int q = requant_u8_fold(acc, bias, __fdiv_rn(mult, e.rq.y_scale), e.rq);
        if (e.residual != nullptr) q = residual_fold(q, res_byte, e.rq);
        return q;
    }
    const int a = (int)((unsigned)acc + (unsigned)bias);
    int q = requant_one(a, mult, e.rq);
    if (e.residual != nullptr) q = residual_one(q, res_byte, e.rq);
    return q;
}

}  // namespace chxq
