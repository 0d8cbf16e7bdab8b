// Internal launch interfaces between the translation units of libchxq.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/chxq.h"
#include "epilogue.cuh"

namespace chxq {

// ---- CUDA-core kernels (simt.cu) ----
// A zero point as the ops receive it: absent (len 0), one value (len 1; read from `ptr`, or `scalar`
// when ptr is null) or a device vector of the operand's dtype aligned with the operand's last axis.
struct ZpSpec {
    const void* ptr;
    int64_t len;
    int scalar;
};

int launch_gemm_simt(
        const void* a, bool a_signed, const void* b, bool b_signed, int64_t batch, int64_t M, int64_t N, int64_t K, const ZpSpec& za,
        const ZpSpec& zb, const EpiArgs& epi, void* y, cudaStream_t s);
int launch_conv_simt(
        const void* x, const void* w, const chxq_conv_geom& g, int has_x_zp, int x_zp, const void* w_zp, int64_t w_zp_len, const EpiArgs& epi,
        void* y, cudaStream_t s, const void* x_zp_dev = nullptr);  // x_zp_dev: the activation zero point as a device scalar of x's dtype
// A[row, k], row = (n, ho, wo), k = tap * c_pitch + c, row length k_pad (multiple of 16); padding
// positions hold pad_byte, columns with c >= C or tap >= KH*KW hold 0.
int launch_im2col(const void* x, const chxq_conv_geom& g, int c_pitch, int k_pad, int pad_byte, void* a, cudaStream_t s);

// ---- depthwise kernel (depthwise.cu): group == C == M, NHWC, requantizing epilogue ----
bool depthwise_eligible(const chxq_conv_geom& g, const void* x, const void* y, const void* residual);
// 3x3 depthwise on uint8 maps with zero point 0 and symmetric weights (dw3x3_rows_kernel); w: OIHW weights (row stride 9, tap stride 1,
// w_diag 0) or the diagonal-block pack of the tensor-core path (row stride k_total, tap stride 64, w_diag 1)
bool depthwise3x3_eligible(const chxq_conv_geom& g, const void* x, const void* y, int x_zp, const EpiArgs& epi);
int launch_depthwise3x3(const void* x, const void* w, int w_row_stride, int w_tap_stride, int w_diag, const chxq_conv_geom& g, const EpiArgs& epi,
                        void* y, cudaStream_t s);
// the same with the input rows staged in shared memory by TMA (dw3x3_staged_kernel): needs a 16-byte aligned map with a 16-byte pixel pitch
bool depthwise3x3_staged_eligible(const chxq_conv_geom& g, const void* x, const void* y, int x_zp, const EpiArgs& epi);
int launch_depthwise3x3_staged(const void* x, const void* w, int w_row_stride, int w_tap_stride, int w_diag, const chxq_conv_geom& g,
                               const EpiArgs& epi, void* y, cudaStream_t s);
int tc_variant_value();  // chxq_tc_variant's current setting
int launch_depthwise(
        const void* x, const void* w, const chxq_conv_geom& g, int x_zp, const void* w_zp, int64_t w_zp_len, const EpiArgs& epi, void* y,
        cudaStream_t s);

// ---- tcgen05 implicit-GEMM kernel (tc_igemm.cu) ----
// Problem: D[row, col] = sum_k A[row, k] * B[col, k] over u8/s8 operands, both K-major.
// A is read through a 4-D tensor map {C, W, H, N} (an NHWC activation, or a plain matrix with
// W = rows and H = N = 1); a tile is a box of Wb x Hb x Nb = 128 output positions and the K loop
// walks taps (kh, kw) x channel chunks, shifting the box by the tap offset (stride-1 convolution
// with zero fill outside the map).  B is a packed weight matrix [cols, taps * c_pad].
struct TcProblem {
    // A operand
    const void* a;
    int a_signed;
    int C;            // channels (K extent per tap) present in memory
    int64_t a_cs;     // bytes between consecutive W positions
    int64_t a_row_bytes;  // bytes between consecutive H rows; 0 = W * a_cs (a larger value lets rows of C bytes overlap: a_cs < C)
    int W, H, N;      // extents of the A map
    // B operand
    const void* b;    // [cols][taps * c_pad]
    int b_signed;
    int cols;
    int c_pad;        // per-tap K extent in B (multiple of bk)
    int bk;           // 32 / 64 / 128
    // convolution taps (1,1,0,0 for a plain GEMM)
    int KH, KW, pad_top, pad_left;
    int sw, sh;       // convolution strides, applied by the TMA box as element strides (0 reads as 1)
    // grouped convolution: output columns [g * group_cols, (g + 1) * group_cols) read input channels starting at g * group_cin
    // (0 = one group).  The column tile must not straddle groups: bn divides group_cols.
    int group_cols, group_cin;
    // output extents (positions) and tile box
    int Wo, Ho, No;
    int Wb, Hb, Nb;
    int bn;           // 64 / 128 / 256 ; 0 = choose
    // output
    void* y;
    int64_t ldc;      // elements between consecutive output positions
    // zero-point terms: acc = raw - col_scale * col_corr[col] - col_mul[col] * row_corr[pos]
    const int32_t* col_corr;
    int col_scale;
    const int32_t* col_mul;
    const int32_t* row_corr;
    EpiArgs epi;
    double alg_macs;  // multiply-accumulates of the problem as the op defines it (no padding), for profiling
    // Fused 3x3 / stride-2 / pad-0 max pooling of the uint8 output: y is then the pooled map [No, pool_ho, pool_wo] x ldc and the
    // convolution's own output is never written.  Needs a 64-byte K tile, the box 16 x 8 x 1 and no residual.  0 = no pooling.
    int pool_ho, pool_wo;
};

int launch_tc_igemm(const TcProblem& p, cudaStream_t s);
// q1 followed by the 1x1 convolution q2 as one kernel (the map between them is never written); CHXQ_ERR_UNSUPPORTED when the pair has none.
int launch_tc_chain_igemm(const TcProblem& q1, const TcProblem& q2, cudaStream_t s);

// Tensor-core planning shared by pre-packing and execution.
enum TcConvPath : int { kTcNone = 0, kTcDirect = 1, kTcIm2col = 2, kTcS2d = 3 };
struct TcConvPlan {
    int path;
    int bk;
    int c_pitch;   // K index = tap * c_pitch + c
    int k_total;   // packed weight row length (multiple of bk)
    int a_pitch;   // row length of the explicit im2col matrix (multiple of 16; the K tail up to k_total is TMA zero fill)
    int Wb, Hb, Nb;
    // kTcS2d (stride 2, at most 4 channels): the map is repacked as 2x2 pixel blocks of 16 bytes; a K tile is one row of
    // kw2 blocks, there are kh2 such rows per output; t0h / t0w are the (negative) block offsets of the first tap;
    // rows2 x cols2 blocks per image including the halo.
    int kh2, kw2, t0h, t0w, rows2, cols2;
    // grouped convolutions on the direct path (see TcProblem::group_cols); diag: depthwise weights expanded to dense
    // 64 x 64 diagonal blocks
    int group_cols, group_cin, diag;
};
TcConvPlan plan_tc_conv(const chxq_conv_geom& g);
int choose_bk(int k);

}  // namespace chxq
