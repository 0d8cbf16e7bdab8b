/*
 * chxq.h - C ABI of libchxq.so: hand-written sm_100a CUDA kernels for the quantized-inference
 * VM ops of chainer-compiler (QuantizeLinear, DequantizeLinear, QLinearConv, QLinearMatMul,
 * ConvInteger, MatMulInteger) and its fused elementwise groups (ElementWiseNvrtc).
 *
 * Conventions
 *  - Every pointer named x/w/y/a/b/bias/..._zp/..._scale that is not marked "host" is a DEVICE
 *    pointer on the current CUDA device.  `stream` is a cudaStream_t passed as void*.
 *  - Functions return CHXQ_OK (0) or an error code; chxq_last_error() gives the thread-local
 *    message.  Nothing here aborts, allocates outputs, or synchronises unless it says so.
 *    The reference's op bodies CHECK()/abort on the same conditions (common/log.h:31-44); a
 *    C++ op body translates a non-zero status back into CHECK/exception.
 *  - Scalars the reference receives as VM `Scalar` arguments (runtime/chxvm_defs.py SCALAR /
 *    OPTIONAL_SCALAR kinds) are passed by value from the host.  Array-kind zero points and
 *    scales stay on the device and are never read back by the host.
 *  - Dtype codes are the reference's (compiler/dtype.h:14-26).
 *  - A device-side wait that expires (bounded mbarrier spin in the tensor-core kernels) sets a
 *    status word that chxq_device_status() returns; kernels never trap or hang.
 */
#ifndef CHXQ_H_
#define CHXQ_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CHXQ_OK 0
#define CHXQ_ERR_INVALID_ARGUMENT 1
#define CHXQ_ERR_UNSUPPORTED 2
#define CHXQ_ERR_CUDA 3
#define CHXQ_ERR_JIT 4
#define CHXQ_ERR_DEVICE_TIMEOUT 5
#define CHXQ_ERR_WORKSPACE 6

/* compiler/dtype.h:14-26 */
#define CHXQ_BOOL 1
#define CHXQ_INT8 2
#define CHXQ_INT16 3
#define CHXQ_INT32 4
#define CHXQ_INT64 5
#define CHXQ_UINT8 6
#define CHXQ_FLOAT16 7
#define CHXQ_FLOAT32 8
#define CHXQ_FLOAT64 9

/* Rounding of QuantizeLinear and of every requantizing epilogue. */
#define CHXQ_ROUND_REF_HALF_UP 0 /* (t + 0.5f) then truncation: runtime/ops/quantize.cc:33-34 */
#define CHXQ_ROUND_RNE 1         /* saturate(rint(x / s) + zp), round-half-to-even (ONNX) */

/* Activation layouts.  The reference is NCHW throughout; NHWC is this library's fast layout. */
#define CHXQ_NCHW 0
#define CHXQ_NHWC 1

/* Kernel family selection (argument `path`). */
#define CHXQ_PATH_AUTO 0   /* tensor-core kernel when the problem is eligible (depthwise layers: the CUDA-core depthwise kernels), else SIMT */
#define CHXQ_PATH_SIMT 1   /* general CUDA-core kernels (any shape, layout, zero point) */
#define CHXQ_PATH_TENSOR 2 /* tcgen05 kernels only; CHXQ_ERR_UNSUPPORTED when not eligible */

const char* chxq_last_error(void);
int chxq_version(void);

/* Number of kernels this library has launched in this process so far. */
int64_t chxq_launch_count(void);

/* Timing of the tensor-core kernel: while enabled, each launch is bracketed by CUDA events on its
 * own stream (do not enable during stream capture).  chxq_tc_profile_read SYNCHRONISES the device,
 * returns the summed duration, the launch count and the summed multiply-accumulates (as the ops
 * define them, without padding) of the launches recorded since the last read, and clears them. */
int chxq_tc_profile(int32_t enable);
int chxq_tc_profile_read(double* total_ms, int64_t* launches, double* total_macs);

/* Reads (and clears) the device-side status word of the current device.  SYNCHRONISES `stream`.
 * Returns CHXQ_OK or CHXQ_ERR_DEVICE_TIMEOUT. */
int chxq_device_status(void* stream);

/* ---- QuantizeLinear: runtime/chxvm_defs.py:451-453, body runtime/ops/quantize.cc:16-35,48-53.
 * y_dtype is the dtype of y_zero_point (CHXQ_UINT8 when the optional zero point is absent). */
int chxq_quantize_linear(const float* x, int64_t n, float y_scale, int32_t y_zero_point, int32_t y_dtype, int32_t round_mode, void* y,
                         void* stream);

/* ---- DequantizeLinear: runtime/chxvm_defs.py:454-456, body runtime/ops/quantize.cc:37-44,55-60. */
int chxq_dequantize_linear(const void* x, int32_t x_dtype, int64_t n, float x_scale, int32_t x_zero_point, float* y, void* stream);

/* ---- MatMulInteger: runtime/chxvm_defs.py:462-465, body runtime/ops/quantize.cc:96-114 with
 * NumpyMatMul (runtime/chainerx_util.cc:210-230).  a: [batch,M,K], b: [batch,K,N] (u8 or i8,
 * row-major), y: int32 [batch,M,N].  Zero points are device arrays of the operand's dtype with
 * length 0 (NULL), 1, or K for a / N for b (numpy broadcasting against the last axis). */
size_t chxq_matmul_integer_workspace(int64_t batch, int64_t M, int64_t N, int64_t K);
int chxq_matmul_integer(const void* a, int32_t a_dtype, const void* b, int32_t b_dtype, int64_t batch, int64_t M, int64_t N, int64_t K,
                        const void* a_zero_point, int64_t a_zp_len, const void* b_zero_point, int64_t b_zp_len, int32_t* y,
                        void* workspace, size_t workspace_bytes, int32_t path, void* stream);

/* ---- MatMulInteger for callers that must not allocate.  It has no counterpart in the reference.
 * Same result as chxq_matmul_integer on one matrix pair (no batch), but the scratch the tensor-core path needs
 * (repacked B, zero-point vectors, row sums) sits in a fixed array inside the library image, so this entry calls no
 * cudaMalloc / cudaFree and takes no workspace.  It is meant for callers such as an allocation hook of a memory pool,
 * which runs while the pool's lock is held and cannot ask the pool (or the driver) for more memory, or a serving loop
 * whose device memory was handed out completely at start-up and which must not take the device-wide synchronisation
 * a driver allocation implies.
 *  - Limit: the scratch needed, N * roundup(K, 64 or 128) + 8 * N + 4 * M bytes (each part rounded up to 256; the K tile is
 *    whichever of 64 and 128 pads K less), must fit
 *    CHXQ_NOALLOC_SCRATCH_BYTES; larger problems are refused with CHXQ_ERR_WORKSPACE.  Shapes the tensor-core kernel
 *    does not take (K not a multiple of 16, unaligned A) run on the CUDA-core kernel, which uses no scratch.
 *  - Every GPU that loads the library keeps the array until the process exits.
 *  - The first call on a device looks the array's device address up (cudaGetSymbolAddress); make that first call
 *    before any stream capture on that device (a first call inside a capture is refused with CHXQ_ERR_UNSUPPORTED).
 *  - All calls share the array and it keeps the previous call's bytes.  Nothing in it needs clearing: every byte the
 *    kernels read is written earlier in the same call.  Two calls whose kernels overlap on the GPU (different
 *    streams) race on it; calls on one stream are ordered and safe. */
#define CHXQ_NOALLOC_SCRATCH_BYTES (8 * 1024 * 1024)
int chxq_matmul_integer_noalloc(const void* a, int32_t a_dtype, const void* b, int32_t b_dtype, int64_t M, int64_t N, int64_t K,
                                const void* a_zero_point, int64_t a_zp_len, const void* b_zero_point, int64_t b_zp_len, int32_t* y,
                                void* stream);

/* ---- QLinearMatMul: has no VM op in the reference; ReplaceQLinearMatMul
 * (compiler/simplifier.cc:675-694) expands it to DequantizeLinear x2, MatMul, QuantizeLinear
 * with scalar parameters.  This entry computes that chain's result from the exact int32
 * accumulator: y = Q(float(acc) * (a_scale * b_scale); y_scale, y_zero_point). */
int chxq_qlinear_matmul(const void* a, int32_t a_dtype, float a_scale, int32_t a_zero_point, const void* b, int32_t b_dtype,
                        float b_scale, int32_t b_zero_point, float y_scale, int32_t y_zero_point, int32_t y_dtype, int64_t M, int64_t N,
                        int64_t K, int32_t round_mode, void* y, void* workspace, size_t workspace_bytes, int32_t path, void* stream);

/* ---- Convolution geometry: ComplementStride/ComplementPad (runtime/chainerx_util.cc:180-200),
 * CalculateAutoPad (:276-311), output size of chainerx::Conv (cover_all = false). */
typedef struct chxq_conv_geom {
    int32_t N, C, H, W;       /* input  */
    int32_t M, KH, KW;        /* weight [M, C/group, KH, KW] (OIHW, as the reference stores it) */
    int32_t stride_h, stride_w;
    int32_t pad_top, pad_left, pad_bottom, pad_right;
    int32_t group;
    int32_t Ho, Wo;           /* output */
    int32_t x_dtype, w_dtype; /* CHXQ_UINT8 / CHXQ_INT8 */
    int32_t x_layout, y_layout; /* CHXQ_NCHW / CHXQ_NHWC */
    int32_t x_cstride, y_cstride; /* NHWC only: bytes/elements between pixels (>= C resp. M); 0 = dense */
} chxq_conv_geom;

/* Host-only.  strides/pads: n_strides, n_pads in {0, 2} (empty -> 1 / 0; pads are begin == end as
 * compiler/chxvm/simple_node_emitter.cc:76-86 requires); auto_pad "" / "NOTSET" / "SAME_UPPER". */
int chxq_conv_resolve_geometry(int32_t N, int32_t C, int32_t H, int32_t W, int32_t M, int32_t Cg, int32_t KH, int32_t KW,
                               const int64_t* strides, int32_t n_strides, const int64_t* pads, int32_t n_pads, int32_t group,
                               const char* auto_pad, chxq_conv_geom* out);

/* ---- ConvInteger: runtime/chxvm_defs.py:466-469, body runtime/ops/quantize.cc:116-146.
 * x_zero_point is a host scalar (OPTIONAL_SCALAR; has_x_zp = 0 when absent); w_zero_point is a
 * device array of w's dtype, length 0 (NULL), 1 or M.  Zero padding is applied after the zero
 * point is subtracted, as the reference does.  y: int32, layout g->y_layout. */
/* Worst-case workspace of the tensor-core path for this geometry (weights repacked per call by the
 * unpacked entries, explicit im2col matrix, per-position sums); 0 when only CUDA-core kernels apply.
 * The unpacked entries fall back to the CUDA-core kernels when given less (path AUTO). */
size_t chxq_conv_workspace(const chxq_conv_geom* g);
int chxq_conv_integer(const void* x, const void* w, const chxq_conv_geom* g, int32_t has_x_zp, int32_t x_zero_point,
                      const void* w_zero_point, int64_t w_zp_len, int32_t* y, void* workspace, size_t workspace_bytes, int32_t path,
                      void* stream);

/* ---- QLinearConv: runtime/chxvm_defs.py:457-461, body runtime/ops/quantize.cc:62-94.
 * The result is computed from the exact int32 accumulator:
 *   acc = sum (x - x_zp)(w - w_zp[m]) + bias[m]
 *   y   = Q(float(acc) * (x_scale * w_scale[m]); y_scale, y_zp)
 * which is the reference's dequantize -> fp32 conv -> quantize chain with exact sums (at most
 * one quantization step apart where fp32 accumulation error crosses a rounding boundary).
 * bias follows ONNX (int32, scale x_scale*w_scale[m]); the reference's own bias handling passes
 * the raw int32 values to the fp32 conv and is untested there.
 * Fusions that have no counterpart in the reference (all disabled when zero / NULL):
 *   clamp_hi_q >= 0 : output additionally clamped to <= clamp_hi_q (ReLU6 in the quantized domain;
 *                     ReLU itself is the saturation at y_zp == 0).
 *   residual        : u8 map with the output's shape/layout; the epilogue then evaluates, per
 *                     element, Q(relu(DQ(y; y_scale, y_zp) + DQ(r; res_scale, res_zp)); out_scale, out_zp),
 *                     i.e. the DequantizeLinear, DequantizeLinear, Add, Relu, QuantizeLinear nodes that
 *                     follow the convolution in a residual block. */
typedef struct chxq_qconv_params {
    float x_scale;
    int32_t x_zero_point;
    const float* w_scale;     /* device, length w_params_len */
    const void* w_zero_point; /* device, dtype of w, length w_params_len; NULL = the caller knows every zero point is zero
                                 (symmetric weights): the weight zero-point term and its per-position input sums are then skipped.
                                 A pointer is never read back by the host, so zero points that are present are treated as non-zero. */
    int64_t w_params_len;     /* 1 (per tensor) or M (per output channel) */
    float y_scale;
    int32_t y_zero_point;
    int32_t y_dtype;          /* CHXQ_UINT8 / CHXQ_INT8: dtype of y_zero_point */
    const int32_t* bias;      /* device, length M, or NULL */
    int32_t round_mode;
    int32_t clamp_hi_q;       /* -1 = off */
    const void* residual;     /* device u8, or NULL */
    float res_scale;
    int32_t res_zero_point;
    int32_t res_relu;
    float out_scale;
    int32_t out_zero_point;
    int32_t fold_scales;      /* 0: multiply by x_scale*w_scale[m], then divide by y_scale (the reference's operation order).
                                 1: one multiplier per channel, (x_scale*w_scale[m])/y_scale, and a residual tail on the
                                 pre-divided scales y_scale/out_scale, res_scale/out_scale: fewer instructions per output
                                 byte, at most one step from the other form where a rounding boundary is crossed.
                                 uint8 outputs with zero weight zero points only. */
} chxq_qconv_params;

int chxq_qlinear_conv(const void* x, const void* w, const chxq_conv_geom* g, const chxq_qconv_params* p, void* y, void* workspace,
                      size_t workspace_bytes, int32_t path, void* stream);

/* Weight pre-packing for the tensor-core path (the reference re-dequantizes the weights on every
 * call, runtime/ops/quantize.cc:74-88; constants are packed once here instead).  Packs OIHW
 * weights into K-major rows plus per-channel weight sums and widened zero points.  SYNCHRONISES
 * the stream once to learn whether every weight zero point is zero.  *flags receives
 *   bit 0: the geometry is eligible for the packed tensor-core entries below (else use the
 *          unpacked entry, which falls back to the CUDA-core kernels), and
 *   bit 1: every weight zero point is zero (the per-position input sums are then skipped).
 * Pass the same flags back to the packed entries.  Their workspace (256-byte aligned, size from
 * chxq_conv_workspace) holds the im2col matrix and per-position sums when the geometry or the
 * zero points need them. */
size_t chxq_conv_prepack_bytes(const chxq_conv_geom* g);
/* Exact workspace of the packed entries for this geometry, activation zero point and pack flags. */
size_t chxq_conv_packed_workspace(const chxq_conv_geom* g, int32_t x_zero_point, int32_t packed_flags);
int chxq_conv_prepack(const void* w, const chxq_conv_geom* g, const void* w_zero_point, int64_t w_zp_len, void* packed,
                      size_t packed_bytes, int32_t* flags, void* stream);
int chxq_qlinear_conv_packed(const void* x, const void* packed, const chxq_conv_geom* g, const chxq_qconv_params* p, int32_t packed_flags,
                             void* y, void* workspace, size_t workspace_bytes, void* stream);

/* Two QLinearConv ops as ONE kernel: (g1, p1) is a convolution with 64, 128 or 256 output channels, (g2, p2) the 1x1 / stride-1
 * convolution that is its only reader (p2->x_scale / x_zero_point = p1->y_scale / y_zero_point); p2 may carry the residual tail.
 * The map between them is requantized tile by tile into shared memory and is never written: the first layer's tensor-core work
 * runs under the second layer's epilogue.  The reference runs the two ops one after the other (runtime/ops/quantize.cc:62-94);
 * results are bit-identical to that sequence.  Needs NHWC maps, packed weights with zero weight zero points, zero activation zero
 * points in front of both layers and folded requantizations; CHXQ_ERR_UNSUPPORTED otherwise -- run the two ops then.  No
 * workspace. */
int chxq_qlinear_conv_chain_packed(const void* x, const void* packed1, const chxq_conv_geom* g1, const chxq_qconv_params* p1, int32_t packed_flags1,
                                   const void* packed2, const chxq_conv_geom* g2, const chxq_qconv_params* p2, int32_t packed_flags2, void* y,
                                   void* stream);

/* QuantizeLinear(x; p->x_scale, p->x_zero_point -> uint8, quant_round_mode) fused into the packed QLinearConv that consumes
 * it: x is the fp32 tensor (layout g->x_layout), the uint8 map never exists in memory.  Only for geometries on the
 * space-to-depth path (stride 2, at most 4 channels: network stems), CHXQ_ERR_UNSUPPORTED otherwise.  Bit-identical to
 * chxq_quantize_linear followed by chxq_qlinear_conv_packed.  The reference runs the two ops separately
 * (runtime/ops/quantize.cc:48-53, 62-94). */
int chxq_quantize_qlinear_conv_packed(const float* x, int32_t quant_round_mode, const void* packed, const chxq_conv_geom* g,
                                      const chxq_qconv_params* p, int32_t packed_flags, void* y, void* workspace, size_t workspace_bytes, void* stream);
/* QLinearConv followed by MaxPool(kernel 3, stride 2, pad 0; cover_all as Chainer's max_pooling_2d, i.e. ONNX ceil_mode) as ONE
 * kernel: the pooling runs on the convolution's output tiles while they are in shared memory and only the pooled map
 * y [N, Hp, Wp, M] (NHWC uint8, Hp = (Ho - 3 + cover_all) / 2 + 1) is written.  The reference runs QLinearConv
 * (runtime/ops/quantize.cc:62-94) and MaxPool (runtime/ops/pooling.cc:47-60) as two ops with the full-resolution map in
 * between; results are bit-identical to that sequence.  x_is_f32 != 0: x is the fp32 tensor in front of a QuantizeLinear
 * (as chxq_quantize_qlinear_conv_packed).  Needs packed weights of a geometry whose K tile is 64 bytes (network stems);
 * CHXQ_ERR_UNSUPPORTED otherwise -- run the two ops then.  Workspace: chxq_conv_packed_workspace. */
int chxq_qlinear_conv_maxpool_packed(const void* x, int32_t x_is_f32, int32_t quant_round_mode, const void* packed, const chxq_conv_geom* g,
                                     const chxq_qconv_params* p, int32_t packed_flags, int32_t pool_kernel, int32_t pool_stride, int32_t pool_pad,
                                     int32_t cover_all, void* y, void* workspace, size_t workspace_bytes, void* stream);
int chxq_conv_integer_packed(const void* x, const void* packed, const chxq_conv_geom* g, int32_t has_x_zp, int32_t x_zero_point,
                             int32_t packed_flags, int32_t* y, void* workspace, size_t workspace_bytes, void* stream);

/* ---- Fused elementwise groups.
 * chxq_eltwise_codegen replaces BuildNvrtcProgram (compiler/nvrtc_builder.cc:91-206): same
 * inputs (the group's nodes in any order, its input and output values), output = CUDA C source
 * of one single-pass, 128-bit vectorised, grid-stride kernel `fusion<id>` (+ `fusion<id>_s`, the
 * scalar variant for unaligned buffers).  Node ops: compiler/nvrtc_builder.cc:35-87. */
#define CHXQ_EW_IDENTITY 0
#define CHXQ_EW_TANH 1
#define CHXQ_EW_EXP 2
#define CHXQ_EW_SIGMOID 3
#define CHXQ_EW_ADD 4
#define CHXQ_EW_SUB 5
#define CHXQ_EW_MUL 6
#define CHXQ_EW_DIV 7
#define CHXQ_EW_CONSTANT 8

typedef struct chxq_ew_node {
    int32_t op;        /* CHXQ_EW_* */
    int32_t inputs[2]; /* value ids; unused = -1 */
    int32_t output;    /* value id */
    double constant;   /* CHXQ_EW_CONSTANT only */
} chxq_ew_node;

/* Host-only.  value_names[v] is the graph name of value id v (used, cleansed, as identifier, as the
 * reference does).  Writes a NUL-terminated string of at most buf_len bytes; *needed receives the
 * size required (including the NUL).  dtype: CHXQ_FLOAT16/32/64. */
int chxq_eltwise_codegen(const chxq_ew_node* nodes, int32_t n_nodes, const int32_t* input_ids, int32_t n_inputs,
                         const int32_t* output_ids, int32_t n_outputs, const char* const* value_names, int32_t n_values, int32_t dtype,
                         int32_t fusion_id, char* buf, size_t buf_len, size_t* needed);

/* ElementWiseNvrtc: runtime/chxvm_defs.py:431-434, body runtime/ops/nvrtc.cc:90-161.  `code` is the
 * text produced by chxq_eltwise_codegen; it is compiled for sm_100a on first use and cached by its
 * full text, as the reference caches (runtime/ops/nvrtc.cc:41-84).  All buffers hold n elements of
 * `dtype` (the op body broadcasts and contiguizes first, as the reference's does at :103-112). */
int chxq_eltwise_run(const char* code, int32_t fusion_id, const void* const* inputs /*host array*/, int32_t n_inputs,
                     void* const* outputs /*host array*/, int32_t n_outputs, int64_t n, int32_t dtype, void* stream);

/* Fusion grouping: FuseElementwiseOperations (compiler/fusion_elementwise.cc:10-40) +
 * FuseAllConnectedNodes (compiler/fusion.cc:165-214).  Host-only.  The graph is given as flat
 * arrays; group_of_node[i] receives 0 (not fused) or the 1-based group id. */
typedef struct chxq_graph_node {
    const char* op_type;      /* ONNX op name, e.g. "Add", "Tanh", "Constant" */
    const int32_t* inputs;    /* value ids */
    int32_t n_inputs;
    const int32_t* outputs;   /* value ids */
    int32_t n_outputs;
    int32_t is_grad;          /* Node::IsGradNode() */
    int32_t const_is_float;   /* Constant only */
    int64_t const_num_elements; /* Constant only */
} chxq_graph_node;

typedef struct chxq_graph_value {
    int32_t dtype;            /* CHXQ_* or 0 = unknown */
    int32_t is_graph_output;
} chxq_graph_value;

int chxq_fuse_elementwise(const chxq_graph_node* nodes, int32_t n_nodes, const chxq_graph_value* values, int32_t n_values,
                          int32_t* group_of_node, int32_t* n_groups);

/* Weight quantizer of the --quantize pass: QuantizeData (compiler/quantize.cc:70-89) and its
 * per-output-channel form QuantizeWeightConvolution (:98-129).  HOST pointers (the pass runs at
 * compile time).  w: [M, inner] fp32; to_int8 != 0: symmetric int8 (scale = 2*max|w|/254, zp 0);
 * else asymmetric uint8.  per_channel == 0 quantizes the whole tensor with one scale (scales[0]). */
int chxq_quantize_weights_host(const float* w, int64_t M, int64_t inner, int32_t to_int8, int32_t per_channel, void* q, float* scales,
                               int32_t* zero_points);

/* The same quantizer on the DEVICE, with the Conv + BatchNormalization merge (compiler/merge.cc:142-215) in front of it, for
 * preparing a model without a host pass over the weights.  Device pointers; never synchronizes.
 *   w [M, inner] fp32.  bn_scale / bn_bias / bn_mean / bn_var [M] fp32: all four or none (none = quantize w as it is);
 *   conv_bias [M] fp32 or NULL (only with batch normalization).  With batch normalization
 *       s = bn_scale / sqrt(bn_var + epsilon);  w'[m] = w[m] * s[m];  folded_bias = (conv_bias - bn_mean) * s + bn_bias
 *   and w' is what gets quantized.  q [M, inner] int8 / uint8; scales, zero_points: [M] (per_channel != 0) or [1].
 *   folded_w [M, inner] fp32 or NULL: receives w'.  folded_bias [M] fp32: required with batch normalization.
 *   workspace: chxq_prepare_weights_workspace(M) bytes.
 * Results are bit-identical to chxq_quantize_weights_host applied to a single-rounded fp32 evaluation of the merge. */
size_t chxq_prepare_weights_workspace(int64_t M);
int chxq_prepare_weights(const float* w, int64_t M, int64_t inner, const float* bn_scale, const float* bn_bias, const float* bn_mean,
                         const float* bn_var, float epsilon, const float* conv_bias, int32_t to_int8, int32_t per_channel, void* q, float* scales,
                         int32_t* zero_points, float* folded_w, float* folded_bias, void* workspace, size_t workspace_bytes, void* stream);

/* ---- Glue ops a quantized CNN graph runs between the int8 ops (reference bodies are one-line
 * ChainerX calls; kernels here work on NHWC u8 maps). */
/* MaxPool (runtime/ops/pooling.cc:47-60) on u8 NHWC; cover_all as Chainer's max_pooling_2d. */
int chxq_maxpool_u8_nhwc(const uint8_t* x, int32_t N, int32_t H, int32_t W, int32_t C, int32_t k, int32_t stride, int32_t pad, int32_t Ho,
                         int32_t Wo, uint8_t* y, void* stream);
/* Global AveragePool (pooling.cc:62-75) fused with DequantizeLinear: y[n,c] = mean((q - zp)) * scale. */
int chxq_global_avgpool_dq_nhwc(const uint8_t* x, int32_t N, int32_t HW, int32_t C, float scale, int32_t zp, float* y, void* stream);
/* Linear / Gemm (runtime/ops/connection.cc:12-15): y[n,o] = sum_k x[n,k] w[o,k] + b[o], fp32. */
int chxq_linear_f32(const float* x, const float* w, const float* b, int32_t N, int32_t K, int32_t O, float* y, void* stream);
/* DequantizeLinear, DequantizeLinear, Add, (Relu), QuantizeLinear of two u8 maps in one pass. */
int chxq_qadd_u8(const uint8_t* a, float a_scale, int32_t a_zp, const uint8_t* b, float b_scale, int32_t b_zp, int64_t n, float y_scale,
                 int32_t y_zp, int32_t relu, int32_t round_mode, uint8_t* y, void* stream);
/* NCHW <-> NHWC transposes of 1-byte and 4-byte maps (boundary conversions). */
int chxq_nchw_to_nhwc(const void* x, int32_t elem_bytes, int32_t N, int32_t C, int32_t H, int32_t W, int32_t c_stride, void* y, void* stream);
int chxq_nhwc_to_nchw(const void* x, int32_t elem_bytes, int32_t N, int32_t C, int32_t H, int32_t W, int32_t c_stride, void* y, void* stream);
/* ReduceMin + ReduceMax of an fp32 tensor in one pass (the dynamic-quantization parameter
 * sub-graph of compiler/quantize.cc:172-202); out[0] = min, out[1] = max, both on the device. */
int chxq_minmax_f32(const float* x, int64_t n, float* out2, void* stream);

/* ---- Dynamic quantization without a host round trip.  The reference's --quantize pass feeds every quantized operator from
 * a sub-graph ReduceMin / ReduceMax -> Sub, Div, Floor, Cast -> QuantizeLinear (compiler/quantize.cc:172-207) whose scale and
 * zero point are 0-d device arrays; its VM reads each of them back to the host per op call (runtime/chxvm_var.cc:70-76), which
 * synchronizes the stream and keeps the program out of a CUDA graph.  The three entries below take those scalars where they
 * are: on the device.
 *   chxq_dynamic_quant_params_u8: scale = (rmax - rmin) / 255 (1 when rmax == rmin), zero point = uint8(floor((0 - rmin) /
 *     scale)) in the fp32 operations of the emitted nodes; the range is NOT widened to include zero (as in the reference); the
 *     Cast saturates.  rmin / rmax: the two floats chxq_minmax_f32 writes.
 *   chxq_quantize_linear_dev: chxq_quantize_linear with y_scale and y_zero_point (dtype y_dtype, may be NULL = 0) read from
 *     device memory; same element arithmetic (runtime/ops/quantize.cc:16-35).
 *   chxq_conv_integer_dev: chxq_conv_integer (runtime/ops/quantize.cc:116-146) with the activation zero point read from a device
 *     scalar of x's dtype; runs on the general CUDA-core kernel (the tensor-core path folds a host-known zero point into its
 *     padding value and correction terms).
 * MatMulInteger already takes its zero points as device arrays. */
int chxq_dynamic_quant_params_u8(const float* rmin, const float* rmax, float* scale, uint8_t* zero_point, void* stream);
int chxq_quantize_linear_dev(const float* x, int64_t n, const float* y_scale, const void* y_zero_point, int32_t y_dtype, int32_t round_mode,
                             void* y, void* stream);
int chxq_conv_integer_dev(const void* x, const void* w, const chxq_conv_geom* g, const void* x_zero_point, const void* w_zero_point,
                          int64_t w_zp_len, int32_t* y, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* CHXQ_H_ */
