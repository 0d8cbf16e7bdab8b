// Host side of the tcgen05 implicit-GEMM kernel (device code in tc_kernel.cuh, instantiated per K-tile size in
// tc_bk32.cu / tc_bk64.cu / tc_bk128.cu): planning of tile shapes, tensor maps, dispatch and optional per-launch timing.
#include <cuda.h>

#include <atomic>
#include <mutex>
#include <vector>

#include "common.h"
#include "kernels.h"
#include "tc_launch.h"

namespace chxq {
namespace {

// ------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(
        CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
        CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn) return fn;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess || qres != cudaDriverEntryPointSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    fn = reinterpret_cast<EncodeTiledFn>(p);
    return fn;
}

CUtensorMapSwizzle swizzle_for(int bk) {
    return bk == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : (bk == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
}

// SM count of the current device (grid size and kernel choice depend on it), looked up once per device ordinal.
int num_sms() {
    static std::atomic<int> cache[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) dev = -1;
    int sms = (dev >= 0 && dev < 64) ? cache[dev].load(std::memory_order_relaxed) : 0;
    if (sms == 0) {
        if (dev < 0 || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
        if (dev >= 0 && dev < 64) cache[dev].store(sms, std::memory_order_relaxed);
    }
    return sms;
}

// Optional per-launch timing with CUDA events on the launching stream (chxq_tc_profile / chxq_tc_profile_read).
struct ProfRec {
    cudaEvent_t e0, e1;
    double macs;
};
bool g_prof_on = false;
std::vector<ProfRec> g_prof;
std::mutex g_prof_mu;

#ifdef CHXQ_TL
long long* g_tl_buf = nullptr;
#endif
std::atomic<long long> g_wait_limit_ns{2000000000ll};  // chxq_tc_test_hooks
std::atomic<int> g_test_skip_kb{-1};
std::atomic<int> g_variant{0};  // chxq_tc_variant: 0 = choose, 1 = one tile per step, 2 = grouped tiles where eligible, 3 = grouped + halo tiles

int pick_bn(int cols, int64_t pos_tiles) {
    const int cand[3] = {256, 128, 64};
    const double base[3] = {1.0, 0.92, 0.78};
    double best = -1.0;
    int best_bn = 64;
    for (int i = 0; i < 3; ++i) {
        const int bn = cand[i];
        const int64_t ct = (cols + bn - 1) / bn;
        const int64_t tiles = pos_tiles * ct;
        const int64_t waves = (tiles + num_sms() - 1) / num_sms();
        const double wave_eff = (double)tiles / (double)(waves * num_sms());
        const double fill = (double)cols / (double)(ct * bn);  // columns that are real work
        const double score = wave_eff * fill * base[i];
        if (score > best) {
            best = score;
            best_bn = bn;
        }
    }
    return best_bn;
}

}  // namespace

int tc_variant_value() {
    return g_variant.load(std::memory_order_relaxed);
}

namespace tc {
long long wait_limit_ns_value() {
    return g_wait_limit_ns.load(std::memory_order_relaxed);
}

int encode_nhwc_box_map(CUtensorMap* out, const void* base, int C, int W, int H, int N, int64_t cs, int box_c, int box_w, int box_h) {
    EncodeTiledFn encode = get_encode_fn();
    if (!encode) return set_error(CHXQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    const cuuint64_t dims[4] = {(cuuint64_t)C, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)N};
    const cuuint64_t strides[3] = {(cuuint64_t)cs, (cuuint64_t)cs * W, (cuuint64_t)cs * W * H};
    const cuuint32_t box[4] = {(cuuint32_t)box_c, (cuuint32_t)box_w, (cuuint32_t)box_h, 1u};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    const CUresult r = encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return set_error(CHXQ_ERR_CUDA, "cuTensorMapEncodeTiled(NHWC box) failed with %d", (int)r);
    return CHXQ_OK;
}
}  // namespace tc

int choose_bk(int k) {
    // 64- or 128-byte K tiles, whichever pads K less (128 on a tie): the part of a tile beyond the operand is TMA zero fill, not
    // traffic, and only these two tile sizes have the grouped kernel.
    const int pad128 = (k + 127) / 128 * 128, pad64 = (k + 63) / 64 * 64;
    return pad128 <= pad64 ? 128 : 64;
}

static int largest_pow2_divisor(int v, int cap) {
    int d = 1;
    while (d * 2 <= cap && v % (d * 2) == 0) d *= 2;
    return d;
}

TcConvPlan plan_tc_conv(const chxq_conv_geom& g) {
    TcConvPlan pl{};
    pl.path = kTcNone;
    if (g.y_layout != CHXQ_NHWC) return pl;
    const int taps = g.KH * g.KW;
    const int64_t xcs = g.x_cstride > 0 ? g.x_cstride : g.C;
    if (g.group != 1) {
        // Grouped convolutions: a column tile of 64 output channels reads only its group's input channels.  Depthwise
        // (one channel per group) runs as groups of 64 channels whose 64 x 64 weight blocks are diagonal: 64 times the
        // multiply-accumulates of the definition, on a tensor pipe with that much to spare, against a memory-bound layer.
        const int cg = g.C / g.group, mg = g.M / g.group;
        const bool depthwise = cg == 1 && mg == 1;
        const bool ok = g.x_layout == CHXQ_NHWC && (xcs % 16 == 0) && g.stride_h <= 8 && g.stride_w <= 8 && g.pad_top >= 0 && g.pad_left >= 0 &&
                        g.pad_bottom >= 0 && g.pad_right >= 0 && g.pad_top < g.KH && g.pad_left < g.KW &&
                        (depthwise ? g.C % 16 == 0 : (mg % 64 == 0 && cg % 16 == 0));
        if (!ok) return pl;
        pl.path = kTcDirect;
        pl.diag = depthwise ? 1 : 0;
        pl.group_cols = depthwise ? 64 : mg;
        pl.group_cin = depthwise ? 64 : cg;
        pl.bk = depthwise ? 64 : choose_bk(cg);
        pl.c_pitch = depthwise ? 64 : (cg + pl.bk - 1) / pl.bk * pl.bk;
        pl.k_total = taps * pl.c_pitch;
        pl.a_pitch = pl.k_total;
        pl.Wb = largest_pow2_divisor(g.Wo, 16);
        pl.Hb = largest_pow2_divisor(g.Ho, 128 / pl.Wb);
        pl.Nb = 128 / (pl.Wb * pl.Hb);
        return pl;
    }
    // Stride-2 convolutions over at most 4 channels (network stems): space-to-depth.  A 2x2 pixel block becomes one
    // 16-byte pixel (4 C <= 16 channels), the KH x KW stride-2 window becomes a kh2 x kw2 stride-1 window over blocks, and
    // the kw2 blocks of one window row are contiguous in memory: 16 kw2 bytes, advancing by 16 bytes per output column.
    if (g.stride_h == 2 && g.stride_w == 2 && g.C <= 4 && g.pad_top >= 0 && g.pad_left >= 0 && g.pad_bottom >= 0 && g.pad_right >= 0) {
        auto floor_half = [](int a) { return a >= 0 ? a / 2 : -((-a + 1) / 2); };
        const int t0h = floor_half(-g.pad_top), t0w = floor_half(-g.pad_left);
        const int kh2 = floor_half(g.KH - 1 - g.pad_top) - t0h + 1, kw2 = floor_half(g.KW - 1 - g.pad_left) - t0w + 1;
        if (kw2 * 16 <= 128 && kh2 <= 64) {
            pl.path = kTcS2d;
            pl.bk = kw2 * 16 <= 64 ? 64 : 128;
            pl.c_pitch = pl.bk;
            pl.k_total = kh2 * pl.bk;
            pl.a_pitch = pl.bk;
            pl.kh2 = kh2; pl.kw2 = kw2; pl.t0h = t0h; pl.t0w = t0w;
            pl.rows2 = g.Ho + kh2 - 1;
            pl.cols2 = g.Wo + pl.bk / 16 - 1;  // the last window of a row ends inside the row, zero weights beyond kw2 blocks
            pl.Wb = largest_pow2_divisor(g.Wo, 16);
            pl.Hb = largest_pow2_divisor(g.Ho, 128 / pl.Wb);
            pl.Nb = 128 / (pl.Wb * pl.Hb);
            return pl;
        }
    }
    const bool direct = g.x_layout == CHXQ_NHWC && g.stride_h >= 1 && g.stride_w >= 1 && g.stride_h <= 8 && g.stride_w <= 8 && (xcs % 16 == 0) &&
                        g.pad_top >= 0 && g.pad_left >= 0 &&
                        g.pad_bottom >= 0 && g.pad_right >= 0 && g.pad_top < g.KH && g.pad_left < g.KW && g.C >= 16;
    if (direct) {
        pl.path = kTcDirect;
        pl.bk = choose_bk(g.C);
        pl.c_pitch = (g.C + pl.bk - 1) / pl.bk * pl.bk;
        pl.k_total = taps * pl.c_pitch;
        pl.a_pitch = pl.k_total;
        if (taps == 1 && g.stride_h == 1 && g.stride_w == 1 && g.pad_top == 0 && g.pad_left == 0 && g.pad_bottom == 0 && g.pad_right == 0 &&
            (int64_t)g.N * g.H * g.W < (1ll << 31)) {
            // 1x1: the map is a plain [N*H*W, C] matrix.
            pl.Wb = 128; pl.Hb = 1; pl.Nb = 1;
        } else {
            pl.Wb = largest_pow2_divisor(g.Wo, 16);
            pl.Hb = largest_pow2_divisor(g.Ho, 128 / pl.Wb);
            pl.Nb = 128 / (pl.Wb * pl.Hb);
        }
        return pl;
    }
    // Everything else with one group: explicit im2col into workspace, then a plain GEMM.
    // NCHW maps with up to 4 channels (a network stem) use one 32-bit word per pixel: channel pitch 4.
    const int cp = (g.x_layout == CHXQ_NCHW && g.C < 4) ? 4 : g.C;
    const int K = taps * cp;
    pl.path = kTcIm2col;
    // Large K tiles keep the TMA boxes wide; the part of the last tile beyond the matrix row is zero fill, not traffic.
    pl.bk = K > 64 ? 128 : (K > 32 ? 64 : 32);
    pl.c_pitch = cp;
    pl.k_total = (K + pl.bk - 1) / pl.bk * pl.bk;
    pl.a_pitch = (K + 15) / 16 * 16;
    pl.Wb = 128; pl.Hb = 1; pl.Nb = 1;
    return pl;
}

int launch_tc_igemm(const TcProblem& q, cudaStream_t s) {
    EncodeTiledFn encode = get_encode_fn();
    if (!encode) return set_error(CHXQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    if (q.bk != 32 && q.bk != 64 && q.bk != 128) return set_error(CHXQ_ERR_INVALID_ARGUMENT, "tensor-core kernel: bad bk %d", q.bk);
    if (q.Wb * q.Hb * q.Nb != 128) return set_error(CHXQ_ERR_INVALID_ARGUMENT, "tensor-core kernel: tile box must hold 128 positions");
    if ((reinterpret_cast<uintptr_t>(q.a) & 15u) || (reinterpret_cast<uintptr_t>(q.b) & 15u) || (q.a_cs % 16) || (q.c_pad % q.bk))
        return set_error(CHXQ_ERR_UNSUPPORTED, "tensor-core kernel: operands must be 16-byte aligned with 16-byte row pitch");
    if (q.cols <= 0 || q.Wo <= 0 || q.Ho <= 0 || q.No <= 0) return CHXQ_OK;

    // Epilogue family: the uint8 fast path covers everything except int8 outputs and weight zero-point terms.
    int epi_kind = tc::kEpiKInt32;
    if (q.epi.mode == kEpiRequant) {
        if (q.epi.rq.y_signed || q.col_mul != nullptr || q.epi.rq.round_mode != 0) {
            epi_kind = tc::kEpiKGeneric;  // int8 outputs, weight zero-point terms and round-half-to-even
        } else {
            epi_kind = q.epi.rq.fold ? tc::kEpiKU8Fold : tc::kEpiKU8;
        }
    }
    tc::TcParams p{};
    p.Wb = q.Wb; p.Hb = q.Hb; p.Nb = q.Nb;
    p.tiles_w = (q.Wo + q.Wb - 1) / q.Wb;
    p.tiles_h = (q.Ho + q.Hb - 1) / q.Hb;
    p.tiles_n = (q.No + q.Nb - 1) / q.Nb;
    const int64_t pos_tiles = (int64_t)p.tiles_w * p.tiles_h * p.tiles_n;
    if (q.group_cols > 0 && q.group_cols % 64 != 0)
        return set_error(CHXQ_ERR_UNSUPPORTED, "tensor-core kernel: grouped convolution needs a multiple of 64 output channels per group");
    const int bn = q.group_cols > 0 ? 64 : (epi_kind == tc::kEpiKGeneric ? 128 : (q.bn ? q.bn : pick_bn(q.cols, pos_tiles)));
    p.col_tiles = (q.cols + bn - 1) / bn;
    const int64_t total_tiles = pos_tiles * p.col_tiles;
    if (total_tiles >= (1ll << 31)) return set_error(CHXQ_ERR_UNSUPPORTED, "tensor-core kernel: too many tiles");
    p.Wo = q.Wo; p.Ho = q.Ho; p.No = q.No;
    p.KH = q.KH; p.KW = q.KW; p.pad_top = q.pad_top; p.pad_left = q.pad_left;
    p.sw = q.sw > 0 ? q.sw : 1; p.sh = q.sh > 0 ? q.sh : 1;
    p.group_cols = q.group_cols; p.group_cin = q.group_cin;
    if (p.sw > 8 || p.sh > 8 || q.Wb * p.sw > 256 || q.Hb * p.sh > 256)
        return set_error(CHXQ_ERR_UNSUPPORTED, "tensor-core kernel: stride %d x %d does not fit a TMA box", p.sh, p.sw);
    p.c_pad = q.c_pad;
    p.c_chunks = q.c_pad / q.bk;
    p.cols = q.cols;
    p.ldc = q.ldc;
    // Instruction descriptor (kind::i8): D format s32 (bits 4-5 = 2), A format bits 7-9 and B format bits
    // 10-12 (0 = u8, 1 = s8), both operands K-major (bits 15, 16 = 0), N >> 3 in bits 17-22, M >> 4 in bits 24-28.
    p.idesc = (2u << 4) | ((q.a_signed ? 1u : 0u) << 7) | ((q.b_signed ? 1u : 0u) << 10) | ((uint32_t)(bn >> 3) << 17) | ((128u >> 4) << 24);
    p.col_corr = q.col_corr; p.col_scale = q.col_scale; p.col_mul = q.col_mul; p.row_corr = q.row_corr;
    p.epi = q.epi;
    p.y = q.y;
#ifdef CHXQ_TL
    if (!g_tl_buf) cudaMalloc(&g_tl_buf, 5 * 2048 * sizeof(long long));
    cudaMemsetAsync(g_tl_buf, 0, 5 * 2048 * sizeof(long long), s);
    p.tl = g_tl_buf;
#endif
    p.wait_limit_ns = (unsigned long long)g_wait_limit_ns.load(std::memory_order_relaxed);
    p.test_skip_kb = g_test_skip_kb.load(std::memory_order_relaxed);
    p.status = device_status_ptr();
    if (!p.status) return set_error(CHXQ_ERR_CUDA, "device status word is unavailable");
    const int elt = q.epi.mode == kEpiInt32 ? 4 : 1;
    p.vec_ok = ((reinterpret_cast<uintptr_t>(q.y) & 15u) == 0) && ((q.ldc * elt) % 16 == 0) &&
               (q.epi.residual == nullptr || (reinterpret_cast<uintptr_t>(q.epi.residual) & 15u) == 0);

    // A: {C, W, H, N} bytes, pitches {a_cs, W*a_cs, H*W*a_cs}; box {bk, Wb, Hb, Nb} output positions, i.e. {bk, Wb*sw, Hb*sh, Nb}
    // input elements traversed with element strides {1, sw, sh, 1}; out-of-range reads fill 0.
    alignas(64) CUtensorMap tmA, tmB;
    {
        const cuuint64_t dims[4] = {(cuuint64_t)q.C, (cuuint64_t)q.W, (cuuint64_t)q.H, (cuuint64_t)q.N};
        const cuuint64_t row_bytes = q.a_row_bytes > 0 ? (cuuint64_t)q.a_row_bytes : (cuuint64_t)q.a_cs * q.W;
        const cuuint64_t strides[3] = {(cuuint64_t)q.a_cs, row_bytes, row_bytes * q.H};
        const cuuint32_t box[4] = {(cuuint32_t)q.bk, (cuuint32_t)(q.Wb * p.sw), (cuuint32_t)(q.Hb * p.sh), (cuuint32_t)q.Nb};
        const cuuint32_t estr[4] = {1, (cuuint32_t)p.sw, (cuuint32_t)p.sh, 1};
        CUresult r = encode(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(q.a), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            swizzle_for(q.bk), CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return set_error(CHXQ_ERR_CUDA, "cuTensorMapEncodeTiled(A) failed with %d", (int)r);
    }
    {
        const int taps = q.KH * q.KW;
        const cuuint64_t dims[2] = {(cuuint64_t)taps * q.c_pad, (cuuint64_t)q.cols};
        const cuuint64_t strides[1] = {(cuuint64_t)taps * q.c_pad};
        const cuuint32_t box[2] = {(cuuint32_t)q.bk, (cuuint32_t)bn};
        const cuuint32_t estr[2] = {1, 1};
        CUresult r = encode(&tmB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(q.b), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            swizzle_for(q.bk), CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return set_error(CHXQ_ERR_CUDA, "cuTensorMapEncodeTiled(B) failed with %d", (int)r);
    }
    int grid = total_tiles < num_sms() ? (int)total_tiles : num_sms();

    // Grouped-tile kernel (tc_kernel2.cuh): uint8 epilogues whose outputs (and residual) can move through TMA.
    bool grouped = false, halo = false;
    const bool pool = q.pool_ho > 0;
    const int g_variant = chxq::g_variant.load(std::memory_order_relaxed);  // one consistent value for this launch
    if (pool && (q.bk != 64 || q.Wb != 16 || q.Hb != 8 || q.Nb != 1 || q.epi.residual != nullptr || q.group_cols != 0 || q.pool_wo <= 0))
        return set_error(CHXQ_ERR_UNSUPPORTED, "tensor-core kernel: fused max pooling needs a 64-byte K tile, 16 x 8 position tiles and no residual");
    int bn2 = (q.cols > 64 && q.group_cols == 0 && !pool) ? 128 : 64;
    bool pair = false;  // the CTA-pair kernel (tc_kernel3.cuh)
    int64_t pair_items = 0;
    alignas(64) CUtensorMap tmY, tmR;
    if ((epi_kind == tc::kEpiKU8 || epi_kind == tc::kEpiKU8Fold) && (pool || g_variant != 1) && p.vec_ok && q.ldc % 16 == 0 && (q.bk == 64 || q.bk == 128) &&
        // folded tail: the saturating add clamps at zero, which is the Relu only when the output zero point is zero
        !(epi_kind == tc::kEpiKU8Fold && q.epi.residual != nullptr && q.epi.rq.res_relu && q.epi.rq.out_zp_f != 0.f)) {
        const int r = 256 / bn2;
        // Halo form: a KH x KW (<= 3 x 3) stride-1 convolution over the NHWC map with a 64-byte K tile; tiles are 8 x 16 positions
        // of one image.
        // by default for grouped / depthwise layers (measured: MobileNetV2 -7 %), on request (variant 3) for dense ones (ResNet-50's 3x3
        // layers are faster without: the halo planes are 16-byte TMA rows, and TMA moves about one row per clock)
        halo = !pool && ((g_variant >= 3 && g_variant <= 5) || (g_variant == 0 && q.group_cols > 0)) && q.KH * q.KW > 1 && q.KH <= 3 && q.KW <= 3 && p.sw == 1 && p.sh == 1 &&
               (q.bk == 64 || (q.bk == 128 && bn2 == 128 && q.epi.residual == nullptr)) && q.a_row_bytes == 0 && q.Wo >= 8 && q.Ho >= 8;
        // Space-to-depth stems: the A map is rows of 16-byte blocks read through overlapping 64-byte windows (a_cs 16 < C 64), i.e. a
        // KH x 4 stride-1 convolution over a 16-byte-pixel map.  As a halo tile every block is fetched once per tile instead of once per
        // window that covers it (up to 16 times), and the four blocks of a window are consecutive pixels of the halo row.
        const bool s2d_halo = g_variant != 1 && g_variant != 2 && q.a_row_bytes > 0 && q.a_cs == 16 && q.C == 64 && q.bk == 64 && q.KW == 1 &&
                              q.KH <= 4 && p.sw == 1 && p.sh == 1 && q.group_cols == 0 && q.Wo >= 8 && q.Ho >= 8;
        halo = halo || s2d_halo;
        p.halo_w = 8 + (s2d_halo ? 4 : q.KW) - 1;
        p.halo_h = 16 + q.KH - 1;
        p.halo_planes = s2d_halo ? 1 : q.bk / 16;
        p.halo_lbo = s2d_halo ? 1 : (tc::kHaloPlaneBytes >> 4);
        p.halo_kstep = s2d_halo ? 2 : 2 * (tc::kHaloPlaneBytes >> 4);
        int64_t pos_tiles2 = pos_tiles;
        if (halo) {
            p.Wb = 8; p.Hb = 16; p.Nb = 1;
            p.tiles_w = (q.Wo + 7) / 8; p.tiles_h = (q.Ho + 15) / 16; p.tiles_n = q.No;
            pos_tiles2 = (int64_t)p.tiles_w * p.tiles_h * p.tiles_n;
            if (pos_tiles2 * ((q.cols + bn2 - 1) / bn2) >= (1ll << 31)) return set_error(CHXQ_ERR_UNSUPPORTED, "tensor-core kernel: too many tiles");
        }
        int64_t groups = (pos_tiles2 + r - 1) / r * ((q.cols + bn2 - 1) / bn2);
        if (pool) {
            // a group of 2 x 2 tiles owns 15 x 7 pooled positions (see tc_kernel2.cuh)
            p.pool_wo = q.pool_wo; p.pool_ho = q.pool_ho;
            const int own_w = halo ? 7 : 15, own_h = halo ? 15 : 7;
            p.pool_groups_w = (q.pool_wo + own_w - 1) / own_w; p.pool_groups_h = (q.pool_ho + own_h - 1) / own_h;
            groups = (int64_t)p.pool_groups_w * p.pool_groups_h * q.No * ((q.cols + bn2 - 1) / bn2);
            if (groups >= (1ll << 31)) return set_error(CHXQ_ERR_UNSUPPORTED, "tensor-core kernel: too many tiles");
        }
        // CTA pairs (cta_group::2): dense layers with at least 256 output channels and a 128-byte K tile.  A pair works on two position
        // tiles against a 256-channel block; chosen when there is at least one such item for every second pair of SMs.
        pair_items = (pos_tiles + 1) / 2 * ((q.cols + 255) / 256);
        pair = !pool && !halo && g_variant != 1 && g_variant != 6 && q.bk == 128 && q.group_cols == 0 && q.cols >= 256 && q.a_row_bytes == 0 &&
               pair_items < (1ll << 31) &&
               (g_variant == 7 ||
                // by default where it measures faster: enough items to fill the pairs, and not the short-K layers with a residual tail
                // (fewer than four K tiles per item), which are bound by their epilogue and run slightly faster as grouped tiles
                ((g_variant == 0 || g_variant == 2) && pair_items >= (int64_t)num_sms() / 4 &&
                 !(q.epi.residual != nullptr && q.KH * q.KW * (q.c_pad / q.bk) < 4)));
        if (pair) bn2 = 128;  // the maps below are those of 128-channel blocks: one CTA's half of the weights, halves of the staged output
        // Chosen whenever there is at least one group per SM; smaller problems spread better as single tiles.
        grouped = pair || pool || halo || (g_variant >= 2 && g_variant <= 5) || groups >= (int64_t)num_sms();
        if (halo) {
            // space-to-depth: the block map itself, [N][rows][a_row_bytes / 16 blocks][16 bytes]
            const cuuint64_t dims[4] = {s2d_halo ? 16u : (cuuint64_t)q.C, s2d_halo ? (cuuint64_t)(q.a_row_bytes / 16) : (cuuint64_t)q.W, (cuuint64_t)q.H,
                                        (cuuint64_t)q.N};
            const cuuint64_t row_bytes = s2d_halo ? (cuuint64_t)q.a_row_bytes : (cuuint64_t)q.a_cs * q.W;
            const cuuint64_t strides[3] = {(cuuint64_t)q.a_cs, row_bytes, row_bytes * q.H};
            p.halo_swz = s2d_halo ? 0 : ((g_variant == 4 || g_variant == 5 || q.bk == 128) ? 1 : 0);  // 128-byte pixels: the swizzled form only
            const cuuint32_t box[4] = {p.halo_swz ? (cuuint32_t)q.bk : 16u, (cuuint32_t)p.halo_w, (cuuint32_t)p.halo_h, 1u};
            const cuuint32_t estr[4] = {1, 1, 1, 1};
            p.halo_row_map = s2d_halo ? 1 : 0;
            if (s2d_halo) {
                // rows of blocks are contiguous: {row bytes, rows, images, 1} with a box of halo_h rows of halo_w * 16 bytes moves the same
                // bytes to the same places in 19 long rows instead of 209 16-byte ones
                const cuuint64_t rdims[4] = {(cuuint64_t)q.a_row_bytes, (cuuint64_t)q.H, (cuuint64_t)q.N, 1};
                const cuuint64_t rstrides[3] = {(cuuint64_t)q.a_row_bytes, (cuuint64_t)q.a_row_bytes * q.H, (cuuint64_t)q.a_row_bytes * q.H * q.N};
                const cuuint32_t rbox[4] = {(cuuint32_t)(p.halo_w * 16), (cuuint32_t)p.halo_h, 1u, 1u};
                CUresult r0 = encode(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(q.a), rdims, rstrides, rbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                     CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
                if (r0 != CUDA_SUCCESS) return set_error(CHXQ_ERR_CUDA, "cuTensorMapEncodeTiled(A halo rows) failed with %d", (int)r0);
            } else {
                CUresult r0 = encode(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(q.a), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                     p.halo_swz ? swizzle_for(q.bk) : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
                if (r0 != CUDA_SUCCESS) return set_error(CHXQ_ERR_CUDA, "cuTensorMapEncodeTiled(A halo) failed with %d", (int)r0);
            }
        }
        if (grouped && pool) {
            tmY = tmA;  // the pooling form writes the pooled map with plain stores and reads no residual: the maps are placeholders
            tmR = tmA;
        } else if (grouped) {
            const cuuint64_t dims[4] = {(cuuint64_t)q.cols, (cuuint64_t)q.Wo, (cuuint64_t)q.Ho, (cuuint64_t)q.No};
            const cuuint64_t strides[3] = {(cuuint64_t)q.ldc, (cuuint64_t)q.ldc * q.Wo, (cuuint64_t)q.ldc * q.Wo * q.Ho};
            const cuuint32_t box[4] = {(cuuint32_t)bn2, (cuuint32_t)p.Wb, (cuuint32_t)p.Hb, (cuuint32_t)p.Nb};
            const cuuint32_t estr[4] = {1, 1, 1, 1};
            const CUtensorMapSwizzle sw = bn2 == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
            CUresult r1 = encode(&tmY, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, q.y, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                                 CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r1 != CUDA_SUCCESS) return set_error(CHXQ_ERR_CUDA, "cuTensorMapEncodeTiled(Y) failed with %d", (int)r1);
            void* rbase = q.epi.residual ? const_cast<uint8_t*>(q.epi.residual) : q.y;
            r1 = encode(&tmR, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, rbase, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r1 != CUDA_SUCCESS) return set_error(CHXQ_ERR_CUDA, "cuTensorMapEncodeTiled(R) failed with %d", (int)r1);
        }
        if (grouped) {
            // The weight box and the instruction shape follow the grouped kernel's channel block.
            const int taps = q.KH * q.KW;
            CUresult r1;
            const cuuint64_t bdims[2] = {(cuuint64_t)taps * q.c_pad, (cuuint64_t)q.cols};
            const cuuint64_t bstrides[1] = {(cuuint64_t)taps * q.c_pad};
            const cuuint32_t bbox[2] = {(cuuint32_t)q.bk, (cuuint32_t)bn2};
            const cuuint32_t bestr[2] = {1, 1};
            r1 = encode(&tmB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(q.b), bdims, bstrides, bbox, bestr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        swizzle_for(q.bk), CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r1 != CUDA_SUCCESS) return set_error(CHXQ_ERR_CUDA, "cuTensorMapEncodeTiled(B) failed with %d", (int)r1);
            p.col_tiles = (q.cols + bn2 - 1) / bn2;
            p.idesc = (p.idesc & ~(0x3fu << 17)) | ((uint32_t)(bn2 >> 3) << 17);
            grid = groups < num_sms() ? (int)groups : num_sms();
            if (pair) {
                // one instruction covers the pair: M = 256 (128 rows per CTA), N = 256
                p.col_tiles = (q.cols + 255) / 256;
                p.idesc = (p.idesc & ~((0x3fu << 17) | (0x1fu << 24))) | ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
            }
        }
    }
    // MatMulInteger / ConvInteger on CTA pairs: int32 accumulators written straight from registers (no staging, no output map).
    if (epi_kind == tc::kEpiKInt32 && !pool && g_variant != 1 && g_variant != 6 && q.bk == 128 && q.group_cols == 0 && q.cols >= 256 &&
        q.a_row_bytes == 0) {
        pair_items = (pos_tiles + 1) / 2 * ((q.cols + 255) / 256);
        pair = pair_items < (1ll << 31) && (g_variant == 7 || pair_items >= (int64_t)num_sms() / 4);
        if (pair) {
            const int taps = q.KH * q.KW;
            const cuuint64_t bdims[2] = {(cuuint64_t)taps * q.c_pad, (cuuint64_t)q.cols};
            const cuuint64_t bstrides[1] = {(cuuint64_t)taps * q.c_pad};
            const cuuint32_t bbox[2] = {(cuuint32_t)q.bk, 128u};  // one CTA's half of a 256-column block
            const cuuint32_t bestr[2] = {1, 1};
            CUresult r1 = encode(&tmB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(q.b), bdims, bstrides, bbox, bestr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                 swizzle_for(q.bk), CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r1 != CUDA_SUCCESS) return set_error(CHXQ_ERR_CUDA, "cuTensorMapEncodeTiled(B) failed with %d", (int)r1);
            tmY = tmA;  // placeholders: the int32 form stores from registers and reads no residual
            tmR = tmA;
            p.col_tiles = (q.cols + 255) / 256;
            p.idesc = (p.idesc & ~((0x3fu << 17) | (0x1fu << 24))) | ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
        }
    }
    ProfRec rec{};
    if (g_prof_on) {
        CHXQ_CUDA(cudaEventCreate(&rec.e0));
        CHXQ_CUDA(cudaEventCreate(&rec.e1));
        rec.macs = q.alg_macs;
        CHXQ_CUDA(cudaEventRecord(rec.e0, s));
    }
    if (pool && !grouped)
        return set_error(CHXQ_ERR_UNSUPPORTED, "tensor-core kernel: fused max pooling needs a uint8 epilogue and 16-byte aligned output rows");
    int rc;
    if (pool) {
        rc = tc::launch_tc2_bk64_pool(epi_kind, halo, tmA, tmB, tmY, tmR, p, grid, s);
    } else if (pair) {
        rc = tc::launch_tc3_bk128(epi_kind, epi_kind != tc::kEpiKInt32 && q.epi.residual != nullptr, tmA, tmB, tmY, tmR, p, (int)pair_items, s);
    } else if (grouped) {
        rc = q.bk == 128 ? tc::launch_tc2_bk128(bn2, epi_kind, q.epi.residual != nullptr, halo, tmA, tmB, tmY, tmR, p, grid, s)
                         : tc::launch_tc2_bk64(bn2, epi_kind, q.epi.residual != nullptr, halo, tmA, tmB, tmY, tmR, p, grid, s);
    } else
    switch (q.bk) {
        case 128: rc = tc::launch_tc_bk128(bn, epi_kind, tmA, tmB, p, grid, s); break;
        case 64: rc = tc::launch_tc_bk64(bn, epi_kind, tmA, tmB, p, grid, s); break;
        default: rc = tc::launch_tc_bk32(bn, epi_kind, tmA, tmB, p, grid, s); break;
    }
    if (g_prof_on) {
        CHXQ_CUDA(cudaEventRecord(rec.e1, s));
        std::lock_guard<std::mutex> lock(g_prof_mu);
        g_prof.push_back(rec);
    }
    return rc;
}

// Two convolutions as one kernel (tc_kernel4.cuh): q1 is any direct-path convolution with 64, 128 or 256 output channels and a folded
// uint8 requantization, q2 the 1x1 / stride-1 convolution that is its only reader (q2.a is not used: the intermediate map stays in
// shared memory).  CHXQ_ERR_UNSUPPORTED (without an error message being an error: the caller then runs the two layers) when
// the pair has no kernel.
int launch_tc_chain_igemm(const TcProblem& q1, const TcProblem& q2, cudaStream_t s) {
    EncodeTiledFn encode = get_encode_fn();
    if (!encode) return set_error(CHXQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    const int mid = q1.cols;
    const int bk = mid == 64 ? 64 : 128;
    auto folded_u8 = [](const EpiArgs& e) {
        return e.mode == kEpiRequant && !e.rq.y_signed && e.rq.round_mode == 0 && e.rq.fold != 0;
    };
    const bool ok = (mid == 64 || mid == 128 || mid == 256) && q1.bk == bk && q2.bk == bk && q1.group_cols == 0 && q1.a_row_bytes == 0 &&
                    q1.col_corr == nullptr && q1.col_mul == nullptr && q2.col_corr == nullptr && q2.col_mul == nullptr && folded_u8(q1.epi) &&
                    folded_u8(q2.epi) && q1.epi.residual == nullptr && q1.pool_ho == 0 && q2.pool_ho == 0 && q2.KH == 1 && q2.KW == 1 &&
                    q2.c_pad == mid && q2.C == mid && q2.group_cols == 0 && !q2.a_signed && q2.cols >= 16 && q2.cols <= (mid == 64 ? 512 : 1024) &&
                    q1.Wb * q1.Hb * q1.Nb == 128 && (q1.c_pad % bk) == 0 && (q1.a_cs % 16) == 0 && (q2.ldc % 16) == 0 &&
                    (reinterpret_cast<uintptr_t>(q1.a) & 15u) == 0 && (reinterpret_cast<uintptr_t>(q1.b) & 15u) == 0 &&
                    (reinterpret_cast<uintptr_t>(q2.b) & 15u) == 0 && (reinterpret_cast<uintptr_t>(q2.y) & 15u) == 0 &&
                    (q2.epi.residual == nullptr || (reinterpret_cast<uintptr_t>(q2.epi.residual) & 15u) == 0) &&
                    !(q2.epi.residual != nullptr && q2.epi.rq.res_relu && q2.epi.rq.out_zp_f != 0.f) &&
                    (int64_t)q1.Wo * q1.Ho * q1.No == (int64_t)q2.Wo * q2.Ho * q2.No;
    if (!ok) return set_error(CHXQ_ERR_UNSUPPORTED, "two-convolution kernel: this pair of layers has no fused kernel");
    if (q1.Wo <= 0 || q1.Ho <= 0 || q1.No <= 0) return CHXQ_OK;
    tc::ChainParams p{};
    p.Wb = q1.Wb; p.Hb = q1.Hb; p.Nb = q1.Nb;
    p.tiles_w = (q1.Wo + q1.Wb - 1) / q1.Wb;
    p.tiles_h = (q1.Ho + q1.Hb - 1) / q1.Hb;
    p.tiles_n = (q1.No + q1.Nb - 1) / q1.Nb;
    const int64_t pos_tiles = (int64_t)p.tiles_w * p.tiles_h * p.tiles_n;
    if (pos_tiles >= (1ll << 31) / 16) return set_error(CHXQ_ERR_UNSUPPORTED, "two-convolution kernel: too many tiles");
    p.KH = q1.KH; p.KW = q1.KW; p.pad_top = q1.pad_top; p.pad_left = q1.pad_left;
    p.sw = q1.sw > 0 ? q1.sw : 1; p.sh = q1.sh > 0 ? q1.sh : 1;
    if (p.sw > 8 || p.sh > 8 || q1.Wb * p.sw > 256 || q1.Hb * p.sh > 256)
        return set_error(CHXQ_ERR_UNSUPPORTED, "two-convolution kernel: stride %d x %d does not fit a TMA box", p.sh, p.sw);
    p.c_chunks = q1.c_pad / bk;
    p.out_cols = q2.cols;
    p.idesc1 = (2u << 4) | ((q1.a_signed ? 1u : 0u) << 7) | ((q1.b_signed ? 1u : 0u) << 10) | ((uint32_t)(mid >> 3) << 17) | ((128u >> 4) << 24);
    p.idesc2 = (2u << 4) | ((q2.b_signed ? 1u : 0u) << 10) | ((uint32_t)(128 >> 3) << 17) | ((128u >> 4) << 24);
    p.epi1 = q1.epi;
    p.epi2 = q2.epi;
#ifdef CHXQ_TL
    if (!g_tl_buf) cudaMalloc(&g_tl_buf, 5 * 2048 * sizeof(long long));
    cudaMemsetAsync(g_tl_buf, 0, 5 * 2048 * sizeof(long long), s);
    p.tl = g_tl_buf;
#endif
    p.wait_limit_ns = (unsigned long long)g_wait_limit_ns.load(std::memory_order_relaxed);
    p.status = device_status_ptr();
    if (!p.status) return set_error(CHXQ_ERR_CUDA, "device status word is unavailable");

    alignas(64) CUtensorMap tmA, tmB1, tmB2, tmY, tmR;
    const cuuint32_t ones4[4] = {1, 1, 1, 1};
    {
        const cuuint64_t dims[4] = {(cuuint64_t)q1.C, (cuuint64_t)q1.W, (cuuint64_t)q1.H, (cuuint64_t)q1.N};
        const cuuint64_t row_bytes = (cuuint64_t)q1.a_cs * q1.W;
        const cuuint64_t strides[3] = {(cuuint64_t)q1.a_cs, row_bytes, row_bytes * q1.H};
        const cuuint32_t box[4] = {(cuuint32_t)bk, (cuuint32_t)(q1.Wb * p.sw), (cuuint32_t)(q1.Hb * p.sh), (cuuint32_t)q1.Nb};
        const cuuint32_t estr[4] = {1, (cuuint32_t)p.sw, (cuuint32_t)p.sh, 1};
        CUresult r = encode(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(q1.a), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            swizzle_for(bk), CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return set_error(CHXQ_ERR_CUDA, "cuTensorMapEncodeTiled(A) failed with %d", (int)r);
    }
    {
        // four dimensions (the last two of extent 1): the kernel fetches positions and weights with one instruction form
        const int taps = q1.KH * q1.KW;
        const cuuint64_t row = (cuuint64_t)taps * q1.c_pad;
        const cuuint64_t dims[4] = {row, (cuuint64_t)mid, 1, 1};
        const cuuint64_t strides[3] = {row, row * mid, row * mid};
        const cuuint32_t box[4] = {(cuuint32_t)bk, (cuuint32_t)mid, 1, 1};
        CUresult r = encode(&tmB1, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(q1.b), dims, strides, box, ones4, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            swizzle_for(bk), CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return set_error(CHXQ_ERR_CUDA, "cuTensorMapEncodeTiled(B1) failed with %d", (int)r);
    }
    {
        const cuuint64_t dims[2] = {(cuuint64_t)mid, (cuuint64_t)q2.cols};
        const cuuint64_t strides[1] = {(cuuint64_t)mid};
        const cuuint32_t box[2] = {(cuuint32_t)bk, 128u};
        CUresult r = encode(&tmB2, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(q2.b), dims, strides, box, ones4, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            swizzle_for(bk), CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return set_error(CHXQ_ERR_CUDA, "cuTensorMapEncodeTiled(B2) failed with %d", (int)r);
    }
    {
        const cuuint64_t dims[4] = {(cuuint64_t)q2.cols, (cuuint64_t)q1.Wo, (cuuint64_t)q1.Ho, (cuuint64_t)q1.No};
        const cuuint64_t strides[3] = {(cuuint64_t)q2.ldc, (cuuint64_t)q2.ldc * q1.Wo, (cuuint64_t)q2.ldc * q1.Wo * q1.Ho};
        const cuuint32_t box[4] = {128u, (cuuint32_t)p.Wb, (cuuint32_t)p.Hb, (cuuint32_t)p.Nb};
        CUresult r = encode(&tmY, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, q2.y, dims, strides, box, ones4, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return set_error(CHXQ_ERR_CUDA, "cuTensorMapEncodeTiled(Y) failed with %d", (int)r);
        void* rbase = q2.epi.residual ? const_cast<uint8_t*>(q2.epi.residual) : q2.y;
        r = encode(&tmR, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, rbase, dims, strides, box, ones4, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return set_error(CHXQ_ERR_CUDA, "cuTensorMapEncodeTiled(R) failed with %d", (int)r);
    }
    const int grid = pos_tiles < num_sms() ? (int)pos_tiles : num_sms();
    ProfRec rec{};
    if (g_prof_on) {
        CHXQ_CUDA(cudaEventCreate(&rec.e0));
        CHXQ_CUDA(cudaEventCreate(&rec.e1));
        rec.macs = q1.alg_macs + q2.alg_macs;
        CHXQ_CUDA(cudaEventRecord(rec.e0, s));
    }
    const int rc = tc::launch_tc_chain(mid, q2.epi.residual != nullptr, tmA, tmB1, tmB2, tmY, tmR, p, grid, s);
    if (g_prof_on) {
        CHXQ_CUDA(cudaEventRecord(rec.e1, s));
        std::lock_guard<std::mutex> lock(g_prof_mu);
        g_prof.push_back(rec);
    }
    return rc;
}

}  // namespace chxq

// Chooses between the two tensor-core kernels: 0 = by problem shape, 1 = always one tile per step, 2 = grouped tiles
// whenever the problem is eligible.  Results are identical; the switch exists for measurements and tests.
extern "C" int chxq_tc_variant(int32_t variant) {
    if (variant < 0 || variant > 7) return chxq::set_error(CHXQ_ERR_INVALID_ARGUMENT, "chxq_tc_variant: variant must be 0 .. 7");
    chxq::g_variant.store(variant, std::memory_order_relaxed);
    return CHXQ_OK;
}

#ifdef CHXQ_TL
extern "C" int chxq_tl_read(long long* host) {
    cudaDeviceSynchronize();
    return (int)cudaMemcpy(host, chxq::g_tl_buf, 5 * 2048 * sizeof(long long), cudaMemcpyDeviceToHost);
}
#endif

// Test hooks of the bounded device-side waits (one-tile kernel): the time without progress after which a wait gives up, and the
// K block whose weight load the producer leaves out (-1: none), so that a test can make a wait run out without faulting anything.
extern "C" int chxq_tc_test_hooks(int64_t wait_limit_ns, int32_t skip_weight_load_kb) {
    if (wait_limit_ns < 1000000 || wait_limit_ns > 10000000000ll)
        return chxq::set_error(CHXQ_ERR_INVALID_ARGUMENT, "chxq_tc_test_hooks: the wait limit must lie between 1 ms and 10 s");
    chxq::g_wait_limit_ns.store(wait_limit_ns, std::memory_order_relaxed);
    chxq::g_test_skip_kb.store(skip_weight_load_kb, std::memory_order_relaxed);
    return CHXQ_OK;
}

// Number of CTA pairs of the paired tensor-core kernel that the current device keeps resident at once.
extern "C" int chxq_tc_pair_slots(int32_t* slots) {
    if (!slots) return chxq::set_error(CHXQ_ERR_INVALID_ARGUMENT, "chxq_tc_pair_slots: null pointer");
    int n = 0;
    const int rc = chxq::tc::tc3_pair_slots(&n);
    *slots = n;
    return rc;
}

// Profiling of the tensor-core kernel: while enabled, every launch is bracketed by CUDA events on its stream.
extern "C" int chxq_tc_profile(int32_t enable) {
    std::lock_guard<std::mutex> lock(chxq::g_prof_mu);
    chxq::g_prof_on = enable != 0;
    return CHXQ_OK;
}

// Synchronises the device, sums the recorded launches and clears them.
extern "C" int chxq_tc_profile_read(double* total_ms, int64_t* launches, double* total_macs) {
    using namespace chxq;
    CHXQ_CUDA(cudaDeviceSynchronize());
    std::lock_guard<std::mutex> lock(g_prof_mu);
    double ms = 0.0, macs = 0.0;
    for (auto& r : g_prof) {
        float t = 0.f;
        CHXQ_CUDA(cudaEventElapsedTime(&t, r.e0, r.e1));
        ms += t;
        macs += r.macs;
        cudaEventDestroy(r.e0);
        cudaEventDestroy(r.e1);
    }
    if (total_ms) *total_ms = ms;
    if (launches) *launches = (int64_t)g_prof.size();
    if (total_macs) *total_macs = macs;
    g_prof.clear();
    return CHXQ_OK;
}
