// Interface between the host side of the tensor-core kernel (tc_igemm.cu) and its per-K-tile translation units.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include "epilogue.cuh"

namespace chxq {
namespace tc {

constexpr int kHaloPlaneBytes = 3072;  // bytes reserved per plane of a halo tile: 18 x 10 pixels x 16 bytes = 2880, rounded up to 128

struct TcParams {
    int Wb, Hb, Nb;
    int tiles_w, tiles_h, tiles_n;  // position tiles
    int col_tiles;                   // ceil(cols / BN)
    int Wo, Ho, No;
    int KH, KW, pad_top, pad_left;
    int sw, sh;  // convolution strides: input coordinate = output coordinate * stride - pad + tap
    int halo_swz;  // halo form: 0 = planes of 16-byte rows without swizzle, 1 = one swizzled tile of BK-byte rows
    // halo form: halo tile of halo_w x halo_h pixels in halo_planes planes of [pixel][16 bytes]; the two 16-byte K halves of an MMA are
    // halo_lbo 16-byte units apart (one plane for channel chunks; one pixel for the space-to-depth stem, whose K runs along the row),
    // consecutive MMAs of a tap halo_kstep units
    int halo_w, halo_h, halo_planes, halo_lbo, halo_kstep;
    int halo_row_map;  // the A map is {bytes of a row, rows, images}: a halo tile is halo_h rows of halo_w * 16 contiguous bytes (16-byte pixels only)
    int group_cols, group_cin;  // grouped convolution (0 = one group): first input channel of a column tile = (col0 / group_cols) * group_cin
    int c_chunks;  // c_pad / BK
    int c_pad;
    int cols;
    int64_t ldc;
    uint32_t idesc;
    const int32_t* col_corr;
    int col_scale;
    const int32_t* col_mul;
    const int32_t* row_corr;
    EpiArgs epi;
    void* y;
    int* status;
    int vec_ok;  // rows of y (and of the residual) start on 16-byte boundaries
    // Fused 3x3 / stride-2 max pooling (grouped kernel, 64-channel blocks): y is the POOLED map [No, pool_ho, pool_wo, ldc]; a
    // group is 2 x 2 tiles of 16 x 8 positions and owns 15 x 7 pooled positions (8 x 16 and 7 x 15 with halo tiles).
    // pool_groups_w == 0: no pooling.
    int pool_groups_w, pool_groups_h, pool_wo, pool_ho;
    // Bounded waits: nanoseconds without progress after which a wait gives up (2 s unless a test shortens it), and, for the test of
    // that path only, the K block whose weight load the one-tile kernel's producer leaves out (-1: none).
    unsigned long long wait_limit_ns;
    int test_skip_kb;
#ifdef CHXQ_TL
    long long* tl;  // timeline build: [2 roles][512 K blocks][4] clock stamps of CTA 0
#endif
};

// Parameters of the two-convolution kernel (tc_kernel4.cuh): a KH x KW convolution whose uint8 output feeds a 1x1 / stride-1
// convolution, tile by tile through shared memory.  Position tiles, taps and strides describe the first convolution; the second
// one has the same output positions.
struct ChainParams {
    int Wb, Hb, Nb;
    int tiles_w, tiles_h, tiles_n;
    int KH, KW, pad_top, pad_left;
    int sw, sh;
    int c_chunks;            // K tiles per tap of the first convolution
    int out_cols;            // output channels of the second convolution
    uint32_t idesc1, idesc2;  // instruction descriptors: N = the first convolution's channels, N = 128
    EpiArgs epi1, epi2;      // folded uint8 requantizations; epi2 may carry the residual tail
    int* status;
    unsigned long long wait_limit_ns;
#ifdef CHXQ_TL
    long long* tl;  // timeline build: (code, clock) pairs of CTA 0: [MMA thread | epilogue warp 2 | store warp] x 2048 entries
#endif
};

// Epilogue families (template parameter EPI): dead paths are compiled out, which keeps the unrolled per-element
// code of each kernel small enough for the instruction cache.
constexpr int kEpiKInt32 = 0;    // store the int32 accumulator
constexpr int kEpiKU8 = 1;       // requantize to uint8, optional residual tail
constexpr int kEpiKGeneric = 2;  // int8 output and/or a weight zero-point term: general requantization
constexpr int kEpiKU8Fold = 3;   // uint8 with one folded multiplier per channel (RequantParams::fold)

int launch_tc_bk32(int bn, int epi, const CUtensorMap& tmA, const CUtensorMap& tmB, const TcParams& p, int grid, cudaStream_t s);
int launch_tc_bk64(int bn, int epi, const CUtensorMap& tmA, const CUtensorMap& tmB, const TcParams& p, int grid, cudaStream_t s);
int launch_tc_bk128(int bn, int epi, const CUtensorMap& tmA, const CUtensorMap& tmB, const TcParams& p, int grid, cudaStream_t s);
// Grouped-tile kernel (tc_kernel2.cuh); bn is 64 or 128, epi is kEpiKU8 or kEpiKU8Fold.
// pool: the fused max-pooling form (bn 64, no residual; 64-byte K tiles only), with or without halo tiles.
int launch_tc2_bk64_pool(int epi, bool halo, const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmY, const CUtensorMap& tmR, const TcParams& p,
                         int grid, cudaStream_t s);
int launch_tc2_bk64(int bn, int epi, bool res, bool halo, const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmY, const CUtensorMap& tmR,
                    const TcParams& p, int grid, cudaStream_t s);
int launch_tc2_bk128(int bn, int epi, bool res, bool halo, const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmY, const CUtensorMap& tmR,
                     const TcParams& p, int grid, cudaStream_t s);

// CTA-pair kernel (tc_kernel3.cuh): 256-channel blocks, 128-byte K tiles, uint8 epilogues; tmB's box is one CTA's half of the
// weight block (128 rows), tmY / tmR boxes are 128 channels wide; items = position-tile pairs x 256-channel blocks.
int launch_tc3_bk128(int epi, bool res, const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmY, const CUtensorMap& tmR, const TcParams& p,
                     int items, cudaStream_t s);

// Two-convolution kernel; mid = channels between the two convolutions (64, 128 or 256; K tile 64 bytes for 64, else 128).
int launch_tc_chain(int mid, bool res, const CUtensorMap& tmA, const CUtensorMap& tmB1, const CUtensorMap& tmB2, const CUtensorMap& tmY,
                    const CUtensorMap& tmR, const ChainParams& p, int grid, cudaStream_t s);

int tc3_pair_slots(int* out);  // CTA pairs the current device keeps resident at once

long long wait_limit_ns_value();  // limit of the bounded device-side waits (chxq_tc_test_hooks; default 2 s)
// Unswizzled tensor map over an NHWC uint8 map {C, W, H, N} with cs bytes between pixels (a multiple of 16, base 16-byte aligned); a box is
// box_c bytes (a multiple of 16) x box_w pixels x box_h rows of one image; reads outside the map fill 0.
int encode_nhwc_box_map(CUtensorMap* out, const void* base, int C, int W, int H, int N, int64_t cs, int box_c, int box_w, int box_h);

}  // namespace tc
}  // namespace chxq
