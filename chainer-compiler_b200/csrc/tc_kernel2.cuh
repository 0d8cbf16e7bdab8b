// Grouped-tile variant of the tcgen05 implicit-GEMM kernel for the uint8 requantizing epilogues (device code; the host
// side is in tc_igemm.cu).  Same roles and the same operand staging as tc_kernel.cuh; what changes is the unit of work and
// how results leave the SM:
//
//   * A CTA works on a GROUP of R position tiles (R x 128 output positions) against one block of BN output channels:
//     R = 2 with BN = 128, R = 4 with BN = 64.  One weight stage feeds R MMAs, and an epilogue thread keeps the
//     per-channel multiplier and offset of a 16-channel chunk in registers while it requantizes that chunk of all R
//     tiles, so the shared-memory reads of the per-channel parameters drop by R.
//   * Outputs are written into a swizzled shared-memory staging tile (conflict-free 128-bit stores) and leave through a TMA
//     store; the residual map of a fused residual tail arrives the same way through a TMA load issued by the producer
//     warp.  A thread owns one output position (TMEM lane), so direct global accesses would touch 32 different lines per
//     warp instruction; through shared memory every line is moved once, whole.
//   * The TMA store clips rows and channels beyond the output, so ragged edges need no predicates.
//
//   * The folded requantization runs in units of the output range, so that the saturating fma is both clamps, and on pairs of
//     floats (fma / sub .f32x2) wherever no clamp is involved.
//
//   * A nineteenth warp issues the TMA stores: the epilogue warps only count themselves in on an mbarrier when their part
//     of a group is staged, so they never wait for one another.  A twentieth warp is the weights' TMA producer.
//
// TMEM holds two groups (2 x R x BN = 512 columns): the epilogue of group i overlaps the main loop of group i + 1.  The
// staging tiles are multi-buffered as well.  Every wait is bounded exactly as in tc_kernel.cuh.
#pragma once

#include <utility>

#include "tc_kernel.cuh"

namespace chxq {
namespace tc {

__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(reinterpret_cast<uint64_t>(map)),
                 "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
                 : "memory");
}

__device__ __forceinline__ void tma_store_commit() {
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void tma_store_wait_all() {
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

__device__ __forceinline__ void fence_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// HALO: the A operand of a KH x KW (<= 3 x 3), stride-1 convolution is staged once per tile and channel chunk as the halo
// tile of an 8 x 16 block of output positions of one image -- (16 + KH - 1) x (8 + KW - 1) pixels -- instead of once per
// tap: each tap is a shifted view of the same bytes.  The halo tile is stored WITHOUT swizzle as BK / 16 planes of
// [pixel][16 bytes]: in the canonical K-major layout a core matrix is 8 rows of 16 bytes, 16 bytes apart, so eight
// consecutive pixels of an image row are one core matrix wherever the view starts; the stride between 8-row groups (SBO)
// is one halo row, the stride between the two K halves of an MMA (LBO) is one plane.  Weight stages keep their own ring.
constexpr int kHaloPlane = kHaloPlaneBytes;  // a space-to-depth stem uses one plane of 19 x 11 pixels (3344 bytes) at the start of a tile's planes
constexpr int kHaloWb = 8, kHaloHb = 16;

template <int BN, int BK, bool RES, bool HALO = false>
struct Tc2Config {
    static constexpr int kR = 256 / BN;                  // position tiles per group
    static constexpr int kTileA = HALO ? (BK / 16) * kHaloPlane : 128 * BK;
    static constexpr int kStageA = kR * kTileA;
    static constexpr int kAStages = 2;                   // HALO only: ring of halo-tile stages
    static constexpr int kStageB = BN * BK;
    static constexpr int kStageBytes = HALO ? kStageB : kStageA + kStageB;  // bytes of one stage of the main ring
    static constexpr int kTileOut = 128 * BN;            // one staged output (or residual) tile
    // Staging buffers of kR tiles each.  Without a residual: two, filled by the epilogue and drained by the TMA store.
    // With one: three, each filled by the residual's TMA load, overwritten in place by the epilogue (a thread reads and
    // writes the same 16 bytes) and drained by the store; three, so that the load for group i + 1 can run during the
    // epilogue of group i while the store of group i - 1 is still reading its buffer.
    static constexpr int kBufs = RES ? ((BN == 64 && BK == 128 && !HALO) ? 2 : 3) : 2;  // 64-channel blocks with 128-byte K tiles: two, for room
    static constexpr int kOutBytes = kBufs * kR * kTileOut;
    static constexpr int kFixed = kOutBytes + (HALO ? kAStages * kStageA : 0);
    static constexpr int kBudget = 222 * 1024;
    static constexpr int kStagesRaw = (kBudget - kFixed) / kStageBytes;
    static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
    static constexpr int kTmemCols = 512;
    // barriers: full[kStages], empty[kStages], tmem_full[2], tmem_empty[2], res_full[3], buf_empty[3], buf_full[3],
    // halo_full[2], halo_empty[2]
    static constexpr int kBarBytes = (2 * kStages + 17) * 8;
    static constexpr int kBarOffset = kStages * kStageBytes + kFixed;
    static constexpr int kParamOffset = ((kBarOffset + kBarBytes + 16 + 15) / 16) * 16;
    static constexpr int kParamBytes = 16 * (3 * BN / 4) * 4;  // 16 warps x (BN/4 multipliers + BN/4 additive terms + BN/4 zero-point terms)
    static constexpr int kSmemBytes = 1024 /*alignment slack*/ + kParamOffset + kParamBytes;
    static constexpr bool kUsable = kStages >= 2;
};

// Byte offset of 16-byte unit `unit` of row `row` inside a staged [128][BN] tile laid out with the BN-byte TMA swizzle.
template <int BN>
__device__ __forceinline__ uint32_t staged_offset(int row, int unit) {
    if (BN == 128) return (uint32_t)(row * 128 + ((unit ^ (row & 7)) << 4));
    return (uint32_t)(row * 64 + ((unit ^ ((row >> 1) & 3)) << 4));
}

// K-major descriptor of a shifted view into a halo tile (no swizzle): LBO = one plane, SBO = one halo row.
__device__ __forceinline__ uint64_t make_halo_desc(uint32_t smem_addr, uint32_t row_bytes) {
    return (uint64_t)((smem_addr >> 4) & 0x3fffu) | ((uint64_t)(kHaloPlane >> 4) << 16) | ((uint64_t)(row_bytes >> 4) << 32) | (1ull << 46);
}

// POOL: the 3x3 / stride-2 max pooling that follows the convolution runs on the staged tiles, and only the pooled map is
// written.  A group is then 2 x 2 tiles of 16 x 8 output positions (8 x 16 with halo tiles) whose origin advances by 30
// columns and 14 rows per group (14 and 30), so that every pooling window of the 15 x 7 (7 x 15) pooled positions a group
// owns lies inside it (neighbouring groups recompute the two overlapping columns and rows: 512 positions computed for 420
// kept).  BN = 64 only.
template <bool HALO>
struct PoolGeom {
    static constexpr int kTileW = HALO ? 8 : 16, kTileH = HALO ? 16 : 8;  // positions of one tile
    static constexpr int kW = kTileW - 1, kH = kTileH - 1;                 // pooled positions a group owns
};
// NARROW = V > 0: the operator has at most V x 16 output channels (V = 1 or 2; one column tile).  With every fourth chunk per warp only V
// of the four warps of a lane quarter would have work, so the units (chunk, tile) are dealt out tile by tile instead: warp `sub` takes
// chunk sub % V of tiles (sub + 4 u) / V, and still needs the parameters of one chunk only (cache slot 0).  A template argument, because
// the same choice made at run time cost every other layer 3-8 %.
template <int BN, int BK, int EPI, bool RES, bool HALO, bool POOL = false, int NARROW = 0>
__global__ void __launch_bounds__(640, 1)
tc_igemm2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmY,
                 const __grid_constant__ CUtensorMap tmR, const TcParams p) {
    using Cfg = Tc2Config<BN, BK, RES, HALO>;
    constexpr int kStages = Cfg::kStages;
    constexpr int kR = Cfg::kR;
    constexpr bool kFold = EPI == kEpiKU8Fold;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);  // stays a shared-memory pointer
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + (HALO ? Cfg::kAStages : kStages) * Cfg::kStageA;
    uint8_t* smem_out = smem_b + kStages * Cfg::kStageB;  // [kBufs][kR][128][BN], 1024-byte aligned (all sizes are multiples of 1024)
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kBarOffset);
    uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 17);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

    const uint32_t bar_base = smem_u32(bars);
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * kStages + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * kStages + 2 + a); };
    auto rfull_bar = [&](int b) { return bar_base + 8u * (2 * kStages + 4 + b); };
    // buffer b of the staging ring: empty = the store out of it has read it (the residual load / the epilogue may write it),
    // full = all sixteen epilogue warps have staged their part of it
    auto bempty_bar = [&](int b) { return bar_base + 8u * (2 * kStages + 7 + b); };
    auto bfull_bar = [&](int b) { return bar_base + 8u * (2 * kStages + 10 + b); };
    auto hfull_bar = [&](int a) { return bar_base + 8u * (2 * kStages + 13 + a); };
    auto hempty_bar = [&](int a) { return bar_base + 8u * (2 * kStages + 15 + a); };

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), 16);  // one arrival per epilogue warp
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(hfull_bar(a), 1);
            mbar_init(hempty_bar(a), 1);
        }
        for (int b = 0; b < 3; ++b) {
            mbar_init(rfull_bar(b), 1);
            mbar_init(bempty_bar(b), POOL ? 16 : 1);  // the store warp; pooling form: the sixteen epilogue warps
            mbar_init(bfull_bar(b), 16);  // one arrival per epilogue warp
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_ptr_smem), Cfg::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr_smem;
    pdl_launch_dependents();  // the next kernel's CTAs may take this SM as soon as this CTA leaves it
    pdl_dependency_wait();    // from here on the previous kernel's output (this kernel's input) is complete and visible

    static_assert(!POOL || (BN == 64 && !RES), "fused pooling: 64-channel blocks without a residual");
    using PG = PoolGeom<HALO>;
    const int pos_tiles = p.tiles_w * p.tiles_h * p.tiles_n;
    const int pos_groups = POOL ? p.pool_groups_w * p.pool_groups_h * p.No : (pos_tiles + kR - 1) / kR;
    const int total_groups = pos_groups * p.col_tiles;
    const int taps = p.KH * p.KW;
    const int num_kb = taps * p.c_chunks;

    // Output coordinates of position tile `pt` (tiles past the end land beyond the last image: loads fill zero, stores
    // are skipped).
    auto tile_origin = [&](int pt, int& w0, int& h0, int& n0) {
        const int tw = pt % p.tiles_w;
        pt /= p.tiles_w;
        const int th = pt % p.tiles_h;
        const int tn = pt / p.tiles_h;
        w0 = tw * p.Wb; h0 = th * p.Hb; n0 = tn * p.Nb;
    };
    // POOL: origin of group pg in output coordinates; tile t of the group sits one tile to the right for t & 1, one down for t >> 1.
    auto pool_group_origin = [&](int pg, int& gw0, int& gh0, int& n) {
        const int gw = pg % p.pool_groups_w;
        pg /= p.pool_groups_w;
        const int gh = pg % p.pool_groups_h;
        n = pg / p.pool_groups_h;
        gw0 = gw * (2 * PG::kW);
        gh0 = gh * (2 * PG::kH);
    };

    if (warp == 0 || (warp == 19 && !HALO)) {
        // ---------------- TMA producers ----------------
        // Warp 0 loads the positions (and the residual tiles); without halo tiles warp 19 loads the weights.  One thread per
        // operand: a thread that issues a tensor copy is held until the copy engine takes it, and with one thread for both operands
        // the engine idles while that thread waits for the next free stage.  (Halo form: warp 0 loads both.)
        // Tensor copies issued by one warp are processed one instruction after the other (each takes about one memory latency, whatever
        // its size), but the copies of several lanes of ONE instruction run side by side: so the whole warp walks the loop, and the kR
        // tiles of a stage (or of a residual group) are fetched by kR lanes in a single instruction.
        if (HALO ? lane == 0 : true) {
            const bool is_a = warp == 0;
            int stage = 0, hstage = 0;
            uint32_t phase = 0, hphase = 0;
            bool ok = true;
            int it = 0;
            for (int grp = blockIdx.x; grp < total_groups && ok; grp += gridDim.x, ++it) {
                const int ct = grp % p.col_tiles;
                const int pg = grp / p.col_tiles;
                int w0[kR], h0[kR], n0[kR];
                if (POOL) {
                    int gw0, gh0, gn;
                    pool_group_origin(pg, gw0, gh0, gn);
#pragma unroll
                    for (int t = 0; t < kR; ++t) {
                        w0[t] = gw0 + PG::kTileW * (t & 1);
                        h0[t] = gh0 + PG::kTileH * (t >> 1);
                        n0[t] = gn;
                    }
                } else {
#pragma unroll
                    for (int t = 0; t < kR; ++t) tile_origin(pg * kR + t, w0[t], h0[t], n0[t]);
                }
                // this lane's tile (non-halo form: lane t < kR fetches tile t)
                int lw0 = w0[0], lh0 = h0[0], ln0 = n0[0];
#pragma unroll
                for (int t = 1; t < kR; ++t)
                    if (lane == t) {
                        lw0 = w0[t]; lh0 = h0[t]; ln0 = n0[t];
                    }
                const int gbase = p.group_cols > 0 ? (ct * BN / p.group_cols) * p.group_cin : 0;
                if (RES && is_a) {
                    const int rb = it % Cfg::kBufs;
                    if (HALO) {
                        if (!mbar_wait(bempty_bar(rb), ((uint32_t)(it / Cfg::kBufs) & 1u) ^ 1u, abort_flag, p.status, 5, 0)) break;
                        mbar_expect_tx(rfull_bar(rb), kR * Cfg::kTileOut);
#pragma unroll
                        for (int t = 0; t < kR; ++t)
                            tma_load_4d(smem_u32(smem_out + (rb * kR + t) * Cfg::kTileOut), &tmR, rfull_bar(rb), ct * BN, w0[t], h0[t], n0[t]);
                    } else {
                        ok = __all_sync(0xffffffffu, mbar_wait(bempty_bar(rb), ((uint32_t)(it / Cfg::kBufs) & 1u) ^ 1u, abort_flag, p.status, 5, 0));
                        if (!ok) break;
                        if (lane == 0) mbar_expect_tx(rfull_bar(rb), kR * Cfg::kTileOut);
                        __syncwarp();
                        if (lane < kR) tma_load_4d(smem_u32(smem_out + (rb * kR + lane) * Cfg::kTileOut), &tmR, rfull_bar(rb), ct * BN, lw0, lh0, ln0);
                        __syncwarp();
                    }
                }
                if (HALO) {
                    // one halo tile per position tile and channel chunk, then one weight stage per tap
                    const uint32_t halo_bytes = (uint32_t)(p.halo_w * p.halo_h * 16);
                    for (int cc = 0; cc < p.c_chunks && ok; ++cc) {
                        if (!mbar_wait(hempty_bar(hstage), hphase ^ 1u, abort_flag, p.status, 9, 0)) {
                            ok = false;
                            break;
                        }
                        mbar_expect_tx(hfull_bar(hstage), (uint32_t)(kR * (p.halo_swz ? BK / 16 : p.halo_planes)) * halo_bytes);
                        if (p.halo_swz) {
#pragma unroll
                            for (int t = 0; t < kR; ++t)
                                tma_load_4d(smem_u32(smem_a + hstage * Cfg::kStageA + t * Cfg::kTileA), &tmA, hfull_bar(hstage), gbase + cc * BK,
                                            w0[t] - p.pad_left, h0[t] - p.pad_top, n0[t]);
                        } else {
                            if (p.halo_row_map) {
                                // 16-byte pixels: a halo row is contiguous in memory, so the tile is halo_h long rows, not halo_w x halo_h short ones
#pragma unroll
                                for (int t = 0; t < kR; ++t)
                                    tma_load_4d(smem_u32(smem_a + hstage * Cfg::kStageA + t * Cfg::kTileA), &tmA, hfull_bar(hstage),
                                                16 * (w0[t] - p.pad_left), h0[t] - p.pad_top, n0[t], 0);
                            } else {
#pragma unroll
                                for (int t = 0; t < kR; ++t)
                                    for (int j = 0; j < p.halo_planes; ++j)
                                        tma_load_4d(smem_u32(smem_a + hstage * Cfg::kStageA + t * Cfg::kTileA + j * kHaloPlane), &tmA, hfull_bar(hstage),
                                                    gbase + cc * BK + j * 16, w0[t] - p.pad_left, h0[t] - p.pad_top, n0[t]);
                            }
                        }
                        if (++hstage == Cfg::kAStages) {
                            hstage = 0;
                            hphase ^= 1u;
                        }
                        for (int tap = 0; tap < taps; ++tap) {
                            if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status, 1, 0)) {
                                ok = false;
                                break;
                            }
                            mbar_expect_tx(full_bar(stage), Cfg::kStageB);
                            tma_load_2d(smem_u32(smem_b + stage * Cfg::kStageB), &tmB, full_bar(stage), tap * p.c_pad + cc * BK, ct * BN);
                            if (++stage == kStages) {
                                stage = 0;
                                phase ^= 1u;
                            }
                        }
                    }
                } else {
                    int bcol = 0;  // K offset in the packed weights: tap * c_pad + channel chunk
                    for (int kh = 0; kh < p.KH && ok; ++kh)
                        for (int kw = 0; kw < p.KW && ok; ++kw)
                            for (int cc = 0; cc < p.c_chunks; ++cc, bcol += BK) {
                                ok = __all_sync(0xffffffffu, mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status, 1, 0));
                                if (!ok) break;
                                if (is_a) {
                                    if (lane == 0) mbar_expect_tx(full_bar(stage), Cfg::kStageBytes);  // both operands' bytes
                                    __syncwarp();
                                    if (lane < kR)
                                        tma_load_4d(smem_u32(smem_a + stage * Cfg::kStageA + lane * 128 * BK), &tmA, full_bar(stage), gbase + cc * BK,
                                                    lw0 * p.sw - p.pad_left + kw, lh0 * p.sh - p.pad_top + kh, ln0);
                                } else {
                                    if (lane == 0) tma_load_2d(smem_u32(smem_b + stage * Cfg::kStageB), &tmB, full_bar(stage), bcol, ct * BN);
                                }
                                __syncwarp();
                                if (++stage == kStages) {
                                    stage = 0;
                                    phase ^= 1u;
                                }
                            }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            int stage = 0, hstage = 0;
            uint32_t phase = 0, hphase = 0;
            int it = 0;
            bool ok = true;
            // descriptor halves (see kmajor_desc_hi): stepping is one 32-bit add of a compile-time constant
            const uint32_t desc_hi = kmajor_desc_hi<BK>();
            const uint32_t a_lo0 = kmajor_desc_lo(smem_u32(smem_a)), b_lo0 = kmajor_desc_lo(smem_u32(smem_b));
            const int halo_w = p.halo_w;
            const uint32_t halo_hi = (uint32_t)halo_w | (1u << 14);                                          // SBO = one halo row, no swizzle
            const uint32_t halo_lo0 = (smem_u32(smem_a) >> 4) | ((uint32_t)p.halo_lbo << 16);             // LBO = one plane, or one pixel
            for (int grp = blockIdx.x; grp < total_groups && ok; grp += gridDim.x, ++it) {
                const int acc = it & 1;
                const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
                if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, p.status, 2, 0)) break;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)(acc * 256);
                if (HALO) {
                    for (int cc = 0; cc < p.c_chunks && ok; ++cc) {
                        if (!mbar_wait(hfull_bar(hstage), hphase, abort_flag, p.status, 10, 0)) {
                            ok = false;
                            break;
                        }
                        tc_fence_after();
                        const uint32_t ha_lo = halo_lo0 + (uint32_t)(hstage * (Cfg::kStageA >> 4));
                        for (int tap = 0; tap < taps; ++tap) {
                            const int kh = tap / p.KW, kw = tap - kh * p.KW;
                            if (!mbar_wait(full_bar(stage), phase, abort_flag, p.status, 3, 0)) {
                                ok = false;
                                break;
                            }
                            tc_fence_after();
                            const uint32_t b_lo = b_lo0 + (uint32_t)(stage * (Cfg::kStageB >> 4));
                            const uint32_t accum = (cc > 0 || tap > 0) ? 1u : 0u;
                            if (p.halo_swz) {
                                // one swizzled tile of BK-byte pixels: the view starts (kh, kw) pixels in; 8-row groups are one halo row apart
                                const uint32_t a_lo = a_lo0 + (uint32_t)(hstage * (Cfg::kStageA >> 4)) + (uint32_t)((kh * halo_w + kw) * (BK >> 4));
                                const uint32_t a_hi = (uint32_t)((halo_w * BK) >> 4) | (1u << 14) | ((BK == 128 ? 2u : 4u) << 29);
#pragma unroll
                                for (int k = 0; k < BK / 32; ++k)
#pragma unroll
                                    for (int t = 0; t < kR; ++t)
                                        umma_i8_lohi(tmem_d + (uint32_t)(t * BN), a_lo + (uint32_t)((t * Cfg::kTileA + k * 32) >> 4), a_hi, b_lo + k * 2,
                                                     desc_hi, p.idesc, k > 0 ? 1u : accum);
                            } else {
                                const uint32_t a_lo = ha_lo + (uint32_t)(kh * halo_w + kw);  // the tap's view starts (kh, kw) pixels of 16 bytes in
#pragma unroll
                                for (int k = 0; k < BK / 32; ++k)
#pragma unroll
                                    for (int t = 0; t < kR; ++t)
                                        umma_i8_lohi(tmem_d + (uint32_t)(t * BN), a_lo + (uint32_t)((t * Cfg::kTileA) >> 4) + (uint32_t)(k * p.halo_kstep), halo_hi,
                                                     b_lo + k * 2, desc_hi, p.idesc, k > 0 ? 1u : accum);
                            }
                            umma_commit(empty_bar(stage));
                            if (++stage == kStages) {
                                stage = 0;
                                phase ^= 1u;
                            }
                        }
                        if (ok) umma_commit(hempty_bar(hstage));  // the halo tiles are free once the MMAs of all taps have read them
                        if (++hstage == Cfg::kAStages) {
                            hstage = 0;
                            hphase ^= 1u;
                        }
                    }
                } else
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait(full_bar(stage), phase, abort_flag, p.status, 3, 0)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_lo = a_lo0 + (uint32_t)(stage * (Cfg::kStageA >> 4));
                    const uint32_t b_lo = b_lo0 + (uint32_t)(stage * (Cfg::kStageB >> 4));
                    const uint32_t accum = kb > 0 ? 1u : 0u;
#pragma unroll
                    for (int k = 0; k < BK / 32; ++k)
#pragma unroll
                        for (int t = 0; t < kR; ++t)
                            umma_i8_lohi(tmem_d + (uint32_t)(t * BN), a_lo + (uint32_t)((t * 128 * BK + k * 32) >> 4), desc_hi, b_lo + k * 2, desc_hi,
                                         p.idesc, k > 0 ? 1u : accum);
                    umma_commit(empty_bar(stage));  // frees the stage once these MMAs have read it
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (ok) umma_commit(tfull_bar(acc));  // all kR accumulators complete
            }
        }
    } else if (warp < 18) {
        // ---------------- epilogue warps ----------------
        // Warp w reads TMEM lanes 32*(w % 4) .. +31 (one output position per thread and tile); the four warps of a lane
        // quarter take every fourth 16-channel chunk.  A unit of work is (chunk, tile): 16 accumulators in, 16 bytes out.
        constexpr int kMine = BN / 64;  // chunks per warp
        constexpr int kUnits = kMine * kR;
        constexpr bool kFlat = NARROW > 0;
        constexpr int kV = NARROW > 0 ? NARROW : 1;
        const int e = warp - 2;         // 0..15
        const int quarter = warp & 3;
        const int sub = e >> 2;
        const int row = quarter * 32 + lane;
        float* s_mult = reinterpret_cast<float*>(smem + Cfg::kParamOffset) + e * (3 * BN / 4);
        uint32_t* s_add = reinterpret_cast<uint32_t*>(s_mult + BN / 4);
        uint32_t* s_corr = s_add + BN / 4;  // folded epilogue only: activation zero point x sum of the channel's weights
        const bool has_corr = kFold && p.col_corr != nullptr;
        int cached_ct = -1;
        const RequantParams rq = p.epi.rq;
        const float hi_ph = (float)(rq.clamp_hi_q >= 0 ? rq.clamp_hi_q : 255) + 0.5f;
        const float cy = kMagic23 + rq.y_zp_f, cr = kMagic23 + rq.res_zp_f;
        const float out_half = __fadd_rn(rq.out_zp_f, 0.5f);
        // Relu before the final quantization equals raising the lower clamp bound to the output zero point.
        const float res_lo = rq.res_relu ? out_half : 0.f;
        // Folded epilogue (fold_channel / residual_fold in qmath.cuh): values run in units of the output range, so the saturation of
        // one fused multiply-add is both clamps, and a second one, rounded toward minus infinity onto 2^23, leaves the integer in the
        // low mantissa bits.  No minimum / maximum and no conversion instruction besides the int -> float of the accumulator.
        const uint64_t magic23x2 = pack2(kMagic23, kMagic23);
        const uint64_t hp2 = pack2(hi_ph, hi_ph);
        const uint64_t c255x2 = pack2(255.5f, 255.5f);
        const uint64_t fr2 = pack2(rq.fold_r, rq.fold_r), fc2 = pack2(rq.fold_c, rq.fold_c);
        const float fa = rq.fold_a;
        int it = 0;
        for (int grp = blockIdx.x; grp < total_groups; grp += gridDim.x, ++it) {
            const int acc = it & 1;
            const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
            const int ct = grp % p.col_tiles;
            const int pg = grp / p.col_tiles;
            const int col0 = ct * BN;
            const int buf = it % Cfg::kBufs;

            if (ct != cached_ct) {
                __syncwarp();
                for (int j = lane; j < BN / 4; j += 32) {
                    const int c = col0 + (kFlat ? (sub % kV) : ((j >> 4) * 4 + sub)) * 16 + (j & 15);
                    float m = 0.f;
                    uint32_t add = 0u, corr = 0u;
                    if (c < p.cols) {
                        m = epi_mult(p.epi, c);
                        const int bias = p.epi.bias ? p.epi.bias[c] : 0;
                        if (kFold) {
                            const FoldCh fc = fold_channel(bias, __fdiv_rn(m, rq.y_scale), rq);
                            m = fc.ms;
                            add = __float_as_uint(fc.bs);
                            if (p.col_corr) corr = (uint32_t)p.col_scale * (uint32_t)p.col_corr[c];
                        } else {
                            add = (uint32_t)bias;
                            if (p.col_corr) add -= (uint32_t)p.col_scale * (uint32_t)p.col_corr[c];
                        }
                    }
                    s_mult[j] = m;
                    s_add[j] = add;
                    s_corr[j] = corr;
                }
                __syncwarp();
                cached_ct = ct;
            }

            // The buffer is ready when the store that last used it has read it (no residual) or when this group's residual
            // has landed in it (which the producer starts only after that store).
            uint8_t* out_buf = smem_out + buf * (kR * Cfg::kTileOut);
            const uint32_t use_phase = (uint32_t)(it / Cfg::kBufs) & 1u;
            bool got = RES ? mbar_wait(rfull_bar(buf), use_phase, abort_flag, p.status, 6, 32)
                           : mbar_wait(bempty_bar(buf), use_phase ^ 1u, abort_flag, p.status, 7, 32);
            if (got) got = mbar_wait(tfull_bar(acc), acc_phase, abort_flag, p.status, 4, 32);
            if (!__all_sync(0xffffffffu, got)) break;
            {
                tc_fence_after();
                const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * 256);
                // One unit: 16 accumulators of (chunk i, tile t) in registers -> 16 staged bytes.  The per-channel multiplier
                // and additive term come from the per-warp cache four channels at a time.
                auto process = [&](uint32_t (&r)[16], const int u) {
                    const int i = kFlat ? 0 : u / kR, t = kFlat ? (sub + 4 * u) / kV : u % kR;
                    const int ch = kFlat ? sub % kV : i * 4 + sub;
                    uint8_t* cell = out_buf + t * Cfg::kTileOut + staged_offset<BN>(row, ch);
                    uint4 resv = make_uint4(0u, 0u, 0u, 0u);
                    if (RES) resv = *reinterpret_cast<const uint4*>(cell);
                    const uint32_t resw[4] = {resv.x, resv.y, resv.z, resv.w};
                    const uint4* pm = reinterpret_cast<const uint4*>(s_mult + i * 16);
                    const uint4* pa = reinterpret_cast<const uint4*>(s_add + i * 16);
                    if (has_corr) {  // folded: the bias lives in the float offset, the activation zero-point term stays an integer
                        const uint4* pc = reinterpret_cast<const uint4*>(s_corr + i * 16);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const uint4 c4 = pc[j];
                            r[4 * j] -= c4.x; r[4 * j + 1] -= c4.y; r[4 * j + 2] -= c4.z; r[4 * j + 3] -= c4.w;
                        }
                    }
                    uint32_t outw[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint4 m4 = pm[j], a4 = pa[j];
                        const uint32_t mmw[4] = {m4.x, m4.y, m4.z, m4.w};
                        const uint32_t addw[4] = {a4.x, a4.y, a4.z, a4.w};
                        uint32_t fb[4];
                        if (kFold) {
#pragma unroll
                            for (int h = 0; h < 2; ++h) {
                                const int e0 = 2 * h;
                                float t0 = fma_sat((float)(int)r[4 * j + e0], __uint_as_float(mmw[e0]), __uint_as_float(addw[e0]));
                                float t1 = fma_sat((float)(int)r[4 * j + e0 + 1], __uint_as_float(mmw[e0 + 1]), __uint_as_float(addw[e0 + 1]));
                                uint64_t f2 = fma_rm_x2(pack2(t0, t1), hp2, magic23x2);                  // 2^23 + q
                                if (RES) {
                                    const uint64_t q2 = sub_x2(f2, magic23x2);                               // q, exact
                                    const uint64_t r2 = sub_x2(pack2(byte_to_magic(resw[j], 2 * h), byte_to_magic(resw[j], 2 * h + 1)), magic23x2);
                                    const uint64_t in2 = fma_x2(r2, fr2, fc2);
                                    t0 = fma_sat(lo_of(q2), fa, lo_of(in2));
                                    t1 = fma_sat(hi_of(q2), fa, hi_of(in2));
                                    f2 = fma_rm_x2(pack2(t0, t1), c255x2, magic23x2);
                                }
                                fb[2 * h] = (uint32_t)f2;
                                fb[2 * h + 1] = (uint32_t)(f2 >> 32);
                            }
                        } else {
#pragma unroll
                            for (int b = 0; b < 4; ++b) {
                                const float a = (float)(int)(r[4 * j + b] + addw[b]);
                                float tp = qdiv(__fmul_rn(a, __uint_as_float(mmw[b])), rq.y_div);
                                tp = __fadd_rn(__fadd_rn(tp, rq.y_zp_f), 0.5f);
                                fb[b] = __float_as_uint(quant_u8_up_magic(tp, hi_ph));
                            }
                            if (RES) {
#pragma unroll
                                for (int b = 0; b < 4; ++b) {
                                    const float u8v = __fsub_rn(__uint_as_float(fb[b]), cy);   // q - y_zp, exact
                                    const float w = __fsub_rn(byte_to_magic(resw[j], b), cr);   // r - res_zp, exact
                                    const float v = __fadd_rn(__fmul_rn(u8v, rq.y_scale), __fmul_rn(w, rq.res_scale));
                                    const float tp = __fadd_rn(__fadd_rn(qdiv(v, rq.out_div), rq.out_zp_f), 0.5f);
                                    fb[b] = __float_as_uint(__fadd_rd(fminf(fmaxf(tp, res_lo), 255.5f), kMagic23));
                                }
                            }
                        }
                        const uint32_t lo = __byte_perm(fb[0], fb[1], 0x0040), hi = __byte_perm(fb[2], fb[3], 0x0040);
                        outw[j] = __byte_perm(lo, hi, 0x5410);
                    }
                    *reinterpret_cast<uint4*>(cell) = make_uint4(outw[0], outw[1], outw[2], outw[3]);
                };
                auto unit_valid = [&](int u) {  // warp-uniform; columns beyond the operator's are clipped by the store
                    return kFlat ? (sub + 4 * u) / kV < kR : col0 + ((u / kR) * 4 + sub) * 16 < p.cols;
                };
                auto unit_taddr = [&](int u) {
                    return kFlat ? taddr + (uint32_t)(((sub + 4 * u) / kV) * BN + (sub % kV) * 16) : taddr + (uint32_t)((u % kR) * BN + ((u / kR) * 4 + sub) * 16);
                };
                // The TMEM read of unit u + 1 is in flight while unit u is processed.
                uint32_t ra[16], rb[16];
                __syncwarp();
                if (unit_valid(0)) tmem_ld_32x32b_x16(unit_taddr(0), ra);
#pragma unroll
                for (int u = 0; u < kUnits; ++u) {
                    const bool valid = unit_valid(u);
                    if (u & 1) {
                        if (valid) tmem_ld_wait16(rb);
                        if (u + 1 < kUnits && unit_valid(u + 1)) tmem_ld_32x32b_x16(unit_taddr(u + 1), ra);
                        if (valid) process(rb, u);
                    } else {
                        if (valid) tmem_ld_wait16(ra);
                        if (u + 1 < kUnits && unit_valid(u + 1)) tmem_ld_32x32b_x16(unit_taddr(u + 1), rb);
                        if (valid) process(ra, u);
                    }
                }
                // Hand the accumulators back and the staged tile over to the store warp.
                tc_fence_before();
                fence_async_smem();  // staged bytes become visible to the TMA store
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(tempty_bar(acc));
                    mbar_arrive(bfull_bar(buf));
                }
            }
            if (POOL) {
                // Once all sixteen warps have staged the group, each of the 16 x 32 lanes takes one (pooled position, 16 channels)
                // item of the 105 x 4 the group owns: nine 16-byte reads of the staged tiles, one 16-byte store.  Byte maxima are
                // kept as two words of 16-bit lanes (even bytes, odd bytes), the widest unsigned SIMD maximum the hardware has.
                // Positions outside the convolution's output do not take part (uint8: the maximum with 0).  (One dedicated warp
                // walking the group with a sliding window was three times slower than the whole kernel is now.)
                const bool staged = mbar_wait(bfull_bar(buf), use_phase, abort_flag, p.status, 8, 32);
                if (!__all_sync(0xffffffffu, staged)) break;
                const int q = e * 32 + lane;
                int gw0, gh0, gn;
                pool_group_origin(pg, gw0, gh0, gn);
                const int unit = q & 3, pos = q >> 2;
                const int pi = pos / PG::kW, pj = pos - pi * PG::kW;
                const int ph = (gh0 >> 1) + pi, pw = (gw0 >> 1) + pj;
                if (pos < PG::kW * PG::kH && ph < p.pool_ho && pw < p.pool_wo && col0 + unit * 16 < p.cols) {
                    uint32_t ev[4] = {0u, 0u, 0u, 0u}, od[4] = {0u, 0u, 0u, 0u};
#pragma unroll
                    for (int dr = 0; dr < 3; ++dr) {
                        const int lr = 2 * pi + dr;  // row inside the group
                        if (gh0 + lr >= p.Ho) continue;
#pragma unroll
                        for (int dc = 0; dc < 3; ++dc) {
                            const int lc = 2 * pj + dc;  // column inside the group
                            if (gw0 + lc >= p.Wo) continue;
                            const uint8_t* tile = out_buf + ((lr / PG::kTileH) * 2 + lc / PG::kTileW) * Cfg::kTileOut;
                            const uint4 v = *reinterpret_cast<const uint4*>(tile + staged_offset<BN>((lr % PG::kTileH) * PG::kTileW + lc % PG::kTileW, unit));
                            const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                ev[k] = __vmaxu2(ev[k], w4[k] & 0x00ff00ffu);
                                od[k] = __vmaxu2(od[k], (w4[k] >> 8) & 0x00ff00ffu);
                            }
                        }
                    }
                    uint8_t* dst = static_cast<uint8_t*>(p.y) + (((int64_t)gn * p.pool_ho + ph) * p.pool_wo + pw) * p.ldc + col0 + unit * 16;
                    *reinterpret_cast<uint4*>(dst) = make_uint4(ev[0] | (od[0] << 8), ev[1] | (od[1] << 8), ev[2] | (od[2] << 8), ev[3] | (od[3] << 8));
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(bempty_bar(buf));  // this warp has read what it needs of the buffer
            }
        }
    } else if (warp == 18) {
        // ---------------- store warp ----------------
        // One lane: waits until all sixteen epilogue warps have staged a group, issues its TMA stores, waits until they have
        // read the buffer and hands the buffer back (to the epilogue, or to the producer for the next residual tile).
        if (!POOL) {  // the pooling form stores nothing by TMA: the epilogue warps pool and write
            // the whole warp walks the loop; the kR tiles of a group leave through kR lanes of one instruction (see the producers)
            int it = 0;
            for (int grp = blockIdx.x; grp < total_groups; grp += gridDim.x, ++it) {
                const int ct = grp % p.col_tiles;
                const int pg = grp / p.col_tiles;
                const int buf = it % Cfg::kBufs;
                if (!__all_sync(0xffffffffu, mbar_wait(bfull_bar(buf), (uint32_t)(it / Cfg::kBufs) & 1u, abort_flag, p.status, 8, 0))) break;
                uint8_t* out_buf = smem_out + buf * (kR * Cfg::kTileOut);
                const int pt = pg * kR + lane;
                if (lane < kR && pt < pos_tiles) {
                    int w0, h0, n0;
                    tile_origin(pt, w0, h0, n0);
                    tma_store_4d(&tmY, smem_u32(out_buf + lane * Cfg::kTileOut), ct * BN, w0, h0, n0);
                    tma_store_commit();
                }
                tma_store_wait_read<0>();  // lanes without a store in flight pass at once
                __syncwarp();
                if (lane == 0) mbar_arrive(bempty_bar(buf));
            }
            tma_store_wait_all();
        }
    }

    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 2000000ull) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, Cfg::kTmemCols);
    }
}

// Launch with the programmatic-serialization attribute: the kernel may begin (up to its dependency wait) while the previous
// kernel in the stream drains.
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), int grid, int block, size_t smem, cudaStream_t s, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid, 1, 1);
    cfg.blockDim = dim3((unsigned)block, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

template <int BN, int BK, int EPI, bool RES, bool HALO, bool POOL = false, int NARROW = 0>
int launch_one2(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmY, const CUtensorMap& tmR, const TcParams& p, int grid,
                cudaStream_t s) {
    using Cfg = Tc2Config<BN, BK, RES, HALO>;
    static_assert(Cfg::kUsable, "grouped kernel: not enough shared memory for two stages");
    static std::atomic<bool> attr_set[64] = {};  // per device; host threads may race here, every writer stores true
    int dev = 0;
    CHXQ_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !attr_set[dev].load(std::memory_order_acquire)) {
        CHXQ_CUDA(cudaFuncSetAttribute(tc_igemm2_kernel<BN, BK, EPI, RES, HALO, POOL, NARROW>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
        if (dev >= 0 && dev < 64) attr_set[dev].store(true, std::memory_order_release);
    }
    CHXQ_CUDA(launch_pdl(tc_igemm2_kernel<BN, BK, EPI, RES, HALO, POOL, NARROW>, grid, 640, Cfg::kSmemBytes, s, tmA, tmB, tmY, tmR, p));
    count_launch(1);
    return CHXQ_OK;
}

// Launches the grouped kernel for (bn, BK, epi, residual, halo); CHXQ_ERR_UNSUPPORTED when the combination has no
// instantiation.
template <int BK>
int launch_bk2(int bn, int epi, bool res, bool halo, const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmY,
               const CUtensorMap& tmR, const TcParams& p, int grid, cudaStream_t s) {
    const int key = (bn == 128 ? 4 : 0) + (epi == kEpiKU8Fold ? 2 : 0) + (res ? 1 : 0);
    if (halo) {
        if constexpr (BK == 128) {
            // 128-byte K tiles: one swizzled halo tile per position tile; 128-channel blocks without a residual only (shared memory)
            switch (key) {
                case 4: return launch_one2<128, BK, kEpiKU8, false, true>(tmA, tmB, tmY, tmR, p, grid, s);
                case 6: return launch_one2<128, BK, kEpiKU8Fold, false, true>(tmA, tmB, tmY, tmR, p, grid, s);
            }
        }
        if constexpr (BK == 64) {
            switch (key) {
                case 0: return launch_one2<64, BK, kEpiKU8, false, true>(tmA, tmB, tmY, tmR, p, grid, s);
                case 1: return launch_one2<64, BK, kEpiKU8, true, true>(tmA, tmB, tmY, tmR, p, grid, s);
                case 2: return launch_one2<64, BK, kEpiKU8Fold, false, true>(tmA, tmB, tmY, tmR, p, grid, s);
                case 3: return launch_one2<64, BK, kEpiKU8Fold, true, true>(tmA, tmB, tmY, tmR, p, grid, s);
                case 4: return launch_one2<128, BK, kEpiKU8, false, true>(tmA, tmB, tmY, tmR, p, grid, s);
                case 5: return launch_one2<128, BK, kEpiKU8, true, true>(tmA, tmB, tmY, tmR, p, grid, s);
                case 6: return launch_one2<128, BK, kEpiKU8Fold, false, true>(tmA, tmB, tmY, tmR, p, grid, s);
                case 7: return launch_one2<128, BK, kEpiKU8Fold, true, true>(tmA, tmB, tmY, tmR, p, grid, s);
            }
        }
        return CHXQ_ERR_UNSUPPORTED;
    }
    if (bn == 64 && epi == kEpiKU8Fold && p.col_tiles == 1 && p.cols <= 32) {  // narrow operators (MobileNetV2's projections)
        if (p.cols <= 16)
            return res ? launch_one2<64, BK, kEpiKU8Fold, true, false, false, 1>(tmA, tmB, tmY, tmR, p, grid, s)
                       : launch_one2<64, BK, kEpiKU8Fold, false, false, false, 1>(tmA, tmB, tmY, tmR, p, grid, s);
        return res ? launch_one2<64, BK, kEpiKU8Fold, true, false, false, 2>(tmA, tmB, tmY, tmR, p, grid, s)
                   : launch_one2<64, BK, kEpiKU8Fold, false, false, false, 2>(tmA, tmB, tmY, tmR, p, grid, s);
    }
    switch (key) {
        case 0: return launch_one2<64, BK, kEpiKU8, false, false>(tmA, tmB, tmY, tmR, p, grid, s);
        case 1: return launch_one2<64, BK, kEpiKU8, true, false>(tmA, tmB, tmY, tmR, p, grid, s);
        case 2: return launch_one2<64, BK, kEpiKU8Fold, false, false>(tmA, tmB, tmY, tmR, p, grid, s);
        case 3: return launch_one2<64, BK, kEpiKU8Fold, true, false>(tmA, tmB, tmY, tmR, p, grid, s);
        case 4: return launch_one2<128, BK, kEpiKU8, false, false>(tmA, tmB, tmY, tmR, p, grid, s);
        case 5: return launch_one2<128, BK, kEpiKU8, true, false>(tmA, tmB, tmY, tmR, p, grid, s);
        case 6: return launch_one2<128, BK, kEpiKU8Fold, false, false>(tmA, tmB, tmY, tmR, p, grid, s);
        case 7: return launch_one2<128, BK, kEpiKU8Fold, true, false>(tmA, tmB, tmY, tmR, p, grid, s);
    }
    return CHXQ_ERR_UNSUPPORTED;
}

}  // namespace tc
}  // namespace chxq
