// CTA-pair variant of the grouped-tile tcgen05 implicit-GEMM kernel (device code; the host side is in tc_igemm.cu): two CTAs
// on neighbouring SMs (a cluster of two) compute a 256-position x 256-channel block with tcgen05.mma.cta_group::2.
//
// Why: a one-CTA int8 tile of N = 128 reads 128 operand bytes out of shared memory per tensor-pipe clock -- all the shared
// memory can deliver -- while TMA writes the next stage into the same memory.  In a CTA pair each SM stages its own 128
// positions of A and only HALF of the 256-channel weight block; the pair's MMA reads both halves, so per SM and clock the
// tensor pipe reads 64 bytes and TMA writes 64: the main loop fits the shared-memory bandwidth.
//
// Roles per CTA are those of tc_kernel2.cuh plus a second producer (20 warps): warp 0 TMA producer of the positions, warp 19 TMA
// producer of the weights, warp 1 TMEM allocation and (in the pair's first CTA only) the MMA issuer, warps 2-17 epilogue, warp 18
// TMA stores.  What crosses the pair:
//   * every operand load of both CTAs signals the FIRST CTA's "stage full" barrier (cp.async.bulk.tensor with
//     .cta_group::2; no cluster multicast anywhere: each CTA fetches its own bytes);
//   * the first CTA's tcgen05.commit arrives on the "stage empty" and "accumulator full" barriers of BOTH CTAs;
//   * the epilogue warps of both CTAs arrive on the first CTA's "accumulator empty" barrier.
// Accumulators (128 lanes x 256 columns per CTA, double-buffered: 512 TMEM columns), the staging tiles, the residual loads
// and the output stores are local to each CTA.  Every wait is bounded as in tc_kernel.cuh; a CTA whose wait expires raises
// its abort flag, and its partner's waits then expire in turn; both meet at the cluster barrier in front of the teardown.
#pragma once

#include "tc_kernel2.cuh"

namespace chxq {
namespace tc {

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

// Address of the same shared-memory offset in CTA `rank` of the cluster (a shared::cluster address).
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}

__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Arrival on a barrier that may live in the partner CTA.  Default semantics (release at CTA scope): what the arrival orders here
// are tensor-memory reads, which tcgen05.fence::before_thread_sync covers; a cluster-scope release would cost a memory barrier
// per warp and item.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// Operand loads of a CTA pair: the bytes land in the executing CTA's shared memory, the completion is counted on `bar`, which
// may live in either CTA of the pair (here always the first CTA's).
__device__ __forceinline__ void tma_load_4d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2, int c3) {
    asm volatile(
            "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
            ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
            : "memory");
}

__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
    asm volatile(
            "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
            ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1)
            : "memory");
}

__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}

__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// D[tmem of both CTAs] (+)= A * B over the pair: M = 256 (128 rows per CTA), the N rows of B split between the CTAs.
__device__ __forceinline__ void umma_i8_pair(uint32_t tmem_d, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                             uint32_t accumulate) {
    asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            ".reg .b64 da, db;\n\t"
            "mov.b64 da, {%1, %2};\n\t"
            "mov.b64 db, {%3, %4};\n\t"
            "setp.ne.b32 p, %6, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::i8 [%0], da, db, %5, p;\n\t"
            "}\n" ::"r"(tmem_d),
            "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
            : "memory");
}

// Arrives, once every tcgen05 operation issued so far by this thread has completed, on the barrier at this shared-memory
// offset in every CTA of `cta_mask`.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar, uint16_t cta_mask) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar), "h"(cta_mask)
                 : "memory");
}

constexpr int kPairBN = 256;  // channels of a pair's block

template <int BK, bool RES, bool I32 = false>
struct Tc3Config {
    static constexpr int kTileA = 128 * BK;              // this CTA's 128 positions
    static constexpr int kHalfB = 128 * BK;              // this CTA's half of the 256 weight rows
    static constexpr int kStageBytes = kTileA + kHalfB;
    static constexpr int kHalfOut = 128 * 128;           // one swizzled [128 positions][128 channels] half of the staged output
    static constexpr int kTileOut = 2 * kHalfOut;
    static constexpr int kBufs = I32 ? 0 : (RES ? 3 : 2);  // as in tc_kernel2.cuh; int32 accumulators leave straight from registers
    static constexpr int kOutBytes = kBufs * kTileOut;
    static constexpr int kBudget = 208 * 1024;
    static constexpr int kStagesRaw = (kBudget - kOutBytes) / kStageBytes;
    static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
    static constexpr int kTmemCols = 512;
    // barriers: full[kStages], empty[kStages], tmem_full[2], tmem_empty[2], res_full[3], buf_empty[3], buf_full[3]
    static constexpr int kNumBars = 2 * kStages + 13;
    static constexpr int kBarOffset = kStages * kStageBytes + kOutBytes;
    static constexpr int kParamOffset = ((kBarOffset + kNumBars * 8 + 16 + 15) / 16) * 16;
    static constexpr int kParamBytes = 16 * (3 * kPairBN / 4) * 4;  // 16 warps x 64 channels x (multiplier, additive term, zero-point term)
    static constexpr int kSmemBytes = 1024 /*alignment slack*/ + kParamOffset + kParamBytes;
    static_assert(kStages >= 2, "CTA-pair kernel: not enough shared memory for two stages");
    static_assert(kSmemBytes <= 227 * 1024, "CTA-pair kernel: shared memory over the per-CTA limit");
};

template <int BK, int EPI, bool RES>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(640, 1)
tc_igemm3_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmY,
                 const __grid_constant__ CUtensorMap tmR, const TcParams p) {
    constexpr bool kInt32 = EPI == kEpiKInt32;  // MatMulInteger / ConvInteger: the exact accumulator (minus the zero-point terms)
    using Cfg = Tc3Config<BK, RES, kInt32>;
    constexpr int kStages = Cfg::kStages;
    constexpr int BN = kPairBN;
    constexpr bool kFold = EPI == kEpiKU8Fold;
    static_assert(!(kInt32 && RES), "int32 outputs have no residual tail");
    constexpr int kBufsDiv = Cfg::kBufs > 0 ? Cfg::kBufs : 1;  // divisor that stays valid where the staging ring does not exist
    extern __shared__ uint8_t smem_raw[];
    // The dynamic shared-memory window starts at the same address in both CTAs of a pair (same kernel, same static usage), so
    // the aligned offsets below are the same in both: descriptors and barrier offsets of the first CTA are valid in the second.
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + kStages * Cfg::kTileA;
    uint8_t* smem_out = smem_b + kStages * Cfg::kHalfB;  // [kBufs][2 halves][128][128], 1024-byte aligned
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kBarOffset);
    uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(bars + Cfg::kNumBars);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

    const uint32_t bar_base = smem_u32(bars);
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * kStages + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * kStages + 2 + a); };
    auto rfull_bar = [&](int b) { return bar_base + 8u * (2 * kStages + 4 + b); };
    auto bempty_bar = [&](int b) { return bar_base + 8u * (2 * kStages + 7 + b); };
    auto bfull_bar = [&](int b) { return bar_base + 8u * (2 * kStages + 10 + b); };

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();  // 0: the CTA that issues the pair's MMAs

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full_bar(s), 1);   // first CTA only: its producer's arrive.expect_tx for both CTAs' bytes
            mbar_init(empty_bar(s), 1);  // one commit arrival per CTA
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), 32);  // first CTA only: sixteen epilogue warps of each CTA
        }
        for (int b = 0; b < 3; ++b) {
            mbar_init(rfull_bar(b), 1);
            mbar_init(bempty_bar(b), 1);
            mbar_init(bfull_bar(b), 16);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc_pair(smem_u32(tmem_ptr_smem), Cfg::kTmemCols);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // the partner's barriers are initialised before anything of this CTA can signal them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr_smem;
    pdl_launch_dependents();  // the next kernel's CTAs may take this SM as soon as this CTA leaves it
    pdl_dependency_wait();    // from here on the previous kernel's output (this kernel's input) is complete and visible

    const int pos_tiles = p.tiles_w * p.tiles_h * p.tiles_n;
    const int pos_pairs = (pos_tiles + 1) / 2;
    const int total_items = pos_pairs * p.col_tiles;
    const int num_pairs_launched = (int)(gridDim.x >> 1);
    const int first_item = (int)(blockIdx.x >> 1);
    const int taps = p.KH * p.KW;
    const int num_kb = taps * p.c_chunks;

    // Output coordinates of position tile `pt` (a tile past the end lands beyond the last image: loads fill zero, its store is skipped).
    auto tile_origin = [&](int pt, int& w0, int& h0, int& n0) {
        const int tw = pt % p.tiles_w;
        pt /= p.tiles_w;
        const int th = pt % p.tiles_h;
        const int tn = pt / p.tiles_h;
        w0 = tw * p.Wb; h0 = th * p.Hb; n0 = tn * p.Nb;
    };

    if (warp == 0 || warp == 19) {
        // ---------------- TMA producers (both CTAs): warp 0 loads this CTA's positions (and the residual tile), warp 19 its half
        // of the weights.  One thread per operand, because a thread that issues a tensor copy is held until the copy engine
        // takes it: with one thread for both operands the engine idles while that thread waits for the next free stage.
        if (lane == 0) {
            const bool is_a = warp == 0;
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            int it = 0;
            const uint32_t lead_full0 = map_to_cta(full_bar(0), 0);  // the first CTA's "stage full" barriers
#ifdef CHXQ_TL
            int tlk = 0;
            long long* tlp = p.tl ? p.tl + (is_a ? 0 : 2 * 2048 + 1024) : nullptr;
            const int tlmax = is_a ? 512 : 256;
#endif
            for (int item = first_item; item < total_items && ok; item += num_pairs_launched, ++it) {
                const int ct = item % p.col_tiles;
                const int pt = (item / p.col_tiles) * 2 + (int)rank;
                int w0, h0, n0;
                tile_origin(pt, w0, h0, n0);
                if (RES && is_a) {
                    const int rb = it % kBufsDiv;
                    if (!mbar_wait(bempty_bar(rb), ((uint32_t)(it / kBufsDiv) & 1u) ^ 1u, abort_flag, p.status, 5, 0)) break;
                    mbar_expect_tx(rfull_bar(rb), Cfg::kTileOut);
#pragma unroll
                    for (int hf = 0; hf < 2; ++hf)
                        tma_load_4d(smem_u32(smem_out + rb * Cfg::kTileOut + hf * Cfg::kHalfOut), &tmR, rfull_bar(rb), ct * BN + hf * 128, w0, h0, n0);
                }
                const int wi0 = w0 * p.sw - p.pad_left, hi0 = h0 * p.sh - p.pad_top;
                const int brow = ct * BN + (int)rank * 128;
                int bcol = 0;  // K offset in the packed weights: tap * c_pad + channel chunk
                for (int kh = 0; kh < p.KH && ok; ++kh)
                    for (int kw = 0; kw < p.KW && ok; ++kw, bcol += p.c_pad - p.c_chunks * BK)
                        for (int cc = 0; cc < p.c_chunks; ++cc, bcol += BK) {
#ifdef CHXQ_TL
                            const long long tl0 = clock64();
#endif
                            if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status, 1, 0)) {
                                ok = false;
                                break;
                            }
#ifdef CHXQ_TL
                            const long long tl1 = clock64();
#endif
                            const uint32_t fb = lead_full0 + 8u * stage;
                            if (is_a) {
                                if (rank == 0) mbar_expect_tx(full_bar(stage), 2 * Cfg::kStageBytes);  // both CTAs' operand bytes of this stage
                                tma_load_4d_pair(smem_u32(smem_a + stage * Cfg::kTileA), &tmA, fb, cc * BK, wi0 + kw, hi0 + kh, n0);
                            } else {
                                tma_load_2d_pair(smem_u32(smem_b + stage * Cfg::kHalfB), &tmB, fb, bcol, brow);
                            }
#ifdef CHXQ_TL
                            if (tlp && blockIdx.x == 0 && tlk < tlmax) {
                                tlp[tlk * 4 + 0] = tl0; tlp[tlk * 4 + 1] = tl1; tlp[tlk * 4 + 2] = clock64(); tlp[tlk * 4 + 3] = item;
                                ++tlk;
                            }
#endif
                            if (++stage == kStages) {
                                stage = 0;
                                phase ^= 1u;
                            }
                        }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (first CTA of the pair) ----------------
        if (lane == 0 && rank == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int it = 0;
            bool ok = true;
            const uint32_t desc_hi = kmajor_desc_hi<BK>();
            const uint32_t a_lo0 = kmajor_desc_lo(smem_u32(smem_a)), b_lo0 = kmajor_desc_lo(smem_u32(smem_b));
#ifdef CHXQ_TL
            int tlk = 0;
#endif
            for (int item = first_item; item < total_items && ok; item += num_pairs_launched, ++it) {
                const int acc = it & 1;
                const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
#ifdef CHXQ_TL
                const long long tle0 = clock64();
#endif
                if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, p.status, 2, 0)) break;
#ifdef CHXQ_TL
                if (p.tl && blockIdx.x == 0 && it < 64) { p.tl[2 * 2048 + it * 4] = tle0; p.tl[2 * 2048 + it * 4 + 1] = clock64(); }
#endif
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)(acc * BN);
                for (int kb = 0; kb < num_kb; ++kb) {
#ifdef CHXQ_TL
                    const long long tl0 = clock64();
#endif
                    if (!mbar_wait(full_bar(stage), phase, abort_flag, p.status, 3, 0)) {
                        ok = false;
                        break;
                    }
#ifdef CHXQ_TL
                    const long long tl1 = clock64();
#endif
                    tc_fence_after();
                    const uint32_t a_lo = a_lo0 + (uint32_t)(stage * (Cfg::kTileA >> 4));
                    const uint32_t b_lo = b_lo0 + (uint32_t)(stage * (Cfg::kHalfB >> 4));
#pragma unroll
                    for (int k = 0; k < BK / 32; ++k)
                        umma_i8_pair(tmem_d, a_lo + (uint32_t)(k * 2), desc_hi, b_lo + (uint32_t)(k * 2), desc_hi, p.idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    umma_commit_pair(empty_bar(stage), 3);  // frees the stage in both CTAs once these MMAs have read it
#ifdef CHXQ_TL
                    if (p.tl && blockIdx.x == 0 && tlk < 512) {
                        p.tl[2048 + tlk * 4 + 0] = tl0; p.tl[2048 + tlk * 4 + 1] = tl1; p.tl[2048 + tlk * 4 + 2] = clock64(); p.tl[2048 + tlk * 4 + 3] = item;
                        ++tlk;
                    }
#endif
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (ok) umma_commit_pair(tfull_bar(acc), 3);  // both CTAs' accumulators complete
            }
        }
    } else if (warp < 18) {
        // ---------------- epilogue warps (both CTAs, each on its own 128 positions) ----------------
        constexpr int kUnits = BN / 64;  // 16-channel chunks per warp: chunk i * 4 + sub for i = 0 .. 3
        const int e = warp - 2;          // 0..15
        const int quarter = warp & 3;
        const int sub = e >> 2;
        const int row = quarter * 32 + lane;
        float* s_mult = reinterpret_cast<float*>(smem + Cfg::kParamOffset) + e * (3 * BN / 4);
        uint32_t* s_add = reinterpret_cast<uint32_t*>(s_mult + BN / 4);
        uint32_t* s_corr = s_add + BN / 4;
        const bool has_corr = kFold && p.col_corr != nullptr;
        int cached_ct = -1;
        const RequantParams rq = p.epi.rq;
        const float hi_ph = (float)(rq.clamp_hi_q >= 0 ? rq.clamp_hi_q : 255) + 0.5f;
        const float cy = kMagic23 + rq.y_zp_f, cr = kMagic23 + rq.res_zp_f;
        const float out_half = __fadd_rn(rq.out_zp_f, 0.5f);
        const float res_lo = rq.res_relu ? out_half : 0.f;
        const uint64_t magic23x2 = pack2(kMagic23, kMagic23);
        const uint64_t hp2 = pack2(hi_ph, hi_ph);
        const uint64_t c255x2 = pack2(255.5f, 255.5f);
        const uint64_t fr2 = pack2(rq.fold_r, rq.fold_r), fc2 = pack2(rq.fold_c, rq.fold_c);
        const float fa = rq.fold_a;
        const uint32_t lead_tempty0 = map_to_cta(tempty_bar(0), 0);
        int it = 0;
        for (int item = first_item; item < total_items; item += num_pairs_launched, ++it) {
            const int acc = it & 1;
            const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
            const int ct = item % p.col_tiles;
            const int col0 = ct * BN;
            const int buf = it % kBufsDiv;

            if (ct != cached_ct) {
                __syncwarp();
                for (int j = lane; j < BN / 4; j += 32) {
                    const int c = col0 + ((j >> 4) * 4 + sub) * 16 + (j & 15);
                    float m = 0.f;
                    uint32_t add = 0u, corr = 0u;
                    if (c < p.cols && kInt32) {
                        if (p.col_corr) add = 0u - (uint32_t)p.col_scale * (uint32_t)p.col_corr[c];  // activation zero point x sum of the column's weights
                        if (p.col_mul) corr = (uint32_t)p.col_mul[c];                                   // the column's weight zero point
                    } else if (c < p.cols) {
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

            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BN);
            if constexpr (kInt32) {
                // int32 outputs: every thread owns one output position (row) and writes its sixteen accumulators of a chunk as 64
                // contiguous bytes, straight from registers.
                const int pt = (item / p.col_tiles) * 2 + (int)rank;
                int w0, h0, n0;
                tile_origin(pt, w0, h0, n0);
                const int w_l = row % p.Wb, h_l = (row / p.Wb) % p.Hb, n_l = row / (p.Wb * p.Hb);
                const int wo = w0 + w_l, ho = h0 + h_l, no = n0 + n_l;
                const bool row_ok = pt < pos_tiles && wo < p.Wo && ho < p.Ho && no < p.No;
                const int64_t pos = ((int64_t)no * p.Ho + ho) * p.Wo + wo;
                const uint32_t rowc = (p.row_corr && row_ok) ? (uint32_t)p.row_corr[pos] : 0u;  // sum over the row of (a - za), for the weight zero points
                const bool got = mbar_wait(tfull_bar(acc), acc_phase, abort_flag, p.status, 4, 32);
                if (!__all_sync(0xffffffffu, got)) break;
                tc_fence_after();
#pragma unroll
                for (int i = 0; i < BN / 64; ++i) {
                    const int cbase = col0 + (i * 4 + sub) * 16;
                    if (cbase >= p.cols) continue;  // warp-uniform
                    uint32_t r[16];
                    __syncwarp();
                    tmem_ld_32x32b_x16(taddr + (uint32_t)((i * 4 + sub) * 16), r);
                    tmem_ld_wait16(r);
                    const uint4* pa = reinterpret_cast<const uint4*>(s_add + i * 16);
                    const uint4* pc = reinterpret_cast<const uint4*>(s_corr + i * 16);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint4 a4 = pa[j], c4 = pc[j];
                        r[4 * j] += a4.x - c4.x * rowc; r[4 * j + 1] += a4.y - c4.y * rowc;
                        r[4 * j + 2] += a4.z - c4.z * rowc; r[4 * j + 3] += a4.w - c4.w * rowc;
                    }
                    if (!row_ok) continue;
                    int32_t* yo = static_cast<int32_t*>(p.y) + pos * p.ldc + cbase;
                    if (p.vec_ok && cbase + 16 <= p.cols) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) reinterpret_cast<uint4*>(yo)[j] = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (cbase + j < p.cols) yo[j] = (int32_t)r[j];
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(lead_tempty0 + 8u * acc);
                continue;
            }
            uint8_t* out_buf = smem_out + buf * Cfg::kTileOut;
            const uint32_t use_phase = (uint32_t)(it / kBufsDiv) & 1u;
            bool got = RES ? mbar_wait(rfull_bar(buf), use_phase, abort_flag, p.status, 6, 32)
                           : mbar_wait(bempty_bar(buf), use_phase ^ 1u, abort_flag, p.status, 7, 32);
            if (got) got = mbar_wait(tfull_bar(acc), acc_phase, abort_flag, p.status, 4, 32);
            if (!__all_sync(0xffffffffu, got)) break;
            tc_fence_after();
            // One unit: 16 accumulators of chunk ch in registers -> 16 staged bytes (half ch / 8 of the staged tile, 16-byte unit ch % 8).
            auto process = [&](uint32_t (&r)[16], const int i) {
                const int ch = i * 4 + sub;
                uint8_t* cell = out_buf + (ch >> 3) * Cfg::kHalfOut + staged_offset<128>(row, ch & 7);
                uint4 resv = make_uint4(0u, 0u, 0u, 0u);
                if (RES) resv = *reinterpret_cast<const uint4*>(cell);
                const uint32_t resw[4] = {resv.x, resv.y, resv.z, resv.w};
                const uint4* pm = reinterpret_cast<const uint4*>(s_mult + i * 16);
                const uint4* pa = reinterpret_cast<const uint4*>(s_add + i * 16);
                if (has_corr) {
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
                            uint64_t f2 = fma_rm_x2(pack2(t0, t1), hp2, magic23x2);  // 2^23 + q
                            if (RES) {
                                const uint64_t q2 = sub_x2(f2, magic23x2);
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
                                const float u8v = __fsub_rn(__uint_as_float(fb[b]), cy);
                                const float w = __fsub_rn(byte_to_magic(resw[j], b), cr);
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
            auto unit_valid = [&](int i) { return col0 + (i * 4 + sub) * 16 < p.cols; };  // warp-uniform; beyond: clipped by the store
            auto unit_taddr = [&](int i) { return taddr + (uint32_t)((i * 4 + sub) * 16); };
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
            // Hand the accumulators back to the pair's MMA issuer (in the first CTA) and the staged tile over to this CTA's store warp.
            tc_fence_before();
            fence_async_smem();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive_cluster(lead_tempty0 + 8u * acc);
                mbar_arrive(bfull_bar(buf));
            }
        }
    } else if (warp == 18) {
        // ---------------- store warp (both CTAs; idle for int32 outputs) ----------------
        if (lane == 0 && !kInt32) {
            int it = 0;
            for (int item = first_item; item < total_items; item += num_pairs_launched, ++it) {
                const int ct = item % p.col_tiles;
                const int pt = (item / p.col_tiles) * 2 + (int)rank;
                const int buf = it % kBufsDiv;
                if (!mbar_wait(bfull_bar(buf), (uint32_t)(it / kBufsDiv) & 1u, abort_flag, p.status, 8, 0)) break;
                uint8_t* out_buf = smem_out + buf * Cfg::kTileOut;
                if (pt < pos_tiles) {
                    int w0, h0, n0;
                    tile_origin(pt, w0, h0, n0);
#pragma unroll
                    for (int hf = 0; hf < 2; ++hf)
                        if (ct * BN + hf * 128 < p.cols) tma_store_4d(&tmY, smem_u32(out_buf + hf * Cfg::kHalfOut), ct * BN + hf * 128, w0, h0, n0);
                }
                tma_store_commit();
                tma_store_wait_read<0>();
                mbar_arrive(bempty_bar(buf));
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
    cluster_sync_all();  // neither CTA frees tensor memory or leaves while its partner may still signal or read it
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, Cfg::kTmemCols);
    }
}

// Number of CTA pairs of this instantiation that the current device keeps resident at once (also sets the kernel's
// shared-memory attribute); asked once per device.
template <int BK, int EPI, bool RES>
int pair_slots(int* out) {
    using Cfg = Tc3Config<BK, RES, EPI == kEpiKInt32>;
    static std::atomic<int> max_pairs[64] = {};
    int dev = 0;
    CHXQ_CUDA(cudaGetDevice(&dev));
    int pairs = (dev >= 0 && dev < 64) ? max_pairs[dev].load(std::memory_order_acquire) : 0;
    if (pairs == 0) {
        CHXQ_CUDA(cudaFuncSetAttribute(tc_igemm3_kernel<BK, EPI, RES>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
        int sms = 0;
        CHXQ_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)(sms & ~1), 1, 1);
        cfg.blockDim = dim3(640, 1, 1);
        cfg.dynamicSmemBytes = Cfg::kSmemBytes;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeClusterDimension;
        at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
        cfg.attrs = at;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, tc_igemm3_kernel<BK, EPI, RES>, &cfg) != cudaSuccess || n <= 0) {
            cudaGetLastError();
            n = sms / 2;
        }
        pairs = n < sms / 2 ? n : sms / 2;
        if (pairs <= 0) return set_error(CHXQ_ERR_CUDA, "CTA-pair kernel: no resident cluster fits on this device");
        if (dev >= 0 && dev < 64) max_pairs[dev].store(pairs, std::memory_order_release);
    }
    *out = pairs;
    return CHXQ_OK;
}

template <int BK, int EPI, bool RES>
int launch_one3(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmY, const CUtensorMap& tmR, const TcParams& p, int items,
                cudaStream_t s) {
    using Cfg = Tc3Config<BK, RES, EPI == kEpiKInt32>;
    int pairs = 0;
    const int rc = pair_slots<BK, EPI, RES>(&pairs);
    if (rc != CHXQ_OK) return rc;
    const int launch_pairs = items < pairs ? items : pairs;
    CHXQ_CUDA(launch_pdl(tc_igemm3_kernel<BK, EPI, RES>, 2 * launch_pairs, 640, Cfg::kSmemBytes, s, tmA, tmB, tmY, tmR, p));
    count_launch(1);
    return CHXQ_OK;
}

// Launches the CTA-pair kernel for (epi, residual) with a 128-byte K tile; CHXQ_ERR_UNSUPPORTED when the combination has no
// instantiation.
template <int BK>
int launch_bk3(int epi, bool res, const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmY, const CUtensorMap& tmR, const TcParams& p,
               int items, cudaStream_t s) {
    if (epi == kEpiKInt32) return res ? CHXQ_ERR_UNSUPPORTED : launch_one3<BK, kEpiKInt32, false>(tmA, tmB, tmY, tmR, p, items, s);
    const int key = (epi == kEpiKU8Fold ? 2 : 0) + (res ? 1 : 0);
    switch (key) {
        case 0: return launch_one3<BK, kEpiKU8, false>(tmA, tmB, tmY, tmR, p, items, s);
        case 1: return launch_one3<BK, kEpiKU8, true>(tmA, tmB, tmY, tmR, p, items, s);
        case 2: return launch_one3<BK, kEpiKU8Fold, false>(tmA, tmB, tmY, tmR, p, items, s);
        case 3: return launch_one3<BK, kEpiKU8Fold, true>(tmA, tmB, tmY, tmR, p, items, s);
    }
    return CHXQ_ERR_UNSUPPORTED;
}

}  // namespace tc
}  // namespace chxq
