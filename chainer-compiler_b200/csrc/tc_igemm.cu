// tcgen05 implicit-GEMM kernel for sm_100a: u8/s8 x u8/s8 -> s32 in TMEM (kind::i8), operands staged
// in shared memory by TMA (no cluster multicast anywhere), zero-point terms, per-channel requantize,
// bias, ReLU clamp and the residual tail applied in the epilogue straight out of TMEM.
//
// One persistent CTA per SM, 320 threads:
//   warp 0      : TMA producer (one elected lane): A box {bk, Wb, Hb, Nb} of an NHWC map / matrix,
//                 B box {bk, BN} of the packed weights, ring of kStages shared-memory stages.
//   warp 1      : allocates TMEM, issues tcgen05.mma (one elected lane), M = 128, N = BN, K = 32 per
//                 instruction; accumulators are double-buffered in TMEM (2 x BN columns) so the
//                 epilogue of tile i overlaps the main loop of tile i + 1.
//   warps 2..9  : epilogue; warp w may read TMEM lanes 32*(w % 4) .. +31 (one output position per thread), two
//                 warps per lane quarter split the 32-column chunks; each reads a chunk per tcgen05.ld (the next
//                 chunk's read overlapping this chunk's arithmetic), applies the epilogue from per-warp cached
//                 per-channel parameters and stores 128-bit vectors.
//
// Every mbarrier wait is bounded: after ~2 s without progress the waiting thread raises the CTA's
// abort flag and the device status word, every role leaves its loop, the CTA waits a bounded time
// for copies in flight, frees its TMEM and returns.  Nothing traps.
#include <cuda.h>

#include <mutex>
#include <vector>

#include "common.h"
#include "kernels.h"

namespace chxq {
namespace {

// ------------------------------------------------------------------------------------------
// PTX wrappers
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t"
            "}\n"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
    return ok;
}

__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

constexpr uint64_t kWaitLimitNs = 2000000000ull;  // 2 s

// Bounded wait.  Returns false when the CTA is aborting (either this wait expired or another did).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = global_timer_ns();
    uint32_t it = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((++it & 63u) == 0u) {
            if (*abort_flag) return false;
            if (global_timer_ns() - t0 > kWaitLimitNs) {
                *abort_flag = 1;
                atomicCAS(status, 0, code);
                return false;
            }
        }
    }
}

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2, int c3) {
    asm volatile(
            "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
            ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
            : "memory");
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
    asm volatile(
            "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
            ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1)
            : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}

__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc], kind::i8, issued by one thread.
__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t"
            "}\n" ::"r"(tmem_d),
            "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
            : "memory");
}

// Arrives on the mbarrier once every tcgen05 operation issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
            "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
              "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
              "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
              "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
            : "r"(taddr)
            : "memory");
}

__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major operand tile whose rows are `bk` bytes long and
// stored with the bk-byte swizzle (128B / 64B / 32B), 8-row groups packed back to back:
//   bits  0-13 start address >> 4, 16-29 leading byte offset >> 4 (unused for swizzled K-major, 1),
//   bits 32-45 stride byte offset >> 4 (distance between 8-row groups = 8 * bk),
//   bits 46-47 descriptor version (1 on sm_100), bits 61-63 swizzle mode (2 = 128B, 4 = 64B, 6 = 32B).
template <int BK>
__device__ __forceinline__ uint64_t make_kmajor_desc(uint32_t smem_addr) {
    constexpr uint64_t layout = BK == 128 ? 2ull : (BK == 64 ? 4ull : 6ull);
    constexpr uint64_t sbo = (8ull * BK) >> 4;
    return (uint64_t)((smem_addr >> 4) & 0x3fffu) | (1ull << 16) | (sbo << 32) | (1ull << 46) | (layout << 61);
}

struct TcParams {
    int Wb, Hb, Nb;
    int tiles_w, tiles_h, tiles_n;  // position tiles
    int col_tiles;                   // ceil(cols / BN)
    int Wo, Ho, No;
    int KH, KW, pad_top, pad_left;
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
};

template <int BN, int BK>
struct TcConfig {
    static constexpr int kStageA = 128 * BK;
    static constexpr int kStageB = BN * BK;
    static constexpr int kStageBytes = kStageA + kStageB;
    static constexpr int kStagesRaw = (200 * 1024) / kStageBytes;
    static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
    static constexpr int kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;
    // barriers: full[kStages], empty[kStages], tmem_full[2], tmem_empty[2]
    static constexpr int kBarBytes = (2 * kStages + 4) * 8;
    static constexpr int kParamOffset = ((kStages * kStageBytes + kBarBytes + 16 + 15) / 16) * 16;  // per-warp epilogue parameter caches
    static constexpr int kParamBytes = 8 * (BN / 2) * 8;
    static constexpr int kSmemBytes = 1024 /*alignment slack*/ + kParamOffset + kParamBytes;
};

template <int BN, int BK>
__global__ void __launch_bounds__(320, 1)
tc_igemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const TcParams p) {
    using Cfg = TcConfig<BN, BK>;
    constexpr int kStages = Cfg::kStages;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + kStages * Cfg::kStageA;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * Cfg::kStageBytes);
    uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

    const uint32_t bar_base = smem_u32(bars);
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * kStages + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * kStages + 2 + a); };

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), 8);  // one arrival per epilogue warp
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

    const int pos_tiles = p.tiles_w * p.tiles_h * p.tiles_n;
    const int total_tiles = pos_tiles * p.col_tiles;
    const int taps = p.KH * p.KW;
    const int num_kb = taps * p.c_chunks;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const int ct = tile % p.col_tiles;
                int pt = tile / p.col_tiles;
                const int tw = pt % p.tiles_w;
                pt /= p.tiles_w;
                const int th = pt % p.tiles_h;
                const int tn = pt / p.tiles_h;
                const int w0 = tw * p.Wb - p.pad_left, h0 = th * p.Hb - p.pad_top, n0 = tn * p.Nb;
                for (int kb = 0; kb < num_kb; ++kb) {
                    const int tap = kb / p.c_chunks, cc = kb - tap * p.c_chunks;
                    const int kh = tap / p.KW, kw = tap - kh * p.KW;
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status, 1)) {
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(full_bar(stage), Cfg::kStageBytes);
                    tma_load_4d(smem_u32(smem_a + stage * Cfg::kStageA), &tmA, full_bar(stage), cc * BK, w0 + kw, h0 + kh, n0);
                    tma_load_2d(smem_u32(smem_b + stage * Cfg::kStageB), &tmB, full_bar(stage), tap * p.c_pad + cc * BK, ct * BN);
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
                const int acc = it & 1;
                const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
                if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, p.status, 2)) break;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)(acc * BN);
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait(full_bar(stage), phase, abort_flag, p.status, 3)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem_a + stage * Cfg::kStageA);
                    const uint32_t b_addr = smem_u32(smem_b + stage * Cfg::kStageB);
#pragma unroll
                    for (int k = 0; k < BK / 32; ++k) {
                        umma_i8(tmem_d, make_kmajor_desc<BK>(a_addr + k * 32), make_kmajor_desc<BK>(b_addr + k * 32), p.idesc,
                                (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(empty_bar(stage));  // frees the stage once these MMAs have read it
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (ok) umma_commit(tfull_bar(acc));  // accumulator complete
            }
        }
    } else {
        // ---------------- epilogue warps ----------------
        // Eight warps: warp w may touch TMEM lanes 32*(w % 4) .. +31 only, so two warps share each lane quarter and
        // split the tile's 32-column chunks between them (even / odd).  Warps are independent of one another (no
        // cross-warp barrier): a warp that sees the abort flag leaves on its own; within a warp the decision is made
        // uniform with a vote because tcgen05.ld is a warp-wide (.sync.aligned) instruction.
        constexpr int kChunks = BN / 32;            // 32-column chunks per tile
        constexpr int kMine = kChunks / 2;          // chunks per warp
        const int e = warp - 2;                     // 0..7
        const int quarter = warp & 3;
        const int half = e >> 2;                    // which chunks (even / odd) this warp owns
        const int row = quarter * 32 + lane;
        const int w_l = row % p.Wb, h_l = (row / p.Wb) % p.Hb, n_l = row / (p.Wb * p.Hb);
        const bool requant = p.epi.mode == kEpiRequant;
        // Per-warp cache of the per-column parameters of the chunks this warp owns: {mult, bias - col_scale*col_corr}.
        float2* s_par = reinterpret_cast<float2*>(smem + Cfg::kParamOffset) + e * (BN / 2);
        int cached_ct = -1;
        const RequantParams rq = p.epi.rq;
        const bool fast_u8 = requant && !rq.y_signed && p.col_mul == nullptr;
        const int hi_q = rq.clamp_hi_q >= 0 ? rq.clamp_hi_q : 255;
        int it = 0;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++it) {
            const int acc = it & 1;
            const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
            const int ct = tile % p.col_tiles;
            int pt = tile / p.col_tiles;
            const int tw = pt % p.tiles_w;
            pt /= p.tiles_w;
            const int th = pt % p.tiles_h;
            const int tn = pt / p.tiles_h;
            const int wo = tw * p.Wb + w_l, ho = th * p.Hb + h_l, no = tn * p.Nb + n_l;
            const bool row_ok = wo < p.Wo && ho < p.Ho && no < p.No;
            const int64_t pos = ((int64_t)no * p.Ho + ho) * p.Wo + wo;
            const int col0 = ct * BN;
            const uint32_t rowc = (row_ok && p.row_corr) ? (uint32_t)p.row_corr[pos] : 0u;

            if (ct != cached_ct) {
                __syncwarp();
                for (int j = lane; j < BN / 2; j += 32) {
                    const int c = col0 + ((j >> 5) * 2 + half) * 32 + (j & 31);
                    float m = 0.f;
                    uint32_t bz = 0u;
                    if (c < p.cols) {
                        if (requant) m = epi_mult(p.epi, c);
                        if (requant && p.epi.bias) bz = (uint32_t)p.epi.bias[c];
                        if (p.col_corr) bz -= (uint32_t)p.col_scale * (uint32_t)p.col_corr[c];
                    }
                    s_par[j] = make_float2(m, __uint_as_float(bz));
                }
                __syncwarp();
                cached_ct = ct;
            }

            const bool got = mbar_wait(tfull_bar(acc), acc_phase, abort_flag, p.status, 4);
            if (!__all_sync(0xffffffffu, got)) break;
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BN);
            uint32_t rbuf[2][32];
            __syncwarp();
            tmem_ld_32x32b_x32(taddr + (uint32_t)(half * 32), rbuf[0]);
#pragma unroll
            for (int i = 0; i < kMine; ++i) {
                uint32_t(&r)[32] = rbuf[i & 1];
                tmem_ld_wait();
                if (i + 1 < kMine) {  // next chunk's TMEM read overlaps this chunk's arithmetic
                    __syncwarp();
                    tmem_ld_32x32b_x32(taddr + (uint32_t)(((i + 1) * 2 + half) * 32), rbuf[(i + 1) & 1]);
                }
                const int ch = i * 2 + half;
                const int cbase = col0 + ch * 32;
                if (row_ok && cbase < p.cols) {
                    const bool full_chunk = cbase + 32 <= p.cols;
                    const int64_t o = pos * p.ldc + cbase;
                    const float2* par = s_par + i * 32;
                    // acc = raw + (bias - col_scale*col_corr[c]) - col_mul[c]*row_corr[pos]   (int32 wrap-around)
#pragma unroll
                    for (int j = 0; j < 32; ++j) r[j] += __float_as_uint(par[j].y);
                    if (p.col_mul) {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (full_chunk || cbase + j < p.cols) r[j] -= (uint32_t)__ldg(p.col_mul + cbase + j) * rowc;
                    }
                    if (!requant) {
                        int32_t* yo = static_cast<int32_t*>(p.y) + o;
                        if (full_chunk && p.vec_ok) {
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                reinterpret_cast<uint4*>(yo)[j] = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (cbase + j < p.cols) yo[j] = (int32_t)r[j];
                        }
                    } else {
                        uint8_t* yo = static_cast<uint8_t*>(p.y) + o;
                        const uint8_t* ro = p.epi.residual ? p.epi.residual + o : nullptr;
                        const bool vec = full_chunk && p.vec_ok;
                        uint32_t resw[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
                        if (ro) {
                            if (vec) {
                                const uint4 r0 = reinterpret_cast<const uint4*>(ro)[0], r1 = reinterpret_cast<const uint4*>(ro)[1];
                                resw[0] = r0.x; resw[1] = r0.y; resw[2] = r0.z; resw[3] = r0.w;
                                resw[4] = r1.x; resw[5] = r1.y; resw[6] = r1.z; resw[7] = r1.w;
                            } else {
#pragma unroll
                                for (int j = 0; j < 32; ++j)
                                    if (cbase + j < p.cols) resw[j >> 2] |= (uint32_t)ro[j] << (8 * (j & 3));
                            }
                        }
                        uint32_t outw[8];
#pragma unroll
                        for (int wv = 0; wv < 8; ++wv) {
                            uint32_t o32 = 0u;
#pragma unroll
                            for (int b = 0; b < 4; ++b) {
                                const int j = wv * 4 + b;
                                int q;
                                if (fast_u8) {
                                    q = min(requant_u8_fast((int)r[j], par[j].x, rq), hi_q);
                                } else {
                                    q = requant_one((int)r[j], par[j].x, rq);
                                }
                                if (ro) q = residual_one(q, (int)((resw[wv] >> (8 * b)) & 0xffu), rq);
                                o32 |= ((uint32_t)q & 0xffu) << (8 * b);
                            }
                            outw[wv] = o32;
                        }
                        if (vec) {
                            reinterpret_cast<uint4*>(yo)[0] = make_uint4(outw[0], outw[1], outw[2], outw[3]);
                            reinterpret_cast<uint4*>(yo)[1] = make_uint4(outw[4], outw[5], outw[6], outw[7]);
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (cbase + j < p.cols) yo[j] = (uint8_t)(outw[j >> 2] >> (8 * (j & 3)));
                        }
                    }
                }
            }
            // Hand the accumulator buffer back to the MMA warp.
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar(acc));
        }
    }

    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        // Bounded grace period for copies and MMAs still in flight before shared memory and TMEM go away.
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 2000000ull) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, Cfg::kTmemCols);
    }
}

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

int num_sms() {
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
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
double g_cur_macs = 0.0;

template <int BN, int BK>
int launch_cfg(const CUtensorMap& tmA, const CUtensorMap& tmB, const TcParams& p, int total_tiles, cudaStream_t s) {
    using Cfg = TcConfig<BN, BK>;
    static bool attr_set[64] = {};
    int dev = 0;
    CHXQ_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !attr_set[dev]) {
        CHXQ_CUDA(cudaFuncSetAttribute(tc_igemm_kernel<BN, BK>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
        if (dev >= 0 && dev < 64) attr_set[dev] = true;
    }
    const int grid = total_tiles < num_sms() ? total_tiles : num_sms();
    ProfRec rec{};
    if (g_prof_on) {
        CHXQ_CUDA(cudaEventCreate(&rec.e0));
        CHXQ_CUDA(cudaEventCreate(&rec.e1));
        rec.macs = g_cur_macs;
        CHXQ_CUDA(cudaEventRecord(rec.e0, s));
    }
    tc_igemm_kernel<BN, BK><<<grid, 320, Cfg::kSmemBytes, s>>>(tmA, tmB, p);
    if (g_prof_on) {
        CHXQ_CUDA(cudaEventRecord(rec.e1, s));
        std::lock_guard<std::mutex> lock(g_prof_mu);
        g_prof.push_back(rec);
    }
    CHXQ_LAUNCH_CHECK();
    return CHXQ_OK;
}

template <int BN>
int launch_bn(int bk, const CUtensorMap& tmA, const CUtensorMap& tmB, const TcParams& p, int total_tiles, cudaStream_t s) {
    switch (bk) {
        case 128: return launch_cfg<BN, 128>(tmA, tmB, p, total_tiles, s);
        case 64: return launch_cfg<BN, 64>(tmA, tmB, p, total_tiles, s);
        case 32: return launch_cfg<BN, 32>(tmA, tmB, p, total_tiles, s);
    }
    return set_error(CHXQ_ERR_INVALID_ARGUMENT, "tensor-core kernel: bk must be 32, 64 or 128");
}

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

int choose_bk(int k) {
    const int cand[3] = {128, 64, 32};
    int best = 32, best_cost = 1 << 30;
    for (int i = 0; i < 3; ++i) {
        const int cost = (k + cand[i] - 1) / cand[i] * cand[i];
        if (cost < best_cost) {
            best_cost = cost;
            best = cand[i];
        }
    }
    return best;
}

static int largest_pow2_divisor(int v, int cap) {
    int d = 1;
    while (d * 2 <= cap && v % (d * 2) == 0) d *= 2;
    return d;
}

TcConvPlan plan_tc_conv(const chxq_conv_geom& g) {
    TcConvPlan pl{};
    pl.path = kTcNone;
    if (g.group != 1 || g.y_layout != CHXQ_NHWC) return pl;
    const int taps = g.KH * g.KW;
    const int64_t xcs = g.x_cstride > 0 ? g.x_cstride : g.C;
    const bool direct = g.x_layout == CHXQ_NHWC && g.stride_h == 1 && g.stride_w == 1 && (xcs % 16 == 0) && g.pad_top >= 0 && g.pad_left >= 0 &&
                        g.pad_bottom >= 0 && g.pad_right >= 0 && g.pad_top < g.KH && g.pad_left < g.KW && g.C >= 16;
    if (direct) {
        pl.path = kTcDirect;
        pl.bk = choose_bk(g.C);
        pl.c_pitch = (g.C + pl.bk - 1) / pl.bk * pl.bk;
        pl.k_total = taps * pl.c_pitch;
        if (taps == 1 && g.pad_top == 0 && g.pad_left == 0 && g.pad_bottom == 0 && g.pad_right == 0 && (int64_t)g.N * g.H * g.W < (1ll << 31)) {
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
    const int K = taps * g.C;
    pl.path = kTcIm2col;
    pl.bk = choose_bk(K);
    pl.c_pitch = g.C;
    pl.k_total = (K + pl.bk - 1) / pl.bk * pl.bk;
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

    TcParams p{};
    p.Wb = q.Wb; p.Hb = q.Hb; p.Nb = q.Nb;
    p.tiles_w = (q.Wo + q.Wb - 1) / q.Wb;
    p.tiles_h = (q.Ho + q.Hb - 1) / q.Hb;
    p.tiles_n = (q.No + q.Nb - 1) / q.Nb;
    const int64_t pos_tiles = (int64_t)p.tiles_w * p.tiles_h * p.tiles_n;
    const int bn = q.bn ? q.bn : pick_bn(q.cols, pos_tiles);
    p.col_tiles = (q.cols + bn - 1) / bn;
    const int64_t total_tiles = pos_tiles * p.col_tiles;
    if (total_tiles >= (1ll << 31)) return set_error(CHXQ_ERR_UNSUPPORTED, "tensor-core kernel: too many tiles");
    p.Wo = q.Wo; p.Ho = q.Ho; p.No = q.No;
    p.KH = q.KH; p.KW = q.KW; p.pad_top = q.pad_top; p.pad_left = q.pad_left;
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
    p.status = device_status_ptr();
    if (!p.status) return set_error(CHXQ_ERR_CUDA, "device status word is unavailable");
    const int elt = q.epi.mode == kEpiInt32 ? 4 : 1;
    p.vec_ok = ((reinterpret_cast<uintptr_t>(q.y) & 15u) == 0) && ((q.ldc * elt) % 16 == 0) &&
               (q.epi.residual == nullptr || (reinterpret_cast<uintptr_t>(q.epi.residual) & 15u) == 0);

    // A: {C, W, H, N} bytes, pitches {a_cs, W*a_cs, H*W*a_cs}; box {bk, Wb, Hb, Nb}; out-of-range reads fill 0.
    alignas(64) CUtensorMap tmA, tmB;
    {
        const cuuint64_t dims[4] = {(cuuint64_t)q.C, (cuuint64_t)q.W, (cuuint64_t)q.H, (cuuint64_t)q.N};
        const cuuint64_t strides[3] = {(cuuint64_t)q.a_cs, (cuuint64_t)q.a_cs * q.W, (cuuint64_t)q.a_cs * q.W * q.H};
        const cuuint32_t box[4] = {(cuuint32_t)q.bk, (cuuint32_t)q.Wb, (cuuint32_t)q.Hb, (cuuint32_t)q.Nb};
        const cuuint32_t estr[4] = {1, 1, 1, 1};
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
    g_cur_macs = q.alg_macs;
    switch (bn) {
        case 256: return launch_bn<256>(q.bk, tmA, tmB, p, (int)total_tiles, s);
        case 128: return launch_bn<128>(q.bk, tmA, tmB, p, (int)total_tiles, s);
        case 64: return launch_bn<64>(q.bk, tmA, tmB, p, (int)total_tiles, s);
    }
    return set_error(CHXQ_ERR_INVALID_ARGUMENT, "tensor-core kernel: bn must be 64, 128 or 256");
}

}  // namespace chxq

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
