// tcgen05 implicit-GEMM kernel for sm_100a (device code; see tc_igemm.cu for the host side): u8/s8 x u8/s8 -> s32 in
// TMEM (kind::i8), operands staged in shared memory by TMA (no cluster multicast anywhere), zero-point terms,
// per-channel requantize, bias, ReLU clamp and the residual tail applied in the epilogue straight out of TMEM.
//
// One persistent CTA per SM, 576 threads:
//   warp 0      : TMA producer (one elected lane): A box {bk, Wb, Hb, Nb} of an NHWC map / matrix,
//                 B box {bk, BN} of the packed weights, ring of kStages shared-memory stages.
//   warp 1      : allocates TMEM, issues tcgen05.mma (one elected lane), M = 128, N = BN, K = 32 per
//                 instruction; accumulators are double-buffered in TMEM (2 x BN columns) so the
//                 epilogue of tile i overlaps the main loop of tile i + 1.
//   warps 2..17 : epilogue; warp w may read TMEM lanes 32*(w % 4) .. +31 (one output position per thread), four
//                 warps per lane quarter take every fourth 16-column chunk of the tile; per-channel parameters
//                 come from a per-warp shared-memory cache, outputs leave as 128-bit stores.
//
// Every mbarrier wait is bounded: after ~2 s without progress the waiting thread raises the CTA's
// abort flag and the device status word, every role leaves its loop, the CTA waits a bounded time
// for copies in flight, frees its TMEM and returns.  Nothing traps.
#pragma once

#include <cuda.h>

#include <atomic>

#include "common.h"
#include "kernels.h"
#include "tc_launch.h"

namespace chxq {
namespace tc {

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

// Programmatic dependent launch: a kernel launched with the programmatic-serialization attribute may start while the kernel
// before it in the stream is still running.  launch_dependents lets the next kernel's CTAs be scheduled as soon as this
// kernel's CTAs leave their SMs; dependency_wait blocks until the previous kernel has completed and its writes are visible.
// Everything a CTA does before dependency_wait (barrier initialisation, tensor-memory allocation) overlaps the previous
// kernel's tail; nothing before it may touch global memory that the previous kernel writes or reads.
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_dependency_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

constexpr uint64_t kWaitLimitNs = 2000000000ull;  // 2 s

// Bounded wait.  Returns false when the CTA is aborting (either this wait expired or another did).
// sleep_ns == 0: a tight poll loop (try_wait itself blocks in hardware for a short while, so the loop issues a few
// instructions per ~100 ns) -- for the single-lane producer / MMA / store roles, whose wake-up latency is on the
// critical path of load-bound layers.  sleep_ns > 0: sleep between polls, doubling up to 8 * sleep_ns -- for the sixteen
// epilogue warps, whose polling would otherwise take issue slots from the warps that do the work.
// The abort flag and the clock are looked at every 256 polls.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code, uint32_t sleep_ns = 64,
                                          uint64_t limit_ns = kWaitLimitNs) {
    if (mbar_try_wait(bar, parity)) return true;
    uint64_t t0 = 0;
    uint32_t ns = sleep_ns;
    const uint32_t ns_max = sleep_ns * 8u;
    while (true) {
#pragma unroll 1
        for (int i = 0; i < 256; ++i) {
            if (sleep_ns != 0) {
                __nanosleep(ns);
                if (ns < ns_max) ns <<= 1;
            }
            if (mbar_try_wait(bar, parity)) return true;
        }
        if (*abort_flag) return false;
        const uint64_t now = global_timer_ns();
        if (t0 == 0) t0 = now;
        if (now - t0 > limit_ns) {
            *abort_flag = 1;
            atomicCAS(status, 0, code);
            return false;
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

__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
              "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
            : "r"(taddr)
            : "memory");
}

// Waits for this thread's outstanding TMEM loads.  The destination registers are passed through the statement as
// read-write operands so that no use of them can be scheduled ahead of the wait.
__device__ __forceinline__ void tmem_ld_wait16(uint32_t (&r)[16]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]), "+r"(r[9]),
                   "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
                 :
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

// The same descriptor as two 32-bit halves.  The MMA warp issues from one thread, whose instructions are dependent and
// several cycles apart: rebuilding a 64-bit descriptor per instruction (shifts, masks, ors) costs more cycles than a
// 128 x 64 x 32 MMA takes.  The high word is a constant of the layout; the low word is (address >> 4) plus constant bits,
// so stepping along K or to the next tile of a stage is one 32-bit add of a compile-time constant (shared memory is
// smaller than 256 KB, so the 14-bit address field never carries).
template <int BK>
__device__ __forceinline__ uint32_t kmajor_desc_hi() {
    constexpr uint32_t layout = BK == 128 ? 2u : (BK == 64 ? 4u : 6u);
    return (uint32_t)((8 * BK) >> 4) | (1u << 14) | (layout << 29);
}
__device__ __forceinline__ uint32_t kmajor_desc_lo(uint32_t smem_addr) {
    return (smem_addr >> 4) | (1u << 16);
}

__device__ __forceinline__ void umma_i8_lohi(uint32_t tmem_d, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                             uint32_t accumulate) {
    asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            ".reg .b64 da, db;\n\t"
            "mov.b64 da, {%1, %2};\n\t"
            "mov.b64 db, {%3, %4};\n\t"
            "setp.ne.b32 p, %6, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::i8 [%0], da, db, %5, p;\n\t"
            "}\n" ::"r"(tmem_d),
            "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
            : "memory");
}

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
    static constexpr int kParamBytes = 16 * (BN / 2) * 4;  // 16 warps x (BN/4 multipliers + BN/4 additive terms)
    static constexpr int kSmemBytes = 1024 /*alignment slack*/ + kParamOffset + kParamBytes;
};

template <int BN, int BK, int EPI>
__global__ void __launch_bounds__(576, 1)
tc_igemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const TcParams p) {
    using Cfg = TcConfig<BN, BK>;
    constexpr int kStages = Cfg::kStages;
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment by offset, so that the pointer stays a shared-memory pointer for the compiler (ld.shared / st.shared)
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
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
            mbar_init(tempty_bar(a), 16);  // one arrival per epilogue warp
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
                const int w0 = tw * p.Wb * p.sw - p.pad_left, h0 = th * p.Hb * p.sh - p.pad_top, n0 = tn * p.Nb;
                const int gbase = p.group_cols > 0 ? (ct * BN / p.group_cols) * p.group_cin : 0;
                for (int kb = 0; kb < num_kb; ++kb) {
                    const int tap = kb / p.c_chunks, cc = kb - tap * p.c_chunks;
                    const int kh = tap / p.KW, kw = tap - kh * p.KW;
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status, 1, 0, p.wait_limit_ns)) {
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(full_bar(stage), Cfg::kStageBytes);
                    tma_load_4d(smem_u32(smem_a + stage * Cfg::kStageA), &tmA, full_bar(stage), gbase + cc * BK, w0 + kw, h0 + kh, n0);
                    // (test of the bounded waits only: one weight load left out, so that this stage never fills)
                    if (kb != p.test_skip_kb)
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
            const uint32_t desc_hi = kmajor_desc_hi<BK>();
            const uint32_t a_lo0 = kmajor_desc_lo(smem_u32(smem_a)), b_lo0 = kmajor_desc_lo(smem_u32(smem_b));
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
                const int acc = it & 1;
                const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
                if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, p.status, 2, 0, p.wait_limit_ns)) break;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)(acc * BN);
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait(full_bar(stage), phase, abort_flag, p.status, 3, 0, p.wait_limit_ns)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_lo = a_lo0 + (uint32_t)(stage * (Cfg::kStageA >> 4));
                    const uint32_t b_lo = b_lo0 + (uint32_t)(stage * (Cfg::kStageB >> 4));
#pragma unroll
                    for (int k = 0; k < BK / 32; ++k)
                        umma_i8_lohi(tmem_d, a_lo + k * 2, desc_hi, b_lo + k * 2, desc_hi, p.idesc, (kb > 0 || k > 0) ? 1u : 0u);
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
        // Sixteen warps: warp w may touch TMEM lanes 32*(w % 4) .. +31 only, so four warps share each lane quarter and
        // take every fourth 16-column chunk of the tile.  Warps are independent of one another (no cross-warp barrier):
        // a warp that sees the abort flag leaves on its own; within a warp the decision is made uniform with a vote
        // because tcgen05.ld is warp-wide (.sync.aligned).
        constexpr int kMine = BN / 64;              // 16-column chunks per warp per tile
        const int e = warp - 2;                     // 0..15
        const int quarter = warp & 3;
        const int sub = e >> 2;                     // this warp owns the chunks with (chunk & 3) == sub
        const int row = quarter * 32 + lane;
        const int w_l = row % p.Wb, h_l = (row / p.Wb) % p.Hb, n_l = row / (p.Wb * p.Hb);
        // Per-warp cache of the per-column parameters of this warp's chunks: multiplier and additive int32 term.
        float* s_mult = reinterpret_cast<float*>(smem + Cfg::kParamOffset) + e * (BN / 2);  // [BN/4] floats then [BN/4] ints
        uint32_t* s_add = reinterpret_cast<uint32_t*>(s_mult + BN / 4);
        int cached_ct = -1;
        const RequantParams rq = p.epi.rq;
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

            if (ct != cached_ct) {
                __syncwarp();
                for (int j = lane; j < BN / 4; j += 32) {
                    const int c = col0 + ((j >> 4) * 4 + sub) * 16 + (j & 15);
                    float m = 0.f;
                    uint32_t bz = 0u;
                    if (c < p.cols) {
                        if (EPI != kEpiKInt32) {
                            m = epi_mult(p.epi, c);
                            if (EPI == kEpiKU8Fold || (EPI == kEpiKGeneric && rq.fold)) m = __fdiv_rn(m, rq.y_scale);  // folded: mult / y_scale
                            if (p.epi.bias) bz = (uint32_t)p.epi.bias[c];
                        }
                        if (p.col_corr) bz -= (uint32_t)p.col_scale * (uint32_t)p.col_corr[c];
                    }
                    // additive term: int32 (bias and activation zero-point term) or, folded, the float offset of the bias; the folded
                    // round-half-up form keeps both in units of the output range (fold_channel)
                    if (EPI == kEpiKU8Fold) {
                        const int bias = (c < p.cols && p.epi.bias) ? p.epi.bias[c] : 0;
                        const FoldCh fc = fold_channel(bias, m, rq);
                        s_mult[j] = fc.ms;
                        s_add[j] = __float_as_uint(fc.bs);
                    } else {
                        s_mult[j] = m;
                        s_add[j] = bz;
                    }
                }
                __syncwarp();
                cached_ct = ct;
            }

            // Residual bytes of this warp's chunks are fetched before the accumulator is waited for, so that their latency
            // overlaps the main loop of the tile (vector path only; ragged chunks load theirs bytewise).
            const uint8_t* res_row = (EPI != kEpiKInt32 && p.epi.residual && row_ok) ? p.epi.residual + pos * p.ldc : nullptr;
            auto res_load = [&](int i) -> uint4 {
                const int cb = col0 + (i * 4 + sub) * 16;
                if (EPI != kEpiKInt32 && res_row && p.vec_ok && i < kMine && cb + 16 <= p.cols)
                    return __ldg(reinterpret_cast<const uint4*>(res_row + cb));
                return make_uint4(0u, 0u, 0u, 0u);
            };
            uint4 res0 = res_load(0), res1 = res_load(1);

            const bool got = mbar_wait(tfull_bar(acc), acc_phase, abort_flag, p.status, 4, 32, p.wait_limit_ns);
            if (!__all_sync(0xffffffffu, got)) break;
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BN);
            // One 16-column chunk: registers of TMEM data in, 16 bytes (or 16 int32) out.
            auto process = [&](uint32_t (&r)[16], const int i, const uint4 resv) {
                const int ch = i * 4 + sub;
                const int cbase = col0 + ch * 16;
                if (!(row_ok && cbase < p.cols)) return;
                const bool full_chunk = cbase + 16 <= p.cols;
                const int64_t o = pos * p.ldc + cbase;
                const float4* pm = reinterpret_cast<const float4*>(s_mult + i * 16);
                const uint4* pa = reinterpret_cast<const uint4*>(s_add + i * 16);
                uint32_t addw[16];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint4 a4 = pa[j];
                    addw[4 * j] = a4.x; addw[4 * j + 1] = a4.y; addw[4 * j + 2] = a4.z; addw[4 * j + 3] = a4.w;
                }
                if (EPI != kEpiKU8Fold) {
                    // acc = raw + (bias - col_scale * col_corr[c])   (int32 wrap-around)
#pragma unroll
                    for (int j = 0; j < 16; ++j) r[j] += addw[j];
                } else if (p.col_corr) {
                    // folded: the bias lives in the float offset; only the activation zero-point term is an integer
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (full_chunk || cbase + j < p.cols) r[j] -= (uint32_t)p.col_scale * (uint32_t)__ldg(p.col_corr + cbase + j);
                }
                if (EPI == kEpiKInt32 || EPI == kEpiKGeneric) {
                    if (p.col_mul) {  // weight zero-point term: - zw[c] * sum over the receptive field of (x - zx)
                        const uint32_t rowc = p.row_corr ? (uint32_t)p.row_corr[pos] : 0u;
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (full_chunk || cbase + j < p.cols) r[j] -= (uint32_t)__ldg(p.col_mul + cbase + j) * rowc;
                    }
                }
                if (EPI == kEpiKInt32) {
                    int32_t* yo = static_cast<int32_t*>(p.y) + o;
                    if (full_chunk && p.vec_ok) {
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            reinterpret_cast<uint4*>(yo)[j] = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (cbase + j < p.cols) yo[j] = (int32_t)r[j];
                    }
                } else {
                    uint8_t* yo = static_cast<uint8_t*>(p.y) + o;
                    const uint8_t* ro = p.epi.residual ? p.epi.residual + o : nullptr;
                    const bool vec = full_chunk && p.vec_ok;
                    uint32_t resw[4] = {0u, 0u, 0u, 0u};
                    if (ro) {
                        if (vec) {
                            resw[0] = resv.x; resw[1] = resv.y; resw[2] = resv.z; resw[3] = resv.w;
                        } else {
#pragma unroll
                            for (int j = 0; j < 16; ++j)
                                if (cbase + j < p.cols) resw[j >> 2] |= (uint32_t)ro[j] << (8 * (j & 3));
                        }
                    }
                    uint32_t outw[4];
                    if (EPI == kEpiKGeneric) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float4 m4 = pm[j];
                            const float mm[4] = {m4.x, m4.y, m4.z, m4.w};
                            uint32_t o32 = 0u;
#pragma unroll
                            for (int b = 0; b < 4; ++b) {
                                const int a = (int)r[4 * j + b];
                                const int rb = (int)((resw[j] >> (8 * b)) & 0xffu);
                                int q;
                                if (rq.fold) {
                                    const int cc = cbase + 4 * j + b;
                                    const int bpure = (p.epi.bias && cc < p.cols) ? __ldg(p.epi.bias + cc) : 0;
                                    q = requant_u8_fold((int)(r[4 * j + b] - (uint32_t)bpure), bpure, mm[b], rq);
                                    if (ro) q = residual_fold(q, rb, rq);
                                } else {
                                    q = requant_one(a, mm[b], rq);
                                    if (ro) q = residual_one(q, rb, rq);
                                }
                                o32 |= ((uint32_t)q & 0xffu) << (8 * b);
                            }
                            outw[j] = o32;
                        }
                    } else {
                        // uint8, round-half-up (the other rounding mode takes the general kernel): one int->float conversion
                        // per element, everything else on the add/multiply pipes (see qmath.cuh), no per-element branches
                        // (adding a zero zero point is exact).  Results equal requant_one / residual_one (reference operation
                        // order) or requant_u8_fold / residual_fold (folded: saturating multiply-adds in units of the output
                        // range) bit for bit.
                        constexpr bool kFold = EPI == kEpiKU8Fold;
                        const float hi_ph = (float)hi_q + 0.5f;
                        const float cy = kMagic23 + rq.y_zp_f, cr = kMagic23 + rq.res_zp_f;
                        const float relu_floor = rq.res_relu ? 0.f : -3.0e38f;
                        const float relu_q = rq.res_relu ? kMagic23 + rq.out_zp_f : 0.f;  // folded tail: Relu = clamp at the output zero point
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float4 m4 = pm[j];
                            const float mm[4] = {m4.x, m4.y, m4.z, m4.w};
                            uint32_t fb[4];
#pragma unroll
                            for (int b = 0; b < 4; ++b) {
                                const float a = (float)(int)r[4 * j + b];
                                if (kFold) {
                                    const float t = __saturatef(__fmaf_rn(a, mm[b], __uint_as_float(addw[4 * j + b])));
                                    fb[b] = __float_as_uint(__fmaf_rd(t, hi_ph, kMagic23));
                                } else {
                                    float tp = qdiv(__fmul_rn(a, mm[b]), rq.y_div);
                                    tp = __fadd_rn(__fadd_rn(tp, rq.y_zp_f), 0.5f);
                                    fb[b] = __float_as_uint(quant_u8_up_magic(tp, hi_ph));
                                }
                            }
                            if (ro) {
#pragma unroll
                                for (int b = 0; b < 4; ++b) {
                                    if (kFold) {
                                        const float qf = __fsub_rn(__uint_as_float(fb[b]), kMagic23);     // q, exact
                                        const float rf = __fsub_rn(byte_to_magic(resw[j], b), kMagic23);   // r, exact
                                        const float t = __saturatef(__fmaf_rn(qf, rq.fold_a, __fmaf_rn(rf, rq.fold_r, rq.fold_c)));
                                        fb[b] = __float_as_uint(fmaxf(__fmaf_rd(t, 255.5f, kMagic23), relu_q));
                                        continue;
                                    }
                                    const float u = __fsub_rn(__uint_as_float(fb[b]), cy);           // q - y_zp, exact
                                    const float w = __fsub_rn(byte_to_magic(resw[j], b), cr);          // r - res_zp, exact
                                    float v = __fadd_rn(__fmul_rn(u, rq.y_scale), __fmul_rn(w, rq.res_scale));
                                    v = fmaxf(v, relu_floor);
                                    v = qdiv(v, rq.out_div);
                                    const float tp = __fadd_rn(__fadd_rn(v, rq.out_zp_f), 0.5f);
                                    fb[b] = __float_as_uint(quant_u8_up_magic(tp, 255.5f));
                                }
                            }
                            const uint32_t lo = __byte_perm(fb[0], fb[1], 0x0040), hi = __byte_perm(fb[2], fb[3], 0x0040);
                            outw[j] = __byte_perm(lo, hi, 0x5410);
                        }
                    }
                    if (vec) {
                        *reinterpret_cast<uint4*>(yo) = make_uint4(outw[0], outw[1], outw[2], outw[3]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (cbase + j < p.cols) yo[j] = (uint8_t)(outw[j >> 2] >> (8 * (j & 3)));
                    }
                }
            };
            // Chunks are processed one after the other, fully unrolled (at most four per warp); the other warps of the
            // scheduler cover the TMEM read latency.
            uint4 resv[4] = {res0, res1, res_load(2), res_load(3)};
#pragma unroll
            for (int i = 0; i < kMine; ++i) {
                uint32_t ra[16];
                __syncwarp();
                tmem_ld_32x32b_x16(taddr + (uint32_t)((i * 4 + sub) * 16), ra);
                tmem_ld_wait16(ra);
                process(ra, i, resv[i]);
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

// Launches the instantiation for (bn, BK, epi).  Called from the per-BK translation units.
template <int BN, int BK, int EPI>
int launch_one(const CUtensorMap& tmA, const CUtensorMap& tmB, const TcParams& p, int grid, cudaStream_t s) {
    using Cfg = TcConfig<BN, BK>;
    static std::atomic<bool> attr_set[64] = {};  // per device; host threads may race here, every writer stores true
    int dev = 0;
    CHXQ_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !attr_set[dev].load(std::memory_order_acquire)) {
        CHXQ_CUDA(cudaFuncSetAttribute(tc_igemm_kernel<BN, BK, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
        if (dev >= 0 && dev < 64) attr_set[dev].store(true, std::memory_order_release);
    }
    tc_igemm_kernel<BN, BK, EPI><<<grid, 576, Cfg::kSmemBytes, s>>>(tmA, tmB, p);
    CHXQ_LAUNCH_CHECK();
    return CHXQ_OK;
}

template <int BK>
int launch_bk(int bn, int epi, const CUtensorMap& tmA, const CUtensorMap& tmB, const TcParams& p, int grid, cudaStream_t s) {
    if (epi == kEpiKGeneric) return launch_one<128, BK, kEpiKGeneric>(tmA, tmB, p, grid, s);  // rare path: one tile shape
    switch (bn * 4 + epi) {
        case 64 * 4 + kEpiKInt32: return launch_one<64, BK, kEpiKInt32>(tmA, tmB, p, grid, s);
        case 128 * 4 + kEpiKInt32: return launch_one<128, BK, kEpiKInt32>(tmA, tmB, p, grid, s);
        case 256 * 4 + kEpiKInt32: return launch_one<256, BK, kEpiKInt32>(tmA, tmB, p, grid, s);
        case 64 * 4 + kEpiKU8: return launch_one<64, BK, kEpiKU8>(tmA, tmB, p, grid, s);
        case 128 * 4 + kEpiKU8: return launch_one<128, BK, kEpiKU8>(tmA, tmB, p, grid, s);
        case 256 * 4 + kEpiKU8: return launch_one<256, BK, kEpiKU8>(tmA, tmB, p, grid, s);
        case 64 * 4 + kEpiKU8Fold: return launch_one<64, BK, kEpiKU8Fold>(tmA, tmB, p, grid, s);
        case 128 * 4 + kEpiKU8Fold: return launch_one<128, BK, kEpiKU8Fold>(tmA, tmB, p, grid, s);
        case 256 * 4 + kEpiKU8Fold: return launch_one<256, BK, kEpiKU8Fold>(tmA, tmB, p, grid, s);
    }
    return set_error(CHXQ_ERR_INVALID_ARGUMENT, "tensor-core kernel: no instantiation for bn %d, epilogue %d", bn, epi);
}

}  // namespace tc
}  // namespace chxq
