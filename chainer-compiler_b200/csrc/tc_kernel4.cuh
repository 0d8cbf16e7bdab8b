// Two convolutions as one tcgen05 kernel: a KH x KW convolution with MID output channels whose only reader is a 1x1 / stride-1
// convolution (the second and third layer of a ResNet bottleneck; the residual tail of the block rides on the second
// product's epilogue).  The intermediate map never exists in global memory: the first product's requantized uint8 tile (128
// positions x MID channels) is written by the epilogue warps into shared memory in the K-major swizzled layout of an A operand,
// and the second product reads it from there.
//
// Why: run separately, the first layer is bound by the tensor pipe and its operand loads and leaves the issue slots idle,
// the second (K = MID is short, four times as many outputs, residual tail) is bound by the instructions of its epilogue and
// leaves the tensor pipe idle.  Here the first product of tile i + 1 is issued between the column passes of the second
// product of tile i, so the tensor pipe works for one tile while the epilogue warps requantize the other.
//
// Roles (640 threads): warp 0 loads both operands of the first product, warp 1 issues its MMAs, warp 19 issues the MMAs of the second
// product and loads its weights, warps 2-17 run both epilogues, warp 18 issues the TMA stores and the loads of the residual tiles.
//
// Tensor memory (512 columns): [0, 256) the first product's accumulators (two buffers of MID columns, one when MID = 256),
// [256, 512) two buffers of 128 columns for the second product, which runs in passes of 128 output channels.
//
// The two products have their own operand rings and their own MMA threads, so neither waits for the other: the first product of the
// next tiles runs ahead as far as its accumulator buffers allow, whatever the pace of the epilogue, and a pass of the second product is
// issued the moment the epilogue hands an accumulator buffer back.  (One thread that polls both streams' barriers loses: a barrier test
// costs ~150-200 cycles while the epilogue warps use the shared-memory pipe.)  The epilogue warps produce the NEXT tile's intermediate
// tile before the last pass of the current one, so that the round trip through the tensor pipe for the next tile's first pass hides
// behind that pass.
//
// Every wait is bounded as in tc_kernel.cuh.  Results are bit-identical to the two layers run one after the other.
#pragma once

#include "tc_kernel2.cuh"

namespace chxq {
namespace tc {

#ifdef CHXQ_TL
// timeline build: (code, clock) pairs of CTA 0 per role into p.tl
#define CHXQ_TL4(region, cap, code)                                               \
    do {                                                                          \
        if (p.tl && blockIdx.x == 0 && tl_n < (cap)) {                            \
            p.tl[(region) + 2 * tl_n] = (code);                                   \
            p.tl[(region) + 2 * tl_n + 1] = clock64();                            \
            ++tl_n;                                                               \
        }                                                                         \
    } while (0)
#else
#define CHXQ_TL4(region, cap, code) do {} while (0)
#endif

template <int MID>
struct Tc4Config {
    static constexpr int BK = MID == 64 ? 64 : 128;       // K tile in bytes of both products
    static constexpr int kChunks2 = MID / BK;             // K blocks of the second product
    // A stage of the first ring holds kSub consecutive K blocks of the first product (positions + weights each): with 64-byte K
    // blocks one block is only two MMAs, too few for the round trip through the barriers that every stage costs the single-thread roles.
    static constexpr int kSub = MID == 64 ? 3 : 1;
    static constexpr int kStageA = 128 * BK;              // one K block of positions
    static constexpr int kStageB = MID * BK;              // one K block of weights
    static constexpr int kStageBytes = kSub * (kStageA + kStageB);  // [kSub position blocks][kSub weight blocks]
    static constexpr int kSlot2 = 128 * BK;               // second ring: one K block of 128 output channels' weights per slot
    static constexpr int kSlots2 = 3;
    static constexpr int kA2Bytes = 128 * MID;            // the intermediate tile: kChunks2 swizzled [128][BK] blocks
    static constexpr int kTileOut = 128 * 128;            // one staged output (or residual) tile of a pass
    // staging buffers (up to four): a residual tile is fetched into a buffer as soon as the store of the pass that used it before has
    // read it (measured: four buffers are no faster than three and cost a stage of the first ring)
    static constexpr int kBufs = MID == 256 ? 2 : 3;
    static constexpr int kOutBytes = kBufs * kTileOut;
    static constexpr int kD1Bufs = MID == 256 ? 1 : 2;
    static constexpr int kMaxOut = MID == 64 ? 512 : 1024;  // output channels of the second convolution the tables have room for
    static constexpr int kParamBytes = (MID + kMaxOut) * 8;  // per channel: multiplier and offset of the folded requantization
    static constexpr int kBudget = 225 * 1024;
    static constexpr int kStagesRaw = (kBudget - kSlots2 * kSlot2 - kA2Bytes - kOutBytes - kParamBytes - 512) / kStageBytes;
    static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
    static constexpr int kNumBars = 2 * kStages + 2 * kSlots2 + 21;
    static constexpr int kRing2Offset = kStages * kStageBytes;
    static constexpr int kA2Offset = kRing2Offset + kSlots2 * kSlot2;
    static constexpr int kOutOffset = kA2Offset + kA2Bytes;
    static constexpr int kBarOffset = kOutOffset + kOutBytes;
    static constexpr int kParamOffset = ((kBarOffset + kNumBars * 8 + 16 + 15) / 16) * 16;
    static constexpr int kSmemBytes = 1024 /*alignment slack*/ + kParamOffset + kParamBytes;
    static constexpr int kThreads = 640;
    static_assert(kStages >= 2, "chain kernel: not enough shared memory for two stages");
    static_assert(kSmemBytes <= 227 * 1024, "chain kernel: shared memory over the limit");
};

__device__ __forceinline__ uint32_t mbar_test(uint32_t bar, uint32_t parity) {  // non-blocking
    uint32_t ok;
    asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t"
            "}\n"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
    return ok;
}

// Sixteen accumulators of consecutive channels -> sixteen bytes: the folded requantization of qmath.cuh (fold_channel /
// residual_fold), on pairs of floats where no clamp is involved.  ms / bs: the channels' multipliers and offsets in shared memory
// (16-byte aligned); resv: the residual bytes (kRes).
template <bool kRes>
__device__ __forceinline__ uint4 fold_chunk16(uint32_t (&r)[16], const float* ms, const float* bs, const uint4 resv, const uint64_t hp2, const uint64_t fr2,
                                              const uint64_t fc2, const float fa) {
    const uint64_t magic23x2 = pack2(kMagic23, kMagic23);
    const uint64_t c255x2 = pack2(255.5f, 255.5f);
    const uint32_t resw[4] = {resv.x, resv.y, resv.z, resv.w};
    const uint4* pm = reinterpret_cast<const uint4*>(ms);
    const uint4* pa = reinterpret_cast<const uint4*>(bs);
    uint32_t outw[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint4 m4 = pm[j], a4 = pa[j];
        const uint32_t mmw[4] = {m4.x, m4.y, m4.z, m4.w};
        const uint32_t addw[4] = {a4.x, a4.y, a4.z, a4.w};
        uint32_t fb[4];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int e0 = 2 * h;
            float t0 = fma_sat((float)(int)r[4 * j + e0], __uint_as_float(mmw[e0]), __uint_as_float(addw[e0]));
            float t1 = fma_sat((float)(int)r[4 * j + e0 + 1], __uint_as_float(mmw[e0 + 1]), __uint_as_float(addw[e0 + 1]));
            uint64_t f2 = fma_rm_x2(pack2(t0, t1), hp2, magic23x2);  // 2^23 + q
            if (kRes) {
                const uint64_t q2 = sub_x2(f2, magic23x2);  // q, exact
                const uint64_t r2 = sub_x2(pack2(byte_to_magic(resw[j], 2 * h), byte_to_magic(resw[j], 2 * h + 1)), magic23x2);
                const uint64_t in2 = fma_x2(r2, fr2, fc2);
                t0 = fma_sat(lo_of(q2), fa, lo_of(in2));
                t1 = fma_sat(hi_of(q2), fa, hi_of(in2));
                f2 = fma_rm_x2(pack2(t0, t1), c255x2, magic23x2);
            }
            fb[2 * h] = (uint32_t)f2;
            fb[2 * h + 1] = (uint32_t)(f2 >> 32);
        }
        const uint32_t lo = __byte_perm(fb[0], fb[1], 0x0040), hi = __byte_perm(fb[2], fb[3], 0x0040);
        outw[j] = __byte_perm(lo, hi, 0x5410);
    }
    return make_uint4(outw[0], outw[1], outw[2], outw[3]);
}

template <int MID, bool RES>
__global__ void __launch_bounds__(640, 1)
tc_chain_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB1, const __grid_constant__ CUtensorMap tmB2,
                const __grid_constant__ CUtensorMap tmY, const __grid_constant__ CUtensorMap tmR, const ChainParams p) {
    using Cfg = Tc4Config<MID>;
    constexpr int BK = Cfg::BK;
    constexpr int kStages = Cfg::kStages;
    constexpr int kD1Bufs = Cfg::kD1Bufs;
    constexpr int kBufs = Cfg::kBufs;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);  // stays a shared-memory pointer
    uint8_t* ring = smem;
    uint8_t* ring2 = smem + Cfg::kRing2Offset;
    uint8_t* smem_a2 = smem + Cfg::kA2Offset;
    uint8_t* smem_out = smem + Cfg::kOutOffset;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kBarOffset);
    uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(bars + Cfg::kNumBars);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);
    volatile int* passes_done = reinterpret_cast<volatile int*>(tmem_ptr_smem + 2);  // passes of the second product the epilogue has finished
    float* tab_ms1 = reinterpret_cast<float*>(smem + Cfg::kParamOffset);
    float* tab_bs1 = tab_ms1 + MID;
    float* tab_ms2 = tab_bs1 + MID;
    float* tab_bs2 = tab_ms2 + Cfg::kMaxOut;

    const uint32_t bar_base = smem_u32(bars);
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
    auto d1full_bar = [&](int a) { return bar_base + 8u * (2 * kStages + a); };
    auto d1empty_bar = [&](int a) { return bar_base + 8u * (2 * kStages + 2 + a); };
    auto d2full_bar = [&](int a) { return bar_base + 8u * (2 * kStages + 4 + a); };
    auto d2empty_bar = [&](int a) { return bar_base + 8u * (2 * kStages + 6 + a); };
    auto a2full_bar = [&]() { return bar_base + 8u * (2 * kStages + 8); };
    auto rfull_bar = [&](int b) { return bar_base + 8u * (2 * kStages + 9 + b); };
    auto bfull_bar = [&](int b) { return bar_base + 8u * (2 * kStages + 13 + b); };
    auto bempty_bar = [&](int b) { return bar_base + 8u * (2 * kStages + 17 + b); };
    auto full2_bar = [&](int s) { return bar_base + 8u * (2 * kStages + 21 + s); };
    auto empty2_bar = [&](int s) { return bar_base + 8u * (2 * kStages + 21 + Cfg::kSlots2 + s); };

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint64_t limit = p.wait_limit_ns;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int s = 0; s < Cfg::kSlots2; ++s) {
            mbar_init(full2_bar(s), 1);
            mbar_init(empty2_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(d1full_bar(a), 1);
            mbar_init(d1empty_bar(a), 16);  // one arrival per epilogue warp
            mbar_init(d2full_bar(a), 1);
            mbar_init(d2empty_bar(a), 8);   // the eight epilogue warps of the group that drains this buffer
        }
        mbar_init(a2full_bar(), 16);
        for (int b = 0; b < 4; ++b) {
            mbar_init(rfull_bar(b), 1);
            mbar_init(bfull_bar(b), 8);
            mbar_init(bempty_bar(b), 1);
        }
        *abort_flag = 0;
        *passes_done = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_ptr_smem), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr_smem;
    pdl_launch_dependents();
    pdl_dependency_wait();

    const int pos_tiles = p.tiles_w * p.tiles_h * p.tiles_n;
    const int my_tiles = (int)blockIdx.x < pos_tiles ? (pos_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
    const int passes = (p.out_cols + 127) / 128;
    const int num_kb = p.KH * p.KW * p.c_chunks;
    constexpr int kSub = Cfg::kSub;
    const int num_st = (num_kb + kSub - 1) / kSub;  // stages of the first product per tile
    auto tile_origin = [&](int i, int& w0, int& h0, int& n0) {  // i: index among this CTA's tiles
        int pt = (int)blockIdx.x + i * (int)gridDim.x;
        const int tw = pt % p.tiles_w;
        pt /= p.tiles_w;
        const int th = pt % p.tiles_h;
        const int tn = pt / p.tiles_h;
        w0 = tw * p.Wb; h0 = th * p.Hb; n0 = tn * p.Nb;
    };

    if (warp == 0) {
        // ---------------- TMA producer of the first product ----------------
        // The whole warp walks the loop and waits; the kSub position blocks and the kSub weight blocks of a stage are fetched by 2 kSub
        // lanes of ONE instruction (the weights' map is declared with four dimensions so that both operands take the same instruction
        // form): a thread sustains only one tensor copy per ~400 cycles, whatever the copy's size.
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        const bool wlane = lane >= kSub;                 // this lane fetches weights
        const int sub = wlane ? lane - kSub : lane;      // ... of the stage's sub-th K block
        const CUtensorMap* my_map = wlane ? &tmB1 : &tmA;
        int l_cc = 0, l_kw = 0, l_kh = 0;                // position lanes: (channel chunk, tap column, tap row) of this lane's K block
        auto lane_step = [&]() {
            if (++l_cc == p.c_chunks) {
                l_cc = 0;
                if (++l_kw == p.KW) {
                    l_kw = 0;
                    ++l_kh;
                }
            }
        };
        for (int i = 0; i < my_tiles && ok; ++i) {
            int w0, h0, n0;
            tile_origin(i, w0, h0, n0);
            w0 = w0 * p.sw - p.pad_left;
            h0 = h0 * p.sh - p.pad_top;
            l_cc = 0; l_kw = 0; l_kh = 0;
            for (int j = 0; j < kSub; ++j)
                if (j < sub) lane_step();
            for (int s = 0; s < num_st && ok; ++s) {
                const int kb0 = s * kSub;
                const int nsub = num_kb - kb0 < kSub ? num_kb - kb0 : kSub;
                ok = __all_sync(0xffffffffu, mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status, 1, 0, limit));
                if (!ok) break;
                uint8_t* st = ring + stage * Cfg::kStageBytes;
                if (lane == 0) mbar_expect_tx(full_bar(stage), (uint32_t)(nsub * (Cfg::kStageA + Cfg::kStageB)));
                __syncwarp();
                const uint32_t dst = smem_u32(wlane ? st + kSub * Cfg::kStageA + sub * Cfg::kStageB : st + sub * Cfg::kStageA);
                const int c0 = wlane ? (kb0 + sub) * BK : l_cc * BK;
                const int c1 = wlane ? 0 : w0 + l_kw, c2 = wlane ? 0 : h0 + l_kh, c3 = wlane ? 0 : n0;
                if (lane < 2 * kSub && sub < nsub) tma_load_4d(dst, my_map, full_bar(stage), c0, c1, c2, c3);
#pragma unroll
                for (int j = 0; j < kSub; ++j) lane_step();
                __syncwarp();
                if (++stage == kStages) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA thread of the first product ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            const uint32_t desc_hi = kmajor_desc_hi<BK>();
            const uint32_t ring_lo = kmajor_desc_lo(smem_u32(ring));
#ifdef CHXQ_TL
            int tl_n = 0;
#endif
            for (int i = 0; i < my_tiles && ok; ++i) {
                const int b1 = kD1Bufs == 2 ? (i & 1) : 0;
                const uint32_t use = (uint32_t)(i / kD1Bufs);
                const uint32_t tmem_d = tmem_base + (uint32_t)(b1 * MID);
                // the epilogue has read the accumulators this buffer held before
                if (!mbar_wait(d1empty_bar(b1), (use & 1u) ^ 1u, abort_flag, p.status, 2, 0, limit)) break;
                tc_fence_after();
                CHXQ_TL4(0, 1000, 400);
                for (int s = 0; s < num_st; ++s) {
                    // Pacing.  This product runs up to two tiles ahead of the epilogue and could issue a tile's MMAs in one burst, behind
                    // which the second product's next pass would queue in the tensor pipe while the epilogue warps wait for it.  So stage s
                    // of tile i goes out only once the epilogue has finished the matching share of the passes of tile i - 2.  Only timing
                    // depends on this: after a bounded number of polls the stage is issued anyway.
                    if (i >= 2) {
                        const int target = (i - 2) * passes + (s * passes) / num_st;
                        for (int spin = 0; spin < 4096 && *passes_done < target; ++spin) __nanosleep(64);
                    }
                    if (!mbar_wait(full_bar(stage), phase, abort_flag, p.status, 3, 0, limit)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_lo = ring_lo + (uint32_t)(stage * (Cfg::kStageBytes >> 4));
                    const uint32_t b_lo = a_lo + (uint32_t)((kSub * Cfg::kStageA) >> 4);
                    const int nsub = num_kb - s * kSub < kSub ? num_kb - s * kSub : kSub;
#pragma unroll
                    for (int j = 0; j < kSub; ++j)
                        if (j < nsub) {
#pragma unroll
                            for (int k = 0; k < BK / 32; ++k)
                                umma_i8_lohi(tmem_d, a_lo + (uint32_t)(j * (Cfg::kStageA >> 4) + k * 2), desc_hi, b_lo + (uint32_t)(j * (Cfg::kStageB >> 4) + k * 2),
                                             desc_hi, p.idesc1, (s > 0 || j > 0 || k > 0) ? 1u : 0u);
                        }
                    umma_commit(empty_bar(stage));
                    CHXQ_TL4(0, 1000, 800 + s);
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (ok) umma_commit(d1full_bar(b1));
                CHXQ_TL4(0, 1000, 500);
            }
        }
    } else if (warp == 19) {
        // ---------------- MMA thread of the second product; it also fetches that product's weights ----------------
        // One K block of 128 output channels' weights per slot of the second ring.  A slot is refilled as soon as the MMAs that read it
        // have completed, with the K block kSlots2 blocks ahead: by then the next pass waits for the epilogue anyway.
        if (lane == 0) {
            const uint32_t desc_hi = kmajor_desc_hi<BK>();
            const uint32_t ring2_lo = kmajor_desc_lo(smem_u32(ring2));
            const uint32_t a2_lo = kmajor_desc_lo(smem_u32(smem_a2));
            const int total = my_tiles * passes * Cfg::kChunks2;  // K blocks of this CTA, in order
            int ld_ps = 0, ld_kc = 0, ld_n = 0, ld_slot = 0;
            uint32_t ld_phase = 0;
            bool ok = true;
            // fetches the next K block in order into the next slot (whose previous MMAs must have completed)
            auto load_next = [&]() {
                if (!mbar_wait(empty2_bar(ld_slot), ld_phase ^ 1u, abort_flag, p.status, 15, 0, limit)) {
                    ok = false;
                    return;
                }
                mbar_expect_tx(full2_bar(ld_slot), Cfg::kSlot2);
                tma_load_2d(smem_u32(ring2 + ld_slot * Cfg::kSlot2), &tmB2, full2_bar(ld_slot), ld_kc * BK, ld_ps * 128);
                ++ld_n;
                if (++ld_slot == Cfg::kSlots2) {
                    ld_slot = 0;
                    ld_phase ^= 1u;
                }
                if (++ld_kc == Cfg::kChunks2) {
                    ld_kc = 0;
                    if (++ld_ps == passes) ld_ps = 0;
                }
            };
            for (int n = 0; n < Cfg::kSlots2 && n < total && ok; ++n) load_next();
#ifdef CHXQ_TL
            int tl_n = 0;
#endif
            int slot = 0, g = 0;
            uint32_t phase2 = 0;
            for (int i = 0; i < my_tiles && ok; ++i) {
                // the intermediate tile of this CTA's i-th tile is in shared memory
                if (!mbar_wait(a2full_bar(), (uint32_t)i & 1u, abort_flag, p.status, 11, 0, limit)) break;
                for (int ps = 0; ps < passes && ok; ++ps, ++g) {
                    const int d2 = g & 1;
                    CHXQ_TL4(8192, 1000, 100 + ps);
                    if (!mbar_wait(d2empty_bar(d2), (((uint32_t)g >> 1) & 1u) ^ 1u, abort_flag, p.status, 12, 0, limit)) {
                        ok = false;
                        break;
                    }
                    CHXQ_TL4(8192, 1000, 150 + ps);
                    const uint32_t tmem_d = tmem_base + 256u + (uint32_t)(d2 * 128);
                    for (int kc = 0; kc < Cfg::kChunks2; ++kc) {
                        while (ld_n <= g * Cfg::kChunks2 + kc && ok) load_next();  // (only when a pass has more K blocks than the ring runs ahead)
                        if (!ok) break;
                        if (!mbar_wait(full2_bar(slot), phase2, abort_flag, p.status, 16, 0, limit)) {
                            ok = false;
                            break;
                        }
                        tc_fence_after();
                        const uint32_t a_lo = a2_lo + (uint32_t)(kc * ((128 * BK) >> 4));
                        const uint32_t b_lo = ring2_lo + (uint32_t)(slot * (Cfg::kSlot2 >> 4));
#pragma unroll
                        for (int k = 0; k < BK / 32; ++k) umma_i8_lohi(tmem_d, a_lo + k * 2, desc_hi, b_lo + k * 2, desc_hi, p.idesc2, (kc > 0 || k > 0) ? 1u : 0u);
                        umma_commit(empty2_bar(slot));
                        if (++slot == Cfg::kSlots2) {
                            slot = 0;
                            phase2 ^= 1u;
                        }
                    }
                    if (!ok) break;
                    umma_commit(d2full_bar(d2));
                    CHXQ_TL4(8192, 1000, 300 + ps);
                    // refill the slots whose last readers are the MMAs of EARLIER passes (complete by now): the thread never waits for the
                    // MMAs it has just issued, so the next pass can go out the moment the epilogue hands its accumulator buffer back
                    const int issued = (g + 1) * Cfg::kChunks2;
                    while (ld_n < total && ld_n - Cfg::kSlots2 < issued - Cfg::kChunks2 && ok) load_next();
                    CHXQ_TL4(8192, 1000, 350 + ps);
                }
            }
        }
    } else if (warp < 18) {
        // ---------------- epilogue warps ----------------
        // Warp w reads TMEM lanes 32 * (w % 4) .. + 31 (one position per thread); the four warps of a lane quarter take every
        // fourth 16-channel chunk.
        const int e = warp - 2;  // 0..15
        const int quarter = warp & 3;
        const int sub = e >> 2;
        const int row = quarter * 32 + lane;
        const RequantParams rq1 = p.epi1.rq, rq2 = p.epi2.rq;
        // per-channel multipliers and offsets of both requantizations, once per CTA
        for (int c = e * 32 + lane; c < MID; c += 512) {
            const FoldCh fc = fold_channel(p.epi1.bias ? p.epi1.bias[c] : 0, __fdiv_rn(epi_mult(p.epi1, c), rq1.y_scale), rq1);
            tab_ms1[c] = fc.ms;
            tab_bs1[c] = fc.bs;
        }
        for (int c = e * 32 + lane; c < passes * 128; c += 512) {
            FoldCh fc;
            fc.ms = 0.f;
            fc.bs = 0.f;
            if (c < p.out_cols) fc = fold_channel(p.epi2.bias ? p.epi2.bias[c] : 0, __fdiv_rn(epi_mult(p.epi2, c), rq2.y_scale), rq2);
            tab_ms2[c] = fc.ms;
            tab_bs2[c] = fc.bs;
        }
        asm volatile("bar.sync 1, 512;" ::: "memory");
        const float hi1 = fold_hi_ph(rq1), hi2 = fold_hi_ph(rq2);
        const uint64_t hp1x2 = pack2(hi1, hi1), hp2x2 = pack2(hi2, hi2);
        const uint64_t fr2 = pack2(rq2.fold_r, rq2.fold_r), fc2 = pack2(rq2.fold_c, rq2.fold_c);
        const float fa = rq2.fold_a;
        constexpr int kMine1 = MID / 64;  // 16-channel chunks of the intermediate tile per warp
        // ---- first product: accumulators of this CTA's i-th tile -> the intermediate tile in shared memory
#ifdef CHXQ_TL
        int tl_n = (warp == 2 && lane == 0) ? 0 : 1 << 30;
#endif
        auto first_epilogue = [&](int i) -> bool {
            const int b1 = kD1Bufs == 2 ? (i & 1) : 0;
            const uint32_t use = (uint32_t)(i / kD1Bufs);
            CHXQ_TL4(2048, 1000, 10);
            const bool got = mbar_wait(d1full_bar(b1), use & 1u, abort_flag, p.status, 4, 32, limit);
            if (!__all_sync(0xffffffffu, got)) return false;
            CHXQ_TL4(2048, 1000, 11);
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(b1 * MID);
            uint32_t ra[16], rb[16];
            __syncwarp();
            tmem_ld_32x32b_x16(taddr + (uint32_t)(sub * 16), ra);
#pragma unroll
            for (int j = 0; j < kMine1; ++j) {
                const int ch = j * 4 + sub;
                uint8_t* cell = smem_a2 + (ch * 16 / BK) * (128 * BK) + staged_offset<BK>(row, (ch * 16 % BK) / 16);
                uint4 o;
                if (j & 1) {
                    tmem_ld_wait16(rb);
                    if (j + 1 < kMine1) tmem_ld_32x32b_x16(taddr + (uint32_t)(((j + 1) * 4 + sub) * 16), ra);
                    o = fold_chunk16<false>(rb, tab_ms1 + ch * 16, tab_bs1 + ch * 16, make_uint4(0u, 0u, 0u, 0u), hp1x2, fr2, fc2, fa);
                } else {
                    tmem_ld_wait16(ra);
                    if (j + 1 < kMine1) tmem_ld_32x32b_x16(taddr + (uint32_t)(((j + 1) * 4 + sub) * 16), rb);
                    o = fold_chunk16<false>(ra, tab_ms1 + ch * 16, tab_bs1 + ch * 16, make_uint4(0u, 0u, 0u, 0u), hp1x2, fr2, fc2, fa);
                }
                *reinterpret_cast<uint4*>(cell) = o;
            }
            tc_fence_before();
            fence_async_smem();  // the tile becomes visible to the tensor core's reads
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(d1empty_bar(b1));
                mbar_arrive(a2full_bar());
            }
            CHXQ_TL4(2048, 1000, 12);
            return true;
        };
        // ---- second product: pass ps (128 output channels) of the i-th tile -> staged bytes.  The sixteen warps form two groups of
        // eight (two warps per lane quarter); a pass belongs to the group of its accumulator buffer, whose warps take four 16-channel
        // chunks each.  While one group waits (for its accumulators, for the residual tile, for its tensor-memory loads) the other one
        // works, and a warp passes its barriers once per four chunks.
        const int grp = sub >> 1, sg = sub & 1;
        auto second_epilogue = [&](int i, int ps) -> bool {
            const int g = i * passes + ps;
            const int d2 = g & 1;
            const int buf = g % kBufs;
            const uint32_t buse = (uint32_t)(g / kBufs) & 1u;
            CHXQ_TL4(2048, 1000, 20 + ps);
            bool got = RES ? mbar_wait(rfull_bar(buf), buse, abort_flag, p.status, 6, 32, limit)
                           : mbar_wait(bempty_bar(buf), buse ^ 1u, abort_flag, p.status, 7, 32, limit);
            CHXQ_TL4(2048, 1000, 40 + ps);
            if (got) got = mbar_wait(d2full_bar(d2), (uint32_t)(g >> 1) & 1u, abort_flag, p.status, 13, 32, limit);
            if (!__all_sync(0xffffffffu, got)) return false;
            CHXQ_TL4(2048, 1000, 60 + ps);
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + 256u + (uint32_t)(d2 * 128);
            uint8_t* out_buf = smem_out + buf * Cfg::kTileOut;
            const int col0 = ps * 128;
            uint32_t ra[16], rb[16];
            auto chunk_of = [&](int j) { return sg + 2 * j; };
            auto valid = [&](int j) { return col0 + chunk_of(j) * 16 < p.out_cols; };  // warp-uniform; beyond: clipped by the store
            auto work = [&](uint32_t (&r)[16], int j) {
                const int ch = chunk_of(j);
                uint8_t* cell = out_buf + staged_offset<128>(row, ch);
                uint4 resv = make_uint4(0u, 0u, 0u, 0u);
                if (RES) resv = *reinterpret_cast<const uint4*>(cell);
                *reinterpret_cast<uint4*>(cell) = fold_chunk16<RES>(r, tab_ms2 + col0 + ch * 16, tab_bs2 + col0 + ch * 16, resv, hp2x2, fr2, fc2, fa);
            };
            __syncwarp();
            if (valid(0)) tmem_ld_32x32b_x16(taddr + (uint32_t)(chunk_of(0) * 16), ra);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const bool v = valid(j);
                if (j & 1) {
                    if (v) tmem_ld_wait16(rb);
                    if (j + 1 < 4 && valid(j + 1)) tmem_ld_32x32b_x16(taddr + (uint32_t)(chunk_of(j + 1) * 16), ra);
                    if (v) work(rb, j);
                } else {
                    if (v) tmem_ld_wait16(ra);
                    if (j + 1 < 4 && valid(j + 1)) tmem_ld_32x32b_x16(taddr + (uint32_t)(chunk_of(j + 1) * 16), rb);
                    if (v) work(ra, j);
                }
            }
            tc_fence_before();
            fence_async_smem();  // staged bytes become visible to the TMA store
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(d2empty_bar(d2));
                mbar_arrive(bfull_bar(buf));
                if (sg == 0 && quarter == 0) atomicAdd(const_cast<int*>(passes_done), 1);  // one warp per group keeps the count
            }
            CHXQ_TL4(2048, 1000, 80 + ps);
            return true;
        };
        // Order: the intermediate tile of the NEXT tile is produced before the last pass of this one, so that the tensor core's round
        // trip for the next tile's first pass (wake the MMA thread, run the MMAs, wake the epilogue) hides behind that pass.  The
        // intermediate tile may be overwritten once the last pass's accumulators are complete: every MMA that read it has run.
        bool alive = my_tiles > 0 && first_epilogue(0);
        for (int i = 0; i < my_tiles && alive; ++i) {
            for (int ps = 0; ps < passes && alive; ++ps) {
                const int g = i * passes + ps;
                if (ps == passes - 1 && i + 1 < my_tiles) {
                    // both groups: the last pass's accumulators are complete, so every MMA that read the intermediate tile has run
                    const bool got = mbar_wait(d2full_bar(g & 1), (uint32_t)(g >> 1) & 1u, abort_flag, p.status, 14, 32, limit);
                    if (!__all_sync(0xffffffffu, got)) {
                        alive = false;
                        break;
                    }
                    alive = first_epilogue(i + 1);
                    if (!alive) break;
                }
                if ((g & 1) == grp) alive = second_epilogue(i, ps);
            }
        }
    } else if (warp == 18) {
        // ---------------- store warp: TMA stores of the staged passes, and the loads of the residual tiles ----------------
        if (lane == 0) {
            const int total = my_tiles * passes;
#ifdef CHXQ_TL
            int tl_n = 0;
#endif
            auto residual_load = [&](int g) {
                const int i = g / passes, ps = g - i * passes, b = g % kBufs;
                int w0, h0, n0;
                tile_origin(i, w0, h0, n0);
                mbar_expect_tx(rfull_bar(b), Cfg::kTileOut);
                tma_load_4d(smem_u32(smem_out + b * Cfg::kTileOut), &tmR, rfull_bar(b), ps * 128, w0, h0, n0);
            };
            if (RES)
                for (int g = 0; g < kBufs && g < total; ++g) residual_load(g);
            for (int g = 0; g < total; ++g) {
                const int i = g / passes, ps = g - i * passes, b = g % kBufs;
                CHXQ_TL4(4096, 1000, 1);
                if (!mbar_wait(bfull_bar(b), (uint32_t)(g / kBufs) & 1u, abort_flag, p.status, 8, 0, limit)) break;
                CHXQ_TL4(4096, 1000, 2);
                int w0, h0, n0;
                tile_origin(i, w0, h0, n0);
                tma_store_4d(&tmY, smem_u32(smem_out + b * Cfg::kTileOut), ps * 128, w0, h0, n0);
                tma_store_commit();
                tma_store_wait_read<0>();
                CHXQ_TL4(4096, 1000, 3);
                if (RES) {
                    if (g + kBufs < total) residual_load(g + kBufs);  // the buffer is free: fetch the residual tile of its next use
                } else {
                    mbar_arrive(bempty_bar(b));
                }
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
        tmem_dealloc(tmem_base, 512);
    }
}

template <int MID, bool RES>
int launch_chain_one(const CUtensorMap& tmA, const CUtensorMap& tmB1, const CUtensorMap& tmB2, const CUtensorMap& tmY, const CUtensorMap& tmR,
                     const ChainParams& p, int grid, cudaStream_t s) {
    using Cfg = Tc4Config<MID>;
    if (p.out_cols > Cfg::kMaxOut) return CHXQ_ERR_UNSUPPORTED;
    static std::atomic<bool> attr_set[64] = {};  // per device; host threads may race here, every writer stores true
    int dev = 0;
    CHXQ_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !attr_set[dev].load(std::memory_order_acquire)) {
        CHXQ_CUDA(cudaFuncSetAttribute(tc_chain_kernel<MID, RES>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
        if (dev >= 0 && dev < 64) attr_set[dev].store(true, std::memory_order_release);
    }
    CHXQ_CUDA(launch_pdl(tc_chain_kernel<MID, RES>, grid, Cfg::kThreads, Cfg::kSmemBytes, s, tmA, tmB1, tmB2, tmY, tmR, p));
    count_launch(1);
    return CHXQ_OK;
}

}  // namespace tc
}  // namespace chxq
