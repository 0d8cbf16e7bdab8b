// Instantiations of the grouped-tile tcgen05 kernel for a 64-byte K tile.
#include "tc_kernel2.cuh"

namespace chxq {
namespace tc {

int launch_tc2_bk64(int bn, int epi, bool res, bool halo, const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmY, const CUtensorMap& tmR,
                    const TcParams& p, int grid, cudaStream_t s) {
    return launch_bk2<64>(bn, epi, res, halo, tmA, tmB, tmY, tmR, p, grid, s);
}

int launch_tc2_bk64_pool(int epi, bool halo, const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmY, const CUtensorMap& tmR, const TcParams& p,
                         int grid, cudaStream_t s) {
    if (halo) {
        if (epi == kEpiKU8Fold) return launch_one2<64, 64, kEpiKU8Fold, false, true, true>(tmA, tmB, tmY, tmR, p, grid, s);
        if (epi == kEpiKU8) return launch_one2<64, 64, kEpiKU8, false, true, true>(tmA, tmB, tmY, tmR, p, grid, s);
        return CHXQ_ERR_UNSUPPORTED;
    }
    if (epi == kEpiKU8Fold) return launch_one2<64, 64, kEpiKU8Fold, false, false, true>(tmA, tmB, tmY, tmR, p, grid, s);
    if (epi == kEpiKU8) return launch_one2<64, 64, kEpiKU8, false, false, true>(tmA, tmB, tmY, tmR, p, grid, s);
    return CHXQ_ERR_UNSUPPORTED;
}

}  // namespace tc
}  // namespace chxq
