// Instantiations of the CTA-pair tcgen05 kernel (cta_group::2, 256 positions x 256 channels per pair) for a 128-byte K tile.
#include "tc_kernel3.cuh"

namespace chxq {
namespace tc {

int launch_tc3_bk128(int epi, bool res, const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmY, const CUtensorMap& tmR, const TcParams& p,
                     int items, cudaStream_t s) {
    return launch_bk3<128>(epi, res, tmA, tmB, tmY, tmR, p, items, s);
}

int tc3_pair_slots(int* out) {
    return pair_slots<128, kEpiKU8Fold, false>(out);
}

}  // namespace tc
}  // namespace chxq
