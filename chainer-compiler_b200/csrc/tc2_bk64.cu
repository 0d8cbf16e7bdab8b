// Instantiations of the grouped-tile tcgen05 kernel for a 64-byte K tile.
#include "tc_kernel2.cuh"

namespace chxq {
namespace tc {

int launch_tc2_bk64(int bn, int epi, bool res, bool halo, const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmY, const CUtensorMap& tmR,
                    const TcParams& p, int grid, cudaStream_t s) {
    return launch_bk2<64>(bn, epi, res, halo, tmA, tmB, tmY, tmR, p, grid, s);
}

}  // namespace tc
}  // namespace chxq
