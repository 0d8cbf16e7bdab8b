// Instantiations of the two-convolution tcgen05 kernel (tc_kernel4.cuh).
#include "tc_kernel4.cuh"

namespace chxq {
namespace tc {

int launch_tc_chain(int mid, bool res, const CUtensorMap& tmA, const CUtensorMap& tmB1, const CUtensorMap& tmB2, const CUtensorMap& tmY,
                    const CUtensorMap& tmR, const ChainParams& p, int grid, cudaStream_t s) {
    switch (mid * 2 + (res ? 1 : 0)) {
        case 128: return launch_chain_one<64, false>(tmA, tmB1, tmB2, tmY, tmR, p, grid, s);
        case 129: return launch_chain_one<64, true>(tmA, tmB1, tmB2, tmY, tmR, p, grid, s);
        case 256: return launch_chain_one<128, false>(tmA, tmB1, tmB2, tmY, tmR, p, grid, s);
        case 257: return launch_chain_one<128, true>(tmA, tmB1, tmB2, tmY, tmR, p, grid, s);
        case 512: return launch_chain_one<256, false>(tmA, tmB1, tmB2, tmY, tmR, p, grid, s);
        case 513: return launch_chain_one<256, true>(tmA, tmB1, tmB2, tmY, tmR, p, grid, s);
    }
    return CHXQ_ERR_UNSUPPORTED;
}

}  // namespace tc
}  // namespace chxq
