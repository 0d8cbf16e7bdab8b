// Instantiations of the tcgen05 implicit-GEMM kernel for a 32-byte K tile (swizzle 32B).
#include "tc_kernel.cuh"

namespace chxq {
namespace tc {

int launch_tc_bk32(int bn, int epi, const CUtensorMap& tmA, const CUtensorMap& tmB, const TcParams& p, int grid, cudaStream_t s) {
    return launch_bk<32>(bn, epi, tmA, tmB, p, grid, s);
}

}  // namespace tc
}  // namespace chxq
