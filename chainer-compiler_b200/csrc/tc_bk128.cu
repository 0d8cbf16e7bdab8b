// Instantiations of the tcgen05 implicit-GEMM kernel for a 128-byte K tile (swizzle 128B).
#include "tc_kernel.cuh"

namespace chxq {
namespace tc {

int launch_tc_bk128(int bn, int epi, const CUtensorMap& tmA, const CUtensorMap& tmB, const TcParams& p, int grid, cudaStream_t s) {
    return launch_bk<128>(bn, epi, tmA, tmB, p, grid, s);
}

}  // namespace tc
}  // namespace chxq
