// Kernel instantiations for the products whose output is also kept in further copies (the row-sharded matMul
// forms reassembled by the kernel's own stores): A[M][K] x B[K][N] and A[M][K] x B[N][K]^T on the 256x256 pair
// tile, FP32-accurate.  Only these carry the code that writes the copies.
#include "gemm_launch.h"

namespace dragon {

cudaError_t launch_gemm_rep(bool b_mn, const GemmParams& p, int grid_z, cudaStream_t stream) {
  if (b_mn) return launch_one<GemmCfg<256, 2, false, true, true, false, false, true>>(p, grid_z, stream);
  return launch_one<GemmCfg<256, 2, false, false, true, false, false, true>>(p, grid_z, stream);
}

}  // namespace dragon
