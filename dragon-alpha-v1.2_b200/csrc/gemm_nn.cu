// Kernel instantiations for A[K][M] x B[K][N]: matMulT1 and batchMatMulT1.
#include "gemm_launch.h"

namespace dragon {

cudaError_t launch_gemm_nn(int tile_cfg, bool x3, const GemmParams& p, int grid_z, cudaStream_t stream) {
  if (x3) { DRAGON_DISPATCH_TILES(true, true, true, false) }
  else    { DRAGON_DISPATCH_TILES(true, true, false, false) }
}

}  // namespace dragon
