// Kernel instantiations for A[M][K] x B[K][N]: matMul and batchMatMul.
#include "gemm_launch.h"

namespace dragon {

cudaError_t launch_gemm_kn(int tile_cfg, bool x3, const GemmParams& p, int grid_z, cudaStream_t stream) {
  if (x3) { DRAGON_DISPATCH_TILES(false, true, true, false) }
  else    { DRAGON_DISPATCH_TILES(false, true, false, false) }
}

}  // namespace dragon
