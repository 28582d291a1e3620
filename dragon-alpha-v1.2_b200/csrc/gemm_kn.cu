// Kernel instantiations for A[M][K] x B[K][N]: matMul and batchMatMul, and - with the A rows
// gathered by an im2col-mode tensor map - the data gradient of the stride-1 convolution, whose
// filter is read in place as [K = OC][N = IC] matrices, one per tap.
#include "gemm_launch.h"

namespace dragon {

cudaError_t launch_gemm_kn(int tile_cfg, bool x3, bool im2col, const GemmParams& p, int grid_z,
                           cudaStream_t stream) {
  if (im2col) {
    if (!x3) return cudaErrorInvalidValue;   // the gradient entry points are FP32-accurate only
    DRAGON_DISPATCH_TILES(false, true, true, true)
  }
  if (x3) { DRAGON_DISPATCH_TILES(false, true, true, false) }
  else    { DRAGON_DISPATCH_TILES(false, true, false, false) }
}

}  // namespace dragon
