// Kernel instantiations for A[M][K] x B[N][K] (both operands reduction-contiguous):
// matMulT2, batchMatMulT2, and the implicit-GEMM convolution, whose A rows are
// gathered from the NHWC feature map by an im2col-mode tensor map.
#include "gemm_launch.h"

namespace dragon {

cudaError_t launch_gemm_kk(int tile_cfg, bool x3, bool im2col, const GemmParams& p, int grid_z,
                           cudaStream_t stream) {
  if (im2col) {
    if (x3) { DRAGON_DISPATCH_TILES(false, false, true, true) }
    else    { DRAGON_DISPATCH_TILES(false, false, false, true) }
  } else {
    if (x3) { DRAGON_DISPATCH_TILES(false, false, true, false) }
    else    { DRAGON_DISPATCH_TILES(false, false, false, false) }
  }
}

}  // namespace dragon
