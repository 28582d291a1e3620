// Kernel instantiations for A[K][M] x im2col(B): the convolution's weight gradient
// deltaW[OC][tap][IC] = sum over output pixels of deltaY[pixel][OC]^T * X[pixel shifted by tap][IC].
#include "gemm_launch.h"

namespace dragon {

cudaError_t launch_gemm_nn_im2col(int tile_cfg, const GemmParams& p, int grid_z, cudaStream_t stream) {
  switch (tile_cfg) {
    case TILE_1x64:  return launch_one<GemmCfg<64, 1, true, true, true, true>>(p, grid_z, stream);
    case TILE_1x128: return launch_one<GemmCfg<128, 1, true, true, true, true>>(p, grid_z, stream);
    case TILE_1x256: return launch_one<GemmCfg<256, 1, true, true, true, true>>(p, grid_z, stream);
    case TILE_2x128: return launch_one<GemmCfg<128, 2, true, true, true, true>>(p, grid_z, stream);
    case TILE_2x256: return launch_one<GemmCfg<256, 2, true, true, true, true>>(p, grid_z, stream);
    case TILE_2x64:  return launch_one<GemmCfg<64, 2, true, true, true, true>>(p, grid_z, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace dragon
