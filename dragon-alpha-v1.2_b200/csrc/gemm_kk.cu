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

template <int BN, int CTAS> static int stage_bytes_of(bool x3) {
  return x3 ? GemmCfg<BN, CTAS, false, false, true>::STAGE_BYTES
            : GemmCfg<BN, CTAS, false, false, false>::STAGE_BYTES;
}
template <int BN, int CTAS> static int stages_of(bool x3) {
  return x3 ? GemmCfg<BN, CTAS, false, false, true>::STAGES
            : GemmCfg<BN, CTAS, false, false, false>::STAGES;
}
int gemm_stage_bytes(int tile_cfg, bool x3) {
  switch (tile_cfg) {
    case TILE_1x64: return stage_bytes_of<64, 1>(x3);
    case TILE_1x128: return stage_bytes_of<128, 1>(x3);
    case TILE_1x256: return stage_bytes_of<256, 1>(x3);
    case TILE_2x128: return stage_bytes_of<128, 2>(x3);
    case TILE_2x256: return stage_bytes_of<256, 2>(x3);
    case TILE_2x64: return stage_bytes_of<64, 2>(x3);
    case TILE_2x192T: return GemmCfg<192, 2, false, false, true, false, true>::STAGE_BYTES;
    case TILE_1x64T: return GemmCfg<64, 1, false, false, true, false, true>::STAGE_BYTES;
    case TILE_1x128T: return GemmCfg<128, 1, false, false, true, false, true>::STAGE_BYTES;
    default: return 0;
  }
}
int gemm_stages(int tile_cfg, bool x3) {
  switch (tile_cfg) {
    case TILE_1x64: return stages_of<64, 1>(x3);
    case TILE_1x128: return stages_of<128, 1>(x3);
    case TILE_1x256: return stages_of<256, 1>(x3);
    case TILE_2x128: return stages_of<128, 2>(x3);
    case TILE_2x256: return stages_of<256, 2>(x3);
    case TILE_2x64: return stages_of<64, 2>(x3);
    case TILE_2x192T: return GemmCfg<192, 2, false, false, true, false, true>::STAGES;
    case TILE_1x64T: return GemmCfg<64, 1, false, false, true, false, true>::STAGES;
    case TILE_1x128T: return GemmCfg<128, 1, false, false, true, false, true>::STAGES;
    default: return 0;
  }
}

}  // namespace dragon
