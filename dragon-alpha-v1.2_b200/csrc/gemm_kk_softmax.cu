// Kernel instantiation for the fused attention scores: P = softmax_rows(alpha * A * B^T) with A[M][K], B[N][K]
// (the batchMatMulT2 layout), rows of at most 512 columns normalised inside the SM before they are stored.
#include "gemm_launch.h"

namespace dragon {

cudaError_t launch_gemm_kk_softmax(const GemmParams& p, int grid_z, cudaStream_t stream) {
  return launch_one<GemmCfg<256, 2, false, false, true, false, true>>(p, grid_z, stream);
}

}  // namespace dragon
