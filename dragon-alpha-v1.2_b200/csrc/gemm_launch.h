// Host-side launch interface between the C-ABI layer and the kernel
// instantiations (one translation unit per operand-layout pair, so they build
// in parallel).
#pragma once
#include <cuda_runtime.h>
#include "gemm_tf32.cuh"

namespace dragon {

// Tile configurations: CTAs per tile x columns per tile.  A tile has 128 rows per CTA.
enum TileCfg : int {
  TILE_1x64 = 0,   // 128 x 64, one CTA   (narrow outputs)
  TILE_1x128 = 1,  // 128 x 128, one CTA
  TILE_1x256 = 2,  // 128 x 256, one CTA
  TILE_2x128 = 3,  // 256 x 128, CTA pair
  TILE_2x256 = 4,  // 256 x 256, CTA pair
  // "T" tiles feed the A operand to the tensor core through TMEM (FP32-accurate mode only)
  TILE_2x192T = 5, // 256 x 192, CTA pair
  TILE_1x64T = 6,  // 128 x 64, one CTA
  TILE_1x128T = 7, // 128 x 128, one CTA
  TILE_2x64 = 8,   // 256 x 64, CTA pair (narrow outputs: halves the MMA instructions per row)
  TILE_COUNT = 9
};

inline int tile_ctas(int cfg) { return (cfg == TILE_2x128 || cfg == TILE_2x256 || cfg == TILE_2x192T || cfg == TILE_2x64) ? 2 : 1; }
inline bool tile_is_ts(int cfg) { return cfg >= TILE_2x192T && cfg <= TILE_1x128T; }
inline int tile_bn(int cfg) {
  switch (cfg) {
    case TILE_1x64: case TILE_1x64T: case TILE_2x64: return 64;
    case TILE_1x128: case TILE_2x128: case TILE_1x128T: return 128;
    case TILE_2x192T: return 192;
    default: return 256;
  }
}

// Operand layouts.  "K" = the reduction axis is contiguous in memory, "N" = the
// row/column (M or N) axis is contiguous.
//   KK : A[M][K], B[N][K]   (matMulT2, batchMatMulT2, convolution with OCxFHxFWxIC filters)
//   KN : A[M][K], B[K][N]   (matMul, batchMatMul)
//   NN : A[K][M], B[K][N]   (matMulT1, batchMatMulT1)
cudaError_t launch_gemm_kk(int tile_cfg, bool x3, bool im2col, const GemmParams& p, int grid_z,
                           cudaStream_t stream);
cudaError_t launch_gemm_kn(int tile_cfg, bool x3, bool im2col, const GemmParams& p, int grid_z,
                           cudaStream_t stream);
cudaError_t launch_gemm_nn(int tile_cfg, bool x3, const GemmParams& p, int grid_z, cudaStream_t stream);
//   NN + im2col : A[K][M], B = im2col walk over an NHWC image, K = output pixels (weight gradient; FP32-accurate only)
cudaError_t launch_gemm_nn_im2col(int tile_cfg, const GemmParams& p, int grid_z, cudaStream_t stream);

// Shared-memory bytes one stage of the given configuration uses (for reporting).
int gemm_stage_bytes(int tile_cfg, bool x3);
int gemm_stages(int tile_cfg, bool x3);

template <class Cfg>
cudaError_t launch_one(const GemmParams& p, int grid_z, cudaStream_t stream) {
  auto kernel = gemm_tf32_kernel<Cfg>;
  // Once per device: opt in to the large dynamic shared-memory carve-out and ask how many
  // CTAs (or CTA pairs) of this kernel can be resident at the same time - the persistent
  // grid must not exceed that, or the surplus CTAs would run after the others have finished.
  static int resident_units[64];  // per device ordinal; 0 = not configured yet
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  int units = __atomic_load_n(&resident_units[dev & 63], __ATOMIC_ACQUIRE);
  if (units == 0) {
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::DYN_SMEM);
    if (e != cudaSuccess) return e;
    if (Cfg::CTAS == 2) {
      cudaLaunchConfig_t q = {};
      q.gridDim = dim3(2 * 148, 1, 1);
      q.blockDim = dim3(Cfg::THREADS, 1, 1);
      q.dynamicSmemBytes = Cfg::DYN_SMEM;
      cudaLaunchAttribute qa[1];
      qa[0].id = cudaLaunchAttributeClusterDimension;
      qa[0].val.clusterDim.x = 2;
      qa[0].val.clusterDim.y = 1;
      qa[0].val.clusterDim.z = 1;
      q.attrs = qa;
      q.numAttrs = 1;
      e = cudaOccupancyMaxActiveClusters(&units, kernel, &q);
      if (e != cudaSuccess) return e;
    } else {
      int sms = 0, per_sm = 0;
      e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
      if (e != cudaSuccess) return e;
      e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, Cfg::THREADS, Cfg::DYN_SMEM);
      if (e != cudaSuccess) return e;
      units = sms * per_sm;
    }
    if (units < 1) return cudaErrorLaunchOutOfResources;
    __atomic_store_n(&resident_units[dev & 63], units, __ATOMIC_RELEASE);
  }
  const long long total_tiles = static_cast<long long>(p.tiles_m) * p.tiles_n * grid_z;
  const long long grid_units = total_tiles < units ? total_tiles : units;
  GemmParams q = p;
  q.zcount = grid_z;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid_units) * Cfg::CTAS, 1, 1);
  cfg.blockDim = dim3(Cfg::THREADS, 1, 1);
  cfg.dynamicSmemBytes = Cfg::DYN_SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  cfg.numAttrs = 0;
  if (Cfg::CTAS == 2) {
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  return cudaLaunchKernelEx(&cfg, kernel, q);
}

// Expands to the switch over tile configurations for one layout pair.
#define DRAGON_DISPATCH_TILES(A_MN, B_MN, X3, IM2COL)                                          \
  switch (tile_cfg) {                                                                          \
    case TILE_1x64:  return launch_one<GemmCfg<64, 1, A_MN, B_MN, X3, IM2COL>>(p, grid_z, stream);  \
    case TILE_1x128: return launch_one<GemmCfg<128, 1, A_MN, B_MN, X3, IM2COL>>(p, grid_z, stream); \
    case TILE_1x256: return launch_one<GemmCfg<256, 1, A_MN, B_MN, X3, IM2COL>>(p, grid_z, stream); \
    case TILE_2x128: return launch_one<GemmCfg<128, 2, A_MN, B_MN, X3, IM2COL>>(p, grid_z, stream); \
    case TILE_2x256: return launch_one<GemmCfg<256, 2, A_MN, B_MN, X3, IM2COL>>(p, grid_z, stream); \
    case TILE_2x192T: return launch_one<GemmCfg<192, 2, A_MN, B_MN, true, IM2COL, true>>(p, grid_z, stream); \
    case TILE_1x64T:  return launch_one<GemmCfg<64, 1, A_MN, B_MN, true, IM2COL, true>>(p, grid_z, stream);  \
    case TILE_1x128T: return launch_one<GemmCfg<128, 1, A_MN, B_MN, true, IM2COL, true>>(p, grid_z, stream); \
    case TILE_2x64:  return launch_one<GemmCfg<64, 2, A_MN, B_MN, X3, IM2COL>>(p, grid_z, stream);  \
    default: return cudaErrorInvalidValue;                                                     \
  }

}  // namespace dragon
