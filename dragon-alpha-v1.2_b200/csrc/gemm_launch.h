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
  TILE_2x64 = 5,   // 256 x 64, CTA pair (narrow outputs: halves the MMA instructions per row)
  TILE_COUNT = 6
};

inline int tile_ctas(int cfg) { return (cfg == TILE_2x128 || cfg == TILE_2x256 || cfg == TILE_2x64) ? 2 : 1; }
inline int tile_bn(int cfg) {
  switch (cfg) {
    case TILE_1x64: case TILE_2x64: return 64;
    case TILE_1x128: case TILE_2x128: return 128;
    default: return 256;
  }
}
// Bytes one k-block of the tile brings into a CTA (one slot of the raw ring, and of the lo ring).
inline int tile_slot_bytes(int cfg) { return (128 + tile_bn(cfg) / tile_ctas(cfg)) * 32 * 4; }

// Streaming multiprocessors of the current device (cached per device ordinal).
inline int device_sm_count() {
  static int cache[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 1;
  int n = __atomic_load_n(&cache[dev & 63], __ATOMIC_ACQUIRE);
  if (n > 0) return n;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n < 1) n = 1;
  __atomic_store_n(&cache[dev & 63], n, __ATOMIC_RELEASE);
  return n;
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
//   KK + row softmax : P = softmax_rows(alpha * A * B^T), at most 512 columns, reduction of at most kc k-blocks
cudaError_t launch_gemm_kk_softmax(const GemmParams& p, int grid_z, cudaStream_t stream);
// output kept in further copies: A[M][K] x B[K][N] (b_mn) or A[M][K] x B[N][K]^T, 256x256 pair tile, FP32-accurate
cudaError_t launch_gemm_rep(bool b_mn, const GemmParams& p, int grid_z, cudaStream_t stream);
//   NN + im2col : A[K][M], B = im2col walk over an NHWC image, K = output pixels (weight gradient; FP32-accurate only)
cudaError_t launch_gemm_nn_im2col(int tile_cfg, const GemmParams& p, int grid_z, cudaStream_t stream);

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
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::MAX_DYN_SMEM);
    if (e != cudaSuccess) return e;
    const int sms = device_sm_count();
    if (Cfg::CTAS == 2) {
      cudaLaunchConfig_t q = {};
      q.gridDim = dim3(2 * sms, 1, 1);
      q.blockDim = dim3(Cfg::THREADS, 1, 1);
      q.dynamicSmemBytes = Cfg::MAX_DYN_SMEM;
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
      int per_sm = 0;
      e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, Cfg::THREADS, Cfg::MAX_DYN_SMEM);
      if (e != cudaSuccess) return e;
      units = sms * per_sm;
    }
    if (units < 1) return cudaErrorLaunchOutOfResources;
    __atomic_store_n(&resident_units[dev & 63], units, __ATOMIC_RELEASE);
  }
  GemmParams q = p;
  q.zcount = grid_z;
  if (q.unit_tiles < 1) q.unit_tiles = 1;
  // work units: tiles, or (softmax mode) groups of unit_tiles tiles that one CTA pair takes in a row
  const long long total_tiles = static_cast<long long>(p.tiles_m) * p.tiles_n * grid_z / (Cfg::SOFTMAX ? q.unit_tiles : 1);
  // a host that runs a collective beside the contraction can keep some SMs out of the persistent grid
  int usable = units - (q.sm_reserve > 0 ? (q.sm_reserve + Cfg::CTAS - 1) / Cfg::CTAS : 0);
  if (usable < 1) usable = 1;
  const long long grid_units = total_tiles < usable ? total_tiles : usable;
  // Rings: 0 = the balanced default (as many raw + lo pairs as fit beside one staging tile per drain warp).
  if (q.ring_raw == 0) { q.ring_raw = Cfg::STAGES; q.ring_lo = Cfg::STAGES; }
  if (q.store_bufs == 0) q.store_bufs = 1;
  if (!Cfg::X3) q.ring_lo = q.ring_raw;
  q.ring_fixed = 0;
  if (p.ring_fixed) {
    if (q.ring_raw == Cfg::STAGES && q.ring_lo == Cfg::STAGES && q.store_bufs == 1 && (!Cfg::X3 || q.ring_paired) &&
        !Cfg::SOFTMAX)
      q.ring_fixed = 1;
    else if (Cfg::ALT_RAW > 0 && q.ring_raw == Cfg::ALT_RAW && q.ring_lo == Cfg::ALT_LO && q.store_bufs == Cfg::ALT_BUFS)
      q.ring_fixed = 2;
  }
  if (q.ring_raw < 2 || q.ring_raw > Cfg::MAX_RING || q.ring_lo < 1 || q.ring_lo > q.ring_raw ||
      q.store_bufs < 1 || q.store_bufs > 2 || Cfg::dyn_smem(q.ring_raw, q.ring_lo, q.store_bufs) > Cfg::MAX_DYN_SMEM)
    return cudaErrorInvalidValue;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid_units) * Cfg::CTAS, 1, 1);
  cfg.blockDim = dim3(Cfg::THREADS, 1, 1);
  cfg.dynamicSmemBytes = Cfg::dyn_smem(q.ring_raw, q.ring_lo, q.store_bufs);
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  cfg.attrs = attr;
  cfg.numAttrs = 0;
  if (Cfg::CTAS == 2) {
    attr[cfg.numAttrs].id = cudaLaunchAttributeClusterDimension;
    attr[cfg.numAttrs].val.clusterDim.x = 2;
    attr[cfg.numAttrs].val.clusterDim.y = 1;
    attr[cfg.numAttrs].val.clusterDim.z = 1;
    ++cfg.numAttrs;
  }
  if (q.overlap_prev) {   // programmatic dependent launch without a dependency: pure overlap with the previous launch
    attr[cfg.numAttrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[cfg.numAttrs].val.programmaticStreamSerializationAllowed = 1;
    ++cfg.numAttrs;
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
    case TILE_2x64:  return launch_one<GemmCfg<64, 2, A_MN, B_MN, X3, IM2COL>>(p, grid_z, stream);  \
    default: return cudaErrorInvalidValue;                                                     \
  }

}  // namespace dragon
