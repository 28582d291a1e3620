// C-ABI layer of libdragon_cu32.so: argument checking, mapping of the reference's
// (N, M, K, pitch) conventions onto the contraction kernel, tensor-map encoding, and
// the two bandwidth kernels of the path (split-K buffer summation, filter remode).
//
// Nothing here allocates device memory or keeps state between calls apart from
// process-wide tuning integers; tensor maps are encoded on the host per call and
// travel to the kernel as launch parameters.
#include <cuda.h>
#include <cuda_runtime.h>
#include <atomic>
#include <vector>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "../../include/dragon_cu32.h"
#include "gemm_launch.h"

namespace dragon {

// ------------------------------------------------------------------ tuning knobs
static std::atomic<int> g_kc{2};
static std::atomic<int> g_kc_fast{4};
static std::atomic<int> g_tile{-1};
static std::atomic<int> g_l2hint{0};
static std::atomic<int> g_ring_raw{0};        // 0 = chosen per call (see choose_rings)
static std::atomic<int> g_ring_lo{0};
static std::atomic<int> g_store_bufs{0};
static std::atomic<int> g_arrive_release{0};
static std::atomic<int> g_sm_reserve{0};
static std::atomic<int> g_force_gather{0};
static std::atomic<int> g_phase_overlap{1};
static std::atomic<int> g_rep_lazy{1};
static std::atomic<int> g_ring_paired{1};
static std::atomic<int> g_ring_fixed{1};
static std::atomic<int> g_phase_fused{1};

static void load_env_once() {
  static std::once_flag once;
  std::call_once(once, [] {
    if (const char* s = std::getenv("DRAGON_CU32_KC")) { int v = std::atoi(s); if (v >= 1) g_kc = v; }
    if (const char* s = std::getenv("DRAGON_CU32_KC_FAST")) { int v = std::atoi(s); if (v >= 1) g_kc_fast = v; }
    if (const char* s = std::getenv("DRAGON_CU32_L2HINT")) { int v = std::atoi(s); if (v >= 0 && v <= 2) g_l2hint = v; }
    if (const char* s = std::getenv("DRAGON_CU32_TILE")) { int v = std::atoi(s); if (v >= -1 && v < TILE_COUNT) g_tile = v; }
    if (const char* s = std::getenv("DRAGON_CU32_RING_RAW")) { int v = std::atoi(s); if (v >= 0 && v <= 8) g_ring_raw = v; }
    if (const char* s = std::getenv("DRAGON_CU32_RING_LO")) { int v = std::atoi(s); if (v >= 0 && v <= 8) g_ring_lo = v; }
    if (const char* s = std::getenv("DRAGON_CU32_STORE_BUFS")) { int v = std::atoi(s); if (v >= 0 && v <= 2) g_store_bufs = v; }
  });
}

// ------------------------------------------------------------------ device status word
__device__ int g_status_word;

static int* status_word_ptr(cudaError_t* err) {
  // The symbol has one instance per device; cache its address per device ordinal.
  static std::atomic<int*> cache[64];
  int dev = 0;
  *err = cudaGetDevice(&dev);
  if (*err != cudaSuccess) return nullptr;
  int* p = cache[dev & 63].load(std::memory_order_acquire);
  if (p) return p;
  void* sym = nullptr;
  *err = cudaGetSymbolAddress(&sym, g_status_word);
  if (*err != cudaSuccess) return nullptr;
  cache[dev & 63].store(static_cast<int*>(sym), std::memory_order_release);
  return static_cast<int*>(sym);
}

// Clock accumulator of the contraction kernel: {SM cycles, nanoseconds, launches} (see GemmParams::clock_acc).
__device__ unsigned long long g_clock_acc[4];
static std::atomic<int> g_clock_on{0};
static std::atomic<int> g_last_tile{-1};

static unsigned long long* clock_acc_ptr() {
  if (!g_clock_on.load()) return nullptr;
  static std::atomic<unsigned long long*> cache[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
  unsigned long long* p = cache[dev & 63].load(std::memory_order_acquire);
  if (p) return p;
  void* sym = nullptr;
  if (cudaGetSymbolAddress(&sym, g_clock_acc) != cudaSuccess) return nullptr;
  cache[dev & 63].store(static_cast<unsigned long long*>(sym), std::memory_order_release);
  return static_cast<unsigned long long*>(sym);
}

// ------------------------------------------------------------------ tensor maps
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
typedef CUresult (*EncodeIm2colFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const int*, const int*,
                                   cuuint32_t, cuuint32_t, const cuuint32_t*,
                                   CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode_tiled = nullptr;
static EncodeIm2colFn g_encode_im2col = nullptr;

static bool load_driver_entry_points() {
  static std::once_flag once;
  std::call_once(once, [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      g_encode_tiled = reinterpret_cast<EncodeTiledFn>(fn);
    fn = nullptr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &fn, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      g_encode_im2col = reinterpret_cast<EncodeIm2colFn>(fn);
  });
  return g_encode_tiled != nullptr;
}

// 3-D FP32 map (inner, outer, batch), zero fill outside the extents.  K-major operands
// (reduction axis innermost) use the plain 128-byte swizzle; MN-major operands use the
// 128-byte swizzle with 32-byte units, the only one the tensor core reads for 32-bit
// MN-major tiles.
static int make_map3(CUtensorMap* m, const float* base, uint64_t d0, uint64_t d1, uint64_t d2,
                     uint64_t pitch1_floats, uint64_t pitch2_floats, uint32_t b0, uint32_t b1,
                     bool mn_major) {
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {pitch1_floats * 4, pitch2_floats * 4};
  cuuint32_t box[3] = {b0, b1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = g_encode_tiled(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), dims,
                              strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? CU32_OK : CU32_E_TENSORMAP;
}

// One contraction, BLAS letters: C[M,N] = A * B over K.
struct GemmCall {
  const float* A; const float* B; float* C; float* Cbuf;
  int M, N, K;              // logical extents of the operands
  int n_store;              // columns of C written (>= N; columns N.. come out 0)
  long long lda, ldb, ldc;  // row pitches in floats
  bool a_mn, b_mn;          // operand stored with its M / N axis contiguous
  int batch; long long sA, sB, sC;
  int gz;                   // split-K slices (1 = none)
  bool x3;                  // FP32-accurate (true) or single-pass TF32
  cudaStream_t stream;
  const float* bias;        // optional row vector (n_store floats) added in the epilogue; needs gz == 1, batch == 1
  int bias_width;           // true width of the rows: columns beyond it are stored as zeros
  bool scale_on = false;   // store alpha * result (one rounding), vector store paths only
  float alpha = 1.0f;
  float* const* replicas = nullptr;   // further output buffers that receive the same stores as C (same layout)
  int n_replicas = 0;
};

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Tile choice: estimated time = waves over the SMs x work per CTA / measured per-CTA
// rate.  The rates are FP32-accurate TFLOP/s measured at 8192^3 on a B200 with every SM
// busy; padded rows and columns count as work, so narrow outputs pick narrow tiles and
// small problems pick small tiles.
static int pick_tile_auto(long long M, int N, long long z) {
  // measured matMul 8192^3 rates per tile shape, TFLOP/s (order of the TileCfg enum)
  static const double rate[TILE_COUNT] = {118.0, 170.0, 190.0, 206.0, 278.0, 105.0};
  const double sms = static_cast<double>(device_sm_count());
  int best = TILE_1x128;
  double best_t = 1e300;
  for (int t = 0; t < TILE_COUNT; ++t) {
    const int ctas = tile_ctas(t), bn = tile_bn(t);
    const double n_cta = static_cast<double>((M + 128 * ctas - 1) / (128 * ctas)) * ((N + bn - 1) / bn) * ctas * z;
    const double waves = static_cast<double>(static_cast<long long>((n_cta + sms - 1.0) / sms));
    const double time = waves * (128.0 * bn) / rate[t];
    if (time < best_t) { best_t = time; best = t; }
  }
  return best;
}
// The tile a call uses: the forced one if a tuning key set it, else the estimate's; remembered for diagnostics.
static int note_tile(int t) { g_last_tile = t; return t; }
static int pick_tile(long long M, int N, long long z) {
  const int forced = g_tile.load();
  return note_tile(forced >= 0 ? forced : pick_tile_auto(M, N, z));
}

// Ring lengths for a launch (see GemmParams): explicit tuning values win, otherwise 0 = the kernel
// configuration's balanced default.
// Also sets how many chunks are summed in registers between flushes to memory: 256 k-blocks (K = 8192).
static void choose_rings(GemmParams* p) {
  p->flush_chunks = 256 / p->kc > 1 ? 256 / p->kc : 1;
  p->ring_raw = g_ring_raw.load();
  p->ring_lo = g_ring_lo.load();
  p->store_bufs = g_store_bufs.load();
  if (p->ring_raw > 0 && p->ring_lo == 0) p->ring_lo = p->ring_raw;
  if (p->ring_raw == 0) p->ring_lo = 0;
  p->arrive_release = g_arrive_release.load();
  p->ring_paired = g_ring_paired.load();
  p->ring_fixed = g_ring_fixed.load();   // allowed; the launcher decides whether the rings are the default ones
  p->sm_reserve = g_sm_reserve.load();
  p->clock_acc = clock_acc_ptr();
}

static int run_gemm(const GemmCall& c) {
  load_env_once();
  if (!c.A || !c.B || !c.C) return CU32_E_NULL;
  if (c.gz > 1 && !c.Cbuf) return CU32_E_NULL;
  if (c.M <= 0 || c.N <= 0 || c.K <= 0 || c.batch <= 0 || c.gz < 1 || c.gz > 65535) return CU32_E_DIM;
  if ((c.lda & 3) || (c.ldb & 3) || (c.sA & 3) || (c.sB & 3) || !aligned16(c.A) || !aligned16(c.B))
    return CU32_E_ALIGN;
  if (c.bias) {
    if (c.gz != 1 || c.batch != 1) return CU32_E_ARG;
    if (c.bias_width <= 0 || c.bias_width > c.n_store) return CU32_E_DIM;
    if (!aligned16(c.bias) || (c.n_store & 3)) return CU32_E_ALIGN;
  }
  if (c.scale_on && (c.gz != 1 || c.bias)) return CU32_E_ARG;
  if (c.n_replicas < 0 || c.n_replicas > 7 || (c.n_replicas > 0 && (!c.replicas || c.gz != 1))) return CU32_E_ARG;
  // the copies are written by two instantiations only: FP32-accurate, row-major A, not a convolution
  if (c.n_replicas > 0 && (!c.x3 || c.a_mn)) return CU32_E_ARG;
  if (!load_driver_entry_points()) return CU32_E_DRIVER;

  int tile = pick_tile(c.M, c.n_store, c.gz > 1 ? c.gz : c.batch);
  // Shapes below the ridge of the FP32-accurate roofline (about 44 flop per byte: short reductions such as the
  // attention-shaped batched products) are paced by loads, stores and the split, not by the tensor pipe; measured
  // on B200 at batch 1024: a 64-column output is fastest on the one-CTA 128x64 tile with six raw slots, a wide
  // output on the 256x256 pair tile with two store-staging tiles per drain warp.
  const double intensity = 2.0 * c.M * c.n_store * c.K / (4.0 * (static_cast<double>(c.M) * c.K +
                           static_cast<double>(c.K) * c.n_store + static_cast<double>(c.M) * c.n_store));
  const bool below_ridge = c.x3 && c.gz == 1 && intensity < 44.0;
  if (below_ridge && g_tile.load() < 0 && c.n_store <= 64 && c.M >= 128) tile = note_tile(TILE_1x64);
  if (c.n_replicas > 0) tile = note_tile(TILE_2x256);
  const int ctas = tile_ctas(tile), bn = tile_bn(tile);

  GemmParams p;
  std::memset(&p, 0, sizeof(p));
  int rc;
  const uint64_t nb = static_cast<uint64_t>(c.batch);
  // A
  if (c.a_mn) rc = make_map3(&p.tmA, c.A, c.M, c.K, nb, c.lda, c.sA ? c.sA : c.lda * c.K, 32, 32, true);
  else        rc = make_map3(&p.tmA, c.A, c.K, c.M, nb, c.lda, c.sA ? c.sA : c.lda * c.M, 32, 128, false);
  if (rc) return rc;
  // B
  if (c.b_mn) rc = make_map3(&p.tmB, c.B, c.N, c.K, nb, c.ldb, c.sB ? c.sB : c.ldb * c.K, 32, 32, true);
  else        rc = make_map3(&p.tmB, c.B, c.K, c.N, nb, c.ldb, c.sB ? c.sB : c.ldb * c.N, 32, bn / ctas, false);
  if (rc) return rc;

  p.C = c.C;
  p.Cbuf = c.Cbuf;
  p.bias = c.bias;
  p.bias_width = c.bias_width;
  p.ldc = c.ldc;
  p.c_stride = c.sC;
  p.M = c.M;
  p.N = c.n_store;
  p.nkb_total = (c.K + 31) / 32;
  p.tiles_m = (c.M + 128 * ctas - 1) / (128 * ctas);
  p.tiles_n = (c.n_store + bn - 1) / bn;
  p.gz = c.gz;
  p.kc = c.x3 ? g_kc.load() : g_kc_fast.load();
  choose_rings(&p);
  if (below_ridge && p.ring_raw == 0) {
    if (tile == TILE_1x64) { p.ring_raw = 6; p.ring_lo = 2; p.store_bufs = 1; }
    else if (tile == TILE_2x256) { p.ring_raw = 3; p.ring_lo = 2; p.store_bufs = 2; }
  }
  p.l2_hints = (p.tiles_n > 1 && p.tiles_m > 1) ? g_l2hint.load() : 0;
  p.vec4_ok = (aligned16(c.C) && !(c.ldc & 3) && !(c.sC & 3) && (c.gz == 1 || aligned16(c.Cbuf))) ? 1 : 0;
  if (p.bias && !p.vec4_ok) return CU32_E_ALIGN;   // the bias is applied on the vector store paths only
  if (c.scale_on && !p.vec4_ok) return CU32_E_ALIGN;
  p.scale_on = c.scale_on ? 1 : 0; p.alpha = c.alpha;
  if (p.vec4_ok) {
    // Output maps for the TMA-store epilogue: (columns, rows, batch) with the caller's pitch.
    const uint64_t zs_c = c.gz > 1 ? 1 : nb;
    const uint64_t sc = c.sC ? c.sC : static_cast<uint64_t>(c.ldc) * c.M;
    rc = make_map3(&p.tmC, c.C, c.n_store, c.M, zs_c, c.ldc, sc, 32, 32, false);
    if (!rc && c.gz > 1) rc = make_map3(&p.tmCbuf, c.Cbuf, c.n_store, c.M, c.gz - 1, c.ldc, sc, 32, 32, false);
    if (rc) return rc;
    p.tma_store = 1;
    for (int i = 0; i < c.n_replicas; ++i) {
      if (!c.replicas[i]) return CU32_E_NULL;
      if (!aligned16(c.replicas[i])) return CU32_E_ALIGN;
      if (int r2 = make_map3(&p.tmRep[i], c.replicas[i], c.n_store, c.M, zs_c, c.ldc, sc, 32, 32, false)) return r2;
    }
    p.n_rep = c.n_replicas;
    if (c.n_replicas > 0 && g_rep_lazy.load() && c.batch == 1 && c.gz == 1) {
      p.rep_lazy = 1;
      for (int i = 0; i < c.n_replicas; ++i) p.rep_ptr[i] = c.replicas[i];
    }
  } else if (c.n_replicas > 0) {
    return CU32_E_ALIGN;   // the copies are written by the tensor-map store path only
  }
  if (c.n_replicas > 0 && (c.bias || c.scale_on)) return CU32_E_ARG;
  cudaError_t e;
  p.status = status_word_ptr(&e);
  if (!p.status) return static_cast<int>(e);

  // Batches (or split-K slices) are folded into the kernel's tile index.
  const int zs = c.gz > 1 ? c.gz : c.batch;
  if (c.n_replicas > 0)       e = launch_gemm_rep(c.b_mn, p, zs, c.stream);
  else if (c.a_mn && c.b_mn)  e = launch_gemm_nn(tile, c.x3, p, zs, c.stream);
  else if (!c.a_mn && c.b_mn) e = launch_gemm_kn(tile, c.x3, false, p, zs, c.stream);
  else if (!c.a_mn)           e = launch_gemm_kk(tile, c.x3, false, p, zs, c.stream);
  else return CU32_E_ARG;
  if (e != cudaSuccess) return static_cast<int>(e);
  e = cudaPeekAtLastError();
  return static_cast<int>(e);
}

static int check_streams(const int64_t* streams, int length, cudaStream_t* s0) {
  if (!streams || length < 1 || length > 10) return CU32_E_STREAMS;
  *s0 = reinterpret_cast<cudaStream_t>(static_cast<intptr_t>(streams[0]));
  return CU32_OK;
}

// ------------------------------------------------------------------ matMul family
enum MatForm { FORM_AB, FORM_T1, FORM_T2 };

static int matmul_any(MatForm form, bool x3, const int64_t* streams, int length, int GridZ,
                      const float* dA, const float* dB, float* dC, float* dCbuf, int N, int M, int K,
                      const float* dBias = nullptr, int width = 0, float* const* replicas = nullptr, int n_replicas = 0) {
  cudaStream_t st;
  if (int rc = check_streams(streams, length, &st)) return rc;
  if (N <= 0 || M <= 0 || K <= 0) return CU32_E_DIM;
  if (GridZ < 1) return CU32_E_ARG;
  GemmCall c{};
  c.A = dA; c.B = dB; c.C = dC; c.Cbuf = dCbuf;
  c.M = N; c.N = M; c.K = K; c.n_store = M;
  c.ldc = M;
  c.batch = 1; c.sA = 0; c.sB = 0;
  c.sC = static_cast<long long>(N) * M;  // distance between split-K partial buffers
  c.gz = GridZ; c.x3 = x3; c.stream = st;
  c.bias = dBias; c.bias_width = width;
  c.replicas = replicas; c.n_replicas = n_replicas;
  switch (form) {
    case FORM_AB: c.a_mn = false; c.lda = K; c.b_mn = true;  c.ldb = M; break;
    case FORM_T1: c.a_mn = true;  c.lda = N; c.b_mn = true;  c.ldb = M; break;
    case FORM_T2: c.a_mn = false; c.lda = K; c.b_mn = false; c.ldb = K; break;
  }
  return run_gemm(c);
}

// ------------------------------------------------------------------ split-K buffer summation
// C += sum_p Cbuf[p], Kahan-compensated, 4 floats per thread per step.  BIAS: the sum then takes
// the bias row (one more FP32 add, exactly what a separate bias kernel would do to the stored
// sum) and the padding columns (col >= width inside each row of row_len floats) become zero.
template <bool BIAS>
__global__ void skbuf_summary_kernel(const float* __restrict__ Cbuf, float* __restrict__ C, int part,
                                     long long sizeC, const float* __restrict__ bias, int row_len, int width) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * 4;
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4; i < sizeC;
       i += stride) {
    if (i + 3 < sizeC) {
      float4 sum = *reinterpret_cast<const float4*>(C + i);
      float4 comp = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int p = 0; p < part; ++p) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(Cbuf + static_cast<long long>(p) * sizeC + i));
        float y, t;
        y = v.x - comp.x; t = sum.x + y; comp.x = (t - sum.x) - y; sum.x = t;
        y = v.y - comp.y; t = sum.y + y; comp.y = (t - sum.y) - y; sum.y = t;
        y = v.z - comp.z; t = sum.z + y; comp.z = (t - sum.z) - y; sum.z = t;
        y = v.w - comp.w; t = sum.w + y; comp.w = (t - sum.w) - y; sum.w = t;
      }
      if (BIAS) {   // row_len is a multiple of 4, so the four elements share a row
        const int col = static_cast<int>(i % row_len);
        const float4 b = __ldg(reinterpret_cast<const float4*>(bias + col));
        sum.x = (col + 0 < width) ? sum.x + b.x : 0.f;
        sum.y = (col + 1 < width) ? sum.y + b.y : 0.f;
        sum.z = (col + 2 < width) ? sum.z + b.z : 0.f;
        sum.w = (col + 3 < width) ? sum.w + b.w : 0.f;
      }
      *reinterpret_cast<float4*>(C + i) = sum;
    } else {
      for (long long j = i; j < sizeC; ++j) {
        float sum = C[j], comp = 0.f;
        for (int p = 0; p < part; ++p) {
          const float y = Cbuf[static_cast<long long>(p) * sizeC + j] - comp;
          const float t = sum + y;
          comp = (t - sum) - y;
          sum = t;
        }
        if (BIAS) {
          const int col = static_cast<int>(j % row_len);
          sum = (col < width) ? sum + bias[col] : 0.f;
        }
        C[j] = sum;
      }
    }
  }
}

// ------------------------------------------------------------------ filter remode
// CW[g][oc] = W[oc][g], g = (fh, fw, ic) flattened: a [OC x G] -> [G x OC] transpose
// through a padded 32x32 shared-memory tile (coalesced on both sides).
__global__ void remode_kernel(const float* __restrict__ W, float* __restrict__ CW, int OC, int G) {
  __shared__ float tile[32][33];
  const int g0 = blockIdx.x * 32, oc0 = blockIdx.y * 32;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int oc = oc0 + r, g = g0 + threadIdx.x;
    tile[r][threadIdx.x] = (oc < OC && g < G) ? W[static_cast<long long>(oc) * G + g] : 0.f;
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int g = g0 + r, oc = oc0 + threadIdx.x;
    if (g < G && oc < OC) CW[static_cast<long long>(g) * OC + oc] = tile[threadIdx.x][r];
  }
}

// ------------------------------------------------------------------ convolution
static int conv_any(bool x3, const int64_t* streams, int length, const float* dX, int IH, int IW,
                    const float* dW, int FH, int FW, float* dY, int OH, int OW, int N, int IC, int OC,
                    int sh, int sw, int ph, int pw, const float* dBias = nullptr, int width = 0,
                    bool flip = false) {
  // flip: the filter is stored as W[IC][FH][FW][OC] (input channel outermost, output channel
  // contiguous) and applied rotated by 180 degrees - the data-gradient of a stride-1 convolution
  // written as a forward convolution of deltaY (see deconv_s1_any).
  load_env_once();
  cudaStream_t st;
  if (int rc = check_streams(streams, length, &st)) return rc;
  if (!dX || !dW || !dY) return CU32_E_NULL;
  if (IH <= 0 || IW <= 0 || FH <= 0 || FW <= 0 || OH <= 0 || OW <= 0 || N <= 0 || IC <= 0 || OC <= 0 ||
      sh <= 0 || sw <= 0 || (!flip && (ph < 0 || pw < 0)))
    return CU32_E_DIM;
  if ((IC & 3) || !aligned16(dX) || !aligned16(dW)) return CU32_E_ALIGN;
  // forward entry points: the output extents must be the ones the geometry gives (the data-gradient callers
  // have derived their padding from the extents already)
  if (!flip && (IH + 2 * ph < FH || IW + 2 * pw < FW || OH != (IH + 2 * ph - FH) / sh + 1 ||
                OW != (IW + 2 * pw - FW) / sw + 1))
    return CU32_E_DIM;
  if (dBias) {
    if (width <= 0 || width > OC) return CU32_E_DIM;
    if (!aligned16(dBias) || (OC & 3)) return CU32_E_ALIGN;
  }
  const long long GM = static_cast<long long>(N) * OH * OW;
  const long long GK = static_cast<long long>(FH) * FW * IC;
  if (GM >= (1LL << 31) || GK >= (1LL << 31) || static_cast<long long>(N) * IH * IW * IC >= (1LL << 31))
    return CU32_E_DIM;
  if (!load_driver_entry_points()) return CU32_E_DRIVER;

  // 1x1 / stride 1 / no padding with matching extents is a plain contraction Y[GM,OC] = X[GM,IC] * W[OC,IC]^T.
  if (FH == 1 && FW == 1 && sh == 1 && sw == 1 && ph == 0 && pw == 0 && OH == IH && OW == IW) {
    GemmCall c{};
    c.A = dX; c.B = dW; c.C = dY; c.Cbuf = nullptr;
    c.M = static_cast<int>(GM); c.N = OC; c.K = IC; c.n_store = OC;
    c.lda = IC; c.ldb = flip ? OC : IC; c.ldc = OC; c.a_mn = false; c.b_mn = flip;   // flip: W is [IC][OC]
    c.batch = 1; c.sA = 0; c.sB = 0; c.sC = 0; c.gz = 1; c.x3 = x3; c.stream = st;
    c.bias = dBias; c.bias_width = width;
    return run_gemm(c);
  }

  if (!g_encode_im2col) return CU32_E_DRIVER;
  // The im2col tensor map walks "base pixels" (the top-left input pixel of each output
  // position) inside the box [lower, extent - 1 + upper] with the convolution stride;
  // the filter tap is added per load as an offset.  Corners must fit 8 signed bits,
  // offsets 8 unsigned bits and strides 3 bits; a geometry beyond that (or one the driver's
  // encoder refuses) is served by the kernel's gather path, slower but without limits.
  const int lower_w = -pw, lower_h = -ph;
  const int upper_w = lower_w + (OW - 1) * sw - (IW - 1);
  const int upper_h = lower_h + (OH - 1) * sh - (IH - 1);
  bool gather = g_force_gather.load() != 0 || lower_w < -128 || lower_w > 127 || lower_h < -128 || lower_h > 127 ||
                upper_w < -128 || upper_w > 127 || upper_h < -128 || upper_h > 127 || FW > 256 || FH > 256 || sw > 8 || sh > 8;

  int tile = pick_tile(GM, OC, 1);
  const int ctas = tile_ctas(tile), bn = tile_bn(tile);

  GemmParams p;
  std::memset(&p, 0, sizeof(p));
  {
    cuuint64_t dims[4] = {static_cast<cuuint64_t>(IC), static_cast<cuuint64_t>(IW),
                          static_cast<cuuint64_t>(IH), static_cast<cuuint64_t>(N)};
    cuuint64_t strides[3] = {static_cast<cuuint64_t>(IC) * 4, static_cast<cuuint64_t>(IW) * IC * 4,
                             static_cast<cuuint64_t>(IH) * IW * IC * 4};
    int lower[2] = {lower_w, lower_h};
    int upper[2] = {upper_w, upper_h};
    cuuint32_t trav[4] = {1, static_cast<cuuint32_t>(sw), static_cast<cuuint32_t>(sh), 1};
    CUresult r = gather ? CUDA_ERROR_INVALID_VALUE
                        : g_encode_im2col(&p.tmA, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(dX), dims,
                                          strides, lower, upper, /*channelsPerPixel=*/32, /*pixelsPerColumn=*/128,
                                          trav, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) gather = true;
    // Drivers up to CUDA 13.1 set a descriptor flag that mis-handles im2col maps over
    // tensors smaller than 128 KiB; NVIDIA's CUTLASS clears bit 21 of the second 64-bit
    // word in that case (cute/atom/copy_traits_sm90_im2col.hpp), and so does this.
    int drv = 0;
    if (cudaDriverGetVersion(&drv) == cudaSuccess && drv <= 13010 &&
        static_cast<long long>(N) * IH * IW * IC * 4 < 131072)
      reinterpret_cast<uint64_t*>(&p.tmA)[1] &= ~(1ULL << 21);
  }
  if (!flip) {
    // Filters W[OC][FH*FW*IC]: reduction axis contiguous.
    if (int rc = make_map3(&p.tmB, dW, static_cast<uint64_t>(GK), OC, 1, GK, GK * OC, 32, bn / ctas, false)) return rc;
  } else {
    // Filters W[IC][FH][FW][OC] read in place as one [IC x OC] matrix per tap, OC contiguous:
    // dims (oc, ic, tap) with pitches (1, FH*FW*OC, OC); 32 x 32 boxes in the 32-byte-unit swizzle.
    if ((OC & 3)) return CU32_E_ALIGN;
    {
      // dims ordered by increasing pitch: (oc, tap, ic) with pitches (1, OC, FH*FW*OC) floats; a load
      // takes 32 oc x 1 tap x 32 ic, which lands as the 32 x 32 MN-major slab the tensor core expects
      cuuint64_t dims[3] = {static_cast<cuuint64_t>(OC), static_cast<cuuint64_t>(FH) * FW, static_cast<cuuint64_t>(IC)};
      cuuint64_t strides[2] = {static_cast<cuuint64_t>(OC) * 4, static_cast<cuuint64_t>(FH) * FW * OC * 4};
      cuuint32_t box[3] = {32, 1, 32};
      cuuint32_t estr[3] = {1, 1, 1};
      CUresult r = g_encode_tiled(&p.tmB, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(dW), dims, strides,
                                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B,
                                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (r != CUDA_SUCCESS) return CU32_E_TENSORMAP;
    }
    p.tap_base = FH * FW - 1; p.tap_sy = -FW; p.tap_sx = -1; p.bmap_order = 0;   // rotated by 180 degrees
  }

  p.bias = dBias; p.bias_width = width;
  p.C = dY; p.Cbuf = nullptr; p.ldc = OC; p.c_stride = 0;
  p.M = static_cast<int>(GM); p.N = OC;
  p.conv_icb = (IC + 31) / 32;
  p.nkb_total = FH * FW * p.conv_icb;
  p.tiles_m = static_cast<int>((GM + 128 * ctas - 1) / (128 * ctas));
  p.tiles_n = (OC + bn - 1) / bn;
  p.gz = 1;
  p.kc = x3 ? g_kc.load() : g_kc_fast.load();
  choose_rings(&p);
  p.l2_hints = (p.tiles_n > 1 && p.tiles_m > 1) ? g_l2hint.load() : 0;
  p.vec4_ok = (aligned16(dY) && !(OC & 3)) ? 1 : 0;
  if (p.bias && !p.vec4_ok) return CU32_E_ALIGN;
  if (p.vec4_ok) {
    if (int rc = make_map3(&p.tmC, dY, OC, static_cast<uint64_t>(GM), 1, OC, static_cast<uint64_t>(GM) * OC, 32, 32, false)) return rc;
    p.tma_store = 1;
  }
  p.conv_OW = OW; p.conv_OH = OH; p.conv_FW = FW; p.conv_IC = IC;
  p.conv_sw = sw; p.conv_sh = sh; p.conv_pw = pw; p.conv_ph = ph;
  p.gather = gather ? 1 : 0; p.g_img = dX; p.g_H = IH; p.g_W = IW; p.g_N = N;
  cudaError_t e;
  p.status = status_word_ptr(&e);
  if (!p.status) return static_cast<int>(e);
  e = flip ? launch_gemm_kn(tile, x3, true, p, 1, st) : launch_gemm_kk(tile, x3, true, p, 1, st);
  if (e != cudaSuccess) return static_cast<int>(e);
  return static_cast<int>(cudaPeekAtLastError());
}

// Data gradient of a stride-1 convolution: deltaX[n,ih,iw,ic] = sum_{fh,fw,oc}
// deltaY[n, ih+ph-fh, iw+pw-fw, oc] * W[oc,fh,fw,ic] (zero outside deltaY) - a forward convolution of
// deltaY (OC channels in, IC channels out) with padding (FH-1-ph, FW-1-pw) and the filter rotated by
// 180 degrees and read "transposed" in place.  The filter rotation is a reversal of the tap index in
// the TMA producer; nothing is re-laid-out or copied.
static int deconv_s1_any(const int64_t* streams, int length, const float* dDY, int OH, int OW, const float* dW,
                         int FH, int FW, float* dDX, int IH, int IW, int N, int IC, int OC, int ph, int pw,
                         const float* dBias = nullptr, int width = 0) {
  if (!dDY || !dW || !dDX) return CU32_E_NULL;
  if (FH <= 0 || FW <= 0 || ph < 0 || pw < 0 || IC <= 0 || OC <= 0) return CU32_E_DIM;
  if ((IC & 3) || (OC & 3)) return CU32_E_ALIGN;
  // Any pair of extents is served, as by the reference's kernels (its own test pairs IH = OH = 64 with an 8x8
  // filter and padding 4): deltaY rows the sum would need outside [0, OH) count as zeros, rows it never needs are
  // never read.
  if (IH <= 0 || IW <= 0 || OH <= 0 || OW <= 0) return CU32_E_DIM;
  // padding beyond the filter reach makes the equivalent forward padding negative (the outermost pixels of deltaY
  // are never used); conv_any takes it as it is
  return conv_any(true, streams, length, dDY, OH, OW, dW, FH, FW, dDX, IH, IW, N, /*in*/ OC, /*out*/ IC, 1, 1,
                  FH - 1 - ph, FW - 1 - pw, dBias, width, true);
}

// ------------------------------------------------------------------ kernel-split filter workspace
// CW[y][x][...] for the sh*sw phases of the strided data gradient: phase (y, x) holds the taps
// fh = y + (CFH_y - 1 - fhr) * sh, fw = x + (CFW_x - 1 - fwr) * sw of W[OC][FH][FW][IC] (zeros where the tap
// does not exist), packed at the start of a slot of OC * mCFH * mCFW * IC floats.  V2 orders a phase as
// [fhr][fwr][oc][ic], the older form as [oc][fhr][fwr][ic]; elements of a slot past the phase's own size
// are left untouched, as in the reference.
template <bool V2>
__global__ void ks_remode_kernel(const float* __restrict__ W, int FH, int FW, float* __restrict__ CW, int mCFH,
                                 int mCFW, int OC, int IC, int sh, int sw) {
  const int by = blockIdx.y;
  CW += static_cast<long long>(by) * OC * mCFH * mCFW * IC;
  const int y = by / sw, x = by - y * sw;
  const int CFH = (FH - y + sh - 1) / sh, CFW = (FW - x + sw - 1) / sw;
  if (CFH <= 0 || CFW <= 0) return;
  const long long n = static_cast<long long>(OC) * CFH * CFW * IC;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    int oc, fhr, fwr, ic;
    long long r = i;
    if (V2) {
      fhr = static_cast<int>(r / (static_cast<long long>(CFW) * OC * IC)); r -= static_cast<long long>(fhr) * CFW * OC * IC;
      fwr = static_cast<int>(r / (static_cast<long long>(OC) * IC));       r -= static_cast<long long>(fwr) * OC * IC;
      oc = static_cast<int>(r / IC); ic = static_cast<int>(r - static_cast<long long>(oc) * IC);
    } else {
      oc = static_cast<int>(r / (static_cast<long long>(CFH) * CFW * IC)); r -= static_cast<long long>(oc) * CFH * CFW * IC;
      fhr = static_cast<int>(r / (static_cast<long long>(CFW) * IC));      r -= static_cast<long long>(fhr) * CFW * IC;
      fwr = static_cast<int>(r / IC); ic = static_cast<int>(r - static_cast<long long>(fwr) * IC);
    }
    const int fh = y + (CFH - 1 - fhr) * sh, fw = x + (CFW - 1 - fwr) * sw;
    CW[i] = (fh < FH && fw < FW) ? W[((static_cast<long long>(oc) * FH + fh) * FW + fw) * IC + ic] : 0.0f;
  }
}

static int ks_remode_any(bool v2, int64_t stream, const float* dW, int FH, int FW, float* dCW, int CFH, int CFW, int OC,
                         int IC, int sh, int sw) {
  if (!dW || !dCW) return CU32_E_NULL;
  if (FH <= 0 || FW <= 0 || OC <= 0 || IC <= 0 || sh <= 0 || sw <= 0) return CU32_E_DIM;
  if (CFH != (FH + sh - 1) / sh || CFW != (FW + sw - 1) / sw) return CU32_E_DIM;
  if (static_cast<long long>(sh) * sw > 65535) return CU32_E_DIM;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(static_cast<intptr_t>(stream));
  const long long n = static_cast<long long>(OC) * CFH * CFW * IC;
  long long bx = (n + 255) / 256;
  if (bx > device_sm_count() * 8) bx = device_sm_count() * 8;
  const dim3 grid(static_cast<unsigned>(bx), static_cast<unsigned>(sh * sw));
  if (v2) ks_remode_kernel<true><<<grid, 256, 0, st>>>(dW, FH, FW, dCW, CFH, CFW, OC, IC, sh, sw);
  else    ks_remode_kernel<false><<<grid, 256, 0, st>>>(dW, FH, FW, dCW, CFH, CFW, OC, IC, sh, sw);
  return static_cast<int>(cudaPeekAtLastError());
}

// Data gradient for any stride, as sh*sw stride-1 sub-problems ("kernel split"): the input pixels ih with
// (ih + ph) % sh == y only ever meet the filter taps fh = y, y + sh, y + 2 sh, ...  For such a phase (y, x)
//   deltaX[n, sh*u + y - ph, sw*v + x - pw, :] = sum_{t, r, oc} deltaY[n, u - t, v - r, oc] * W[oc, y + sh*t, x + sw*r, :]
// which is a forward stride-1 convolution of deltaY with a CFH x CFW sub-filter (taps in reverse order) whose
// output rows are strided pixels of deltaX.  Each phase is one launch of the same kernel: im2col A over deltaY
// with the phase's corners, the sub-filter's [OC x IC] matrices picked tap by tap - from the forward filter where it
// lies, or from the reference's kernel-split workspace CW[y][x][CFH][CFW][OC][IC] - and register stores to the
// strided rows.
static int ceil_div(int a, int b) { return a >= 0 ? (a + b - 1) / b : -((-a) / b); }

static int deconv_strided_any(const int64_t* streams, int length, const float* dDY, int OH, int OW,
                              const float* filt, bool filt_is_cw, int FH, int FW, float* dDX, int IH, int IW, int N,
                              int IC, int OC, int sh, int sw, int ph, int pw, const float* dBias = nullptr,
                              int width = 0) {
  load_env_once();
  cudaStream_t st;
  if (int rc = check_streams(streams, length, &st)) return rc;
  if (!dDY || !filt || !dDX) return CU32_E_NULL;
  if (IH <= 0 || IW <= 0 || OH <= 0 || OW <= 0 || FH <= 0 || FW <= 0 || N <= 0 || IC <= 0 || OC <= 0 || sh <= 0 ||
      sw <= 0 || ph < 0 || pw < 0)
    return CU32_E_DIM;
  if ((IC & 3) || (OC & 3) || !aligned16(dDY) || !aligned16(filt) || !aligned16(dDX)) return CU32_E_ALIGN;
  // extents are taken as given (see deconv_s1_any): what lies outside deltaY counts as zeros
  if (static_cast<long long>(N) * IH * IW * IC >= (1LL << 31) || static_cast<long long>(N) * OH * OW * OC >= (1LL << 31))
    return CU32_E_DIM;
  if (static_cast<long long>(sh) * sw > 4096) return CU32_E_DIM;   // one launch per phase
  if (dBias) {
    if (width <= 0 || width > IC) return CU32_E_DIM;
    if (!aligned16(dBias)) return CU32_E_ALIGN;
    if (FH < sh || FW < sw) return CU32_E_ARG;   // pixels no tap reaches would need the bias alone: use the unbiased native + bias kernel
  }
  if (!load_driver_entry_points() || !g_encode_im2col) return CU32_E_DRIVER;
  const int mCFH = (FH + sh - 1) / sh, mCFW = (FW + sw - 1) / sw;
  cudaError_t e;
  if (FH < sh || FW < sw) {   // some phases meet no tap at all: their pixels are zero
    e = cudaMemsetAsync(dDX, 0, sizeof(float) * static_cast<size_t>(N) * IH * IW * IC, st);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  int* status = status_word_ptr(&e);
  if (!status) return static_cast<int>(e);
  // Every phase with work, heaviest first as the loops run: its tensor maps and the numbers the kernel needs.
  struct Phase {
    CUtensorMap tmA, tmB;
    float* C;
    long long GM;
    int nkb, U, V, CFW, conv_pw, conv_ph, tap_base, tap_sy, tap_sx, bmap_order;
    bool gather;
  };
  std::vector<Phase> phs;
  for (int y = 0; y < sh; ++y)
    for (int x = 0; x < sw; ++x) {
      if (y >= FH || x >= FW) continue;
      const int CFH = (FH - y + sh - 1) / sh, CFW = (FW - x + sw - 1) / sw;
      const int u0 = ceil_div(ph - y, sh), v0 = ceil_div(pw - x, sw);
      const int nu = IH - 1 + ph - y, nv = IW - 1 + pw - x;
      if (nu < 0 || nv < 0) continue;
      const int U = nu / sh - u0 + 1, V = nv / sw - v0 + 1;
      if (U <= 0 || V <= 0) continue;
      const int lower_h = u0 - (CFH - 1), lower_w = v0 - (CFW - 1);
      const int upper_h = lower_h + (U - 1) - (OH - 1), upper_w = lower_w + (V - 1) - (OW - 1);
      Phase q;
      std::memset(&q, 0, sizeof(q));
      q.gather = g_force_gather.load() != 0 || lower_w < -128 || lower_w > 127 || lower_h < -128 || lower_h > 127 ||
                 upper_w < -128 || upper_w > 127 || upper_h < -128 || upper_h > 127 || CFH > 256 || CFW > 256;
      q.GM = static_cast<long long>(N) * U * V;
      {
        cuuint64_t dims[4] = {static_cast<cuuint64_t>(OC), static_cast<cuuint64_t>(OW), static_cast<cuuint64_t>(OH),
                              static_cast<cuuint64_t>(N)};
        cuuint64_t strides[3] = {static_cast<cuuint64_t>(OC) * 4, static_cast<cuuint64_t>(OW) * OC * 4,
                                 static_cast<cuuint64_t>(OH) * OW * OC * 4};
        int lower[2] = {lower_w, lower_h};
        int upper[2] = {upper_w, upper_h};
        cuuint32_t trav[4] = {1, 1, 1, 1};
        CUresult r = q.gather ? CUDA_ERROR_INVALID_VALUE
                              : g_encode_im2col(&q.tmA, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(dDY), dims, strides,
                                                lower, upper, 32, 128, trav, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) q.gather = true;
        int drv = 0;   // same driver workaround as in conv_any
        if (cudaDriverGetVersion(&drv) == cudaSuccess && drv <= 13010 &&
            static_cast<long long>(N) * OH * OW * OC * 4 < 131072)
          reinterpret_cast<uint64_t*>(&q.tmA)[1] &= ~(1ULL << 21);
      }
      if (filt_is_cw) {
        // this phase's slot of CW: [CFH][CFW][OC][IC], taps already reversed by ks_remodev2
        const float* base = filt + static_cast<long long>(y * sw + x) * OC * mCFH * mCFW * IC;
        if (int rc = make_map3(&q.tmB, base, IC, OC, static_cast<uint64_t>(CFH) * CFW, IC,
                               static_cast<uint64_t>(OC) * IC, 32, 32, true))
          return rc;
        q.bmap_order = 1; q.tap_base = 0; q.tap_sy = CFW; q.tap_sx = 1;
      } else {
        cuuint64_t dims[3] = {static_cast<cuuint64_t>(IC), static_cast<cuuint64_t>(FH) * FW, static_cast<cuuint64_t>(OC)};
        cuuint64_t strides[2] = {static_cast<cuuint64_t>(IC) * 4, static_cast<cuuint64_t>(FH) * FW * IC * 4};
        cuuint32_t box[3] = {32, 1, 32};
        cuuint32_t estr[3] = {1, 1, 1};
        CUresult r = g_encode_tiled(&q.tmB, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(filt), dims, strides,
                                    box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B,
                                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return CU32_E_TENSORMAP;
        q.bmap_order = 0;
        q.tap_base = (y + (CFH - 1) * sh) * FW + x + (CFW - 1) * sw;
        q.tap_sy = -sh * FW;
        q.tap_sx = -sw;
      }
      q.C = dDX + (static_cast<long long>(u0 * sh + y - ph) * IW + (v0 * sw + x - pw)) * IC;
      q.nkb = CFH * CFW * ((OC + 31) / 32);
      q.U = U; q.V = V; q.CFW = CFW; q.conv_pw = -lower_w; q.conv_ph = -lower_h;
      phs.push_back(q);
    }
  if (phs.empty()) return static_cast<int>(cudaPeekAtLastError());
  // One launch for all phases when there are 2..4 of them and tensor maps serve them all: a CTA (pair) then takes
  // tile j of every phase in turn, so a short phase's drain and stores run under the next phase's MMAs.  Otherwise
  // one launch per phase; they write disjoint pixels, so every launch after the first may overlap the one before it.
  bool fuse = g_phase_fused.load() != 0 && phs.size() >= 2 && phs.size() <= 4;
  for (const Phase& q : phs) fuse = fuse && !q.gather;
  long long gm_max = 0;
  for (const Phase& q : phs) gm_max = q.GM > gm_max ? q.GM : gm_max;
  const size_t launches = fuse ? 1 : phs.size();
  for (size_t li = 0; li < launches; ++li) {
    const Phase& q = phs[li];
    const long long GM = fuse ? gm_max : q.GM;
    int tile = pick_tile(GM, IC, fuse ? static_cast<long long>(phs.size()) : 1);
    const int ctas = tile_ctas(tile), bn = tile_bn(tile);
    GemmParams p;
    std::memset(&p, 0, sizeof(p));
    p.tmA = q.tmA; p.tmB = q.tmB;
    p.bmap_order = q.bmap_order; p.tap_base = q.tap_base; p.tap_sy = q.tap_sy; p.tap_sx = q.tap_sx;
    p.bias = dBias; p.bias_width = width;
    p.C = q.C;
    p.Cbuf = nullptr; p.ldc = IC; p.c_stride = 0;
    p.os_on = 1; p.os_uv = q.U * q.V; p.os_v = q.V;
    p.os_sn = static_cast<long long>(IH) * IW * IC;
    p.os_su = static_cast<long long>(sh) * IW * IC;
    p.os_sv = static_cast<long long>(sw) * IC;
    p.M = static_cast<int>(q.GM); p.N = IC;
    p.conv_icb = (OC + 31) / 32;
    p.nkb_total = q.nkb;
    p.tiles_m = static_cast<int>((GM + 128 * ctas - 1) / (128 * ctas));
    p.tiles_n = (IC + bn - 1) / bn;
    p.gz = 1;
    p.kc = g_kc.load();
    choose_rings(&p);
    p.vec4_ok = 1;
    p.tma_store = 0;
    p.conv_OW = q.V; p.conv_OH = q.U; p.conv_FW = q.CFW; p.conv_IC = OC;
    p.conv_sw = 1; p.conv_sh = 1; p.conv_pw = q.conv_pw; p.conv_ph = q.conv_ph;
    p.gather = q.gather ? 1 : 0; p.g_img = dDY; p.g_H = OH; p.g_W = OW; p.g_N = N;
    p.status = status;
    if (fuse) {
      p.n_phases = static_cast<int>(phs.size());
      for (size_t i = 1; i < phs.size(); ++i) {
        GemmPhase& x = p.phx[i - 1];
        const Phase& r = phs[i];
        x.tmA = r.tmA; x.tmB = r.tmB; x.C = r.C; x.M = static_cast<int>(r.GM); x.nkb = r.nkb;
        x.OH = r.U; x.OW = r.V; x.FW = r.CFW; x.pw = r.conv_pw; x.ph = r.conv_ph;
        x.tap_base = r.tap_base; x.tap_sy = r.tap_sy; x.tap_sx = r.tap_sx; x.os_uv = r.U * r.V; x.os_v = r.V;
      }
    }
    p.overlap_prev = (li > 0 && g_phase_overlap.load()) ? 1 : 0;
    e = launch_gemm_kn(tile, true, true, p, 1, st);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  return static_cast<int>(cudaPeekAtLastError());
}

// Weight gradient of the convolution:
//   deltaW[oc, fh, fw, ic] = sum_{n, oh, ow} deltaY[n, oh, ow, oc] * X[n, oh*sh - ph + fh, ow*sw - pw + fw, ic]
// For one tap (fh, fw) this is A^T * B with A = deltaY as a [pixels x OC] matrix and B = the [pixels x IC] matrix of
// input pixels shifted by the tap (zero outside the image): the long-K contraction of the fully-connected weight
// gradient, with the B tile fetched by an im2col-mode tensor map over X (32 pixels x 32 channels per load, the
// tap as the load's offset).  All taps and all split-K slices are tiles of one launch (z = slice * taps + tap);
// slice 0 writes deltaW, slice s > 0 the s-th partial buffer, exactly like the matMul split-K protocol, and
// buf_summary folds the partials in.
static int deconvW_any(const int64_t* streams, int length, int GridZ, const float* dX, int IH, int IW,
                       const float* dDY, int OH, int OW, float* dDW, float* dBuf, int FH, int FW, int N, int IC,
                       int OC, int sh, int sw, int ph, int pw) {
  load_env_once();
  cudaStream_t st;
  if (int rc = check_streams(streams, length, &st)) return rc;
  if (!dX || !dDY || !dDW) return CU32_E_NULL;
  if (GridZ < 1) return CU32_E_ARG;
  if (GridZ > 1 && !dBuf) return CU32_E_NULL;
  if (IH <= 0 || IW <= 0 || OH <= 0 || OW <= 0 || FH <= 0 || FW <= 0 || N <= 0 || IC <= 0 || OC <= 0 || sh <= 0 ||
      sw <= 0 || ph < 0 || pw < 0)
    return CU32_E_DIM;
  if ((IC & 3) || (OC & 3) || !aligned16(dX) || !aligned16(dDY) || !aligned16(dDW) || (dBuf && !aligned16(dBuf)))
    return CU32_E_ALIGN;
  // extents are taken as given, as by the reference (see deconv_s1_any): input pixels outside X count as zeros
  const long long GK = static_cast<long long>(N) * OH * OW;
  const long long taps = static_cast<long long>(FH) * FW;
  if (GK >= (1LL << 31) - 64 || static_cast<long long>(N) * IH * IW * IC >= (1LL << 31) || GK * OC >= (1LL << 40) ||
      taps * IC * OC >= (1LL << 31) || taps * GridZ > 65535)
    return CU32_E_DIM;

  // 1x1 / stride 1 / no padding: deltaW[OC, IC] = deltaY[GK, OC]^T * X[GK, IC], the plain A^T*B contraction
  if (FH == 1 && FW == 1 && sh == 1 && sw == 1 && ph == 0 && pw == 0) {
    GemmCall c{};
    c.A = dDY; c.B = dX; c.C = dDW; c.Cbuf = dBuf;
    c.M = OC; c.N = IC; c.K = static_cast<int>(GK); c.n_store = IC;
    c.a_mn = true; c.lda = OC; c.b_mn = true; c.ldb = IC; c.ldc = IC;
    c.batch = 1; c.sA = 0; c.sB = 0; c.sC = static_cast<long long>(OC) * IC;
    c.gz = GridZ; c.x3 = true; c.stream = st;
    return run_gemm(c);
  }

  if (!load_driver_entry_points() || !g_encode_im2col) return CU32_E_DRIVER;
  const int lower_w = -pw, lower_h = -ph;
  const int upper_w = lower_w + (OW - 1) * sw - (IW - 1);
  const int upper_h = lower_h + (OH - 1) * sh - (IH - 1);
  bool gather = g_force_gather.load() != 0 || lower_w < -128 || lower_h < -128 || upper_w < -128 || upper_w > 127 ||
                upper_h < -128 || upper_h > 127 || FW > 256 || FH > 256 || sw > 8 || sh > 8;

  const int zs = static_cast<int>(taps) * GridZ;
  int tile = pick_tile(OC, IC, zs);
  const int ctas = tile_ctas(tile), bn = tile_bn(tile);
  GemmParams p;
  std::memset(&p, 0, sizeof(p));
  if (int rc = make_map3(&p.tmA, dDY, OC, static_cast<uint64_t>(GK), 1, OC, static_cast<uint64_t>(GK) * OC, 32, 32, true))
    return rc;
  {
    cuuint64_t dims[4] = {static_cast<cuuint64_t>(IC), static_cast<cuuint64_t>(IW), static_cast<cuuint64_t>(IH),
                          static_cast<cuuint64_t>(N)};
    cuuint64_t strides[3] = {static_cast<cuuint64_t>(IC) * 4, static_cast<cuuint64_t>(IW) * IC * 4,
                             static_cast<cuuint64_t>(IH) * IW * IC * 4};
    int lower[2] = {lower_w, lower_h};
    int upper[2] = {upper_w, upper_h};
    cuuint32_t trav[4] = {1, static_cast<cuuint32_t>(sw), static_cast<cuuint32_t>(sh), 1};
    CUresult r = gather ? CUDA_ERROR_INVALID_VALUE
                        : g_encode_im2col(&p.tmB, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(dX), dims, strides,
                                          lower, upper, /*channelsPerPixel=*/32, /*pixelsPerColumn=*/32, trav,
                                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B,
                                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) gather = true;
    int drv = 0;   // same driver workaround as in conv_any
    if (cudaDriverGetVersion(&drv) == cudaSuccess && drv <= 13010 &&
        static_cast<long long>(N) * IH * IW * IC * 4 < 131072)
      reinterpret_cast<uint64_t*>(&p.tmB)[1] &= ~(1ULL << 21);
  }
  p.C = dDW; p.Cbuf = dBuf;
  p.ldc = static_cast<int>(taps) * IC;
  p.c_stride = static_cast<long long>(OC) * taps * IC;
  p.M = OC; p.N = IC;
  p.nkb_total = static_cast<int>((GK + 31) / 32);
  p.tiles_m = (OC + 128 * ctas - 1) / (128 * ctas);
  p.tiles_n = (IC + bn - 1) / bn;
  p.gz = GridZ;
  p.ztaps = static_cast<int>(taps);
  p.kc = g_kc.load();
  choose_rings(&p);
  p.vec4_ok = 1;
  p.tma_store = 0;   // a tap's columns end inside the row: register stores clip there
  p.conv_OW = OW; p.conv_OH = OH; p.conv_FW = FW; p.conv_IC = IC;
  p.conv_sw = sw; p.conv_sh = sh; p.conv_pw = pw; p.conv_ph = ph;
  p.gather = gather ? 1 : 0; p.g_img = dX; p.g_H = IH; p.g_W = IW; p.g_N = N;
  cudaError_t e;
  p.status = status_word_ptr(&e);
  if (!p.status) return static_cast<int>(e);
  e = launch_gemm_nn_im2col(tile, p, zs, st);
  if (e != cudaSuccess) return static_cast<int>(e);
  return static_cast<int>(cudaPeekAtLastError());
}

}  // namespace dragon

using namespace dragon;

// ==================================================================== exported C ABI
extern "C" {

int cu32_matMul(const int64_t* s, int n, const float* A, const float* B, float* C, int N, int M, int K) {
  return matmul_any(FORM_AB, true, s, n, 1, A, B, C, nullptr, N, M, K);
}
int cu32_matMulT1(const int64_t* s, int n, const float* A, const float* B, float* C, int N, int M, int K) {
  return matmul_any(FORM_T1, true, s, n, 1, A, B, C, nullptr, N, M, K);
}
int cu32_matMulT2(const int64_t* s, int n, const float* A, const float* B, float* C, int N, int M, int K) {
  return matmul_any(FORM_T2, true, s, n, 1, A, B, C, nullptr, N, M, K);
}
int cu32_matMulSK(const int64_t* s, int n, int GZ, const float* A, const float* B, float* C, float* Cbuf,
                  int N, int M, int K) {
  return matmul_any(FORM_AB, true, s, n, GZ, A, B, C, Cbuf, N, M, K);
}
int cu32_matMulT1SK(const int64_t* s, int n, int GZ, const float* A, const float* B, float* C,
                    float* Cbuf, int N, int M, int K) {
  return matmul_any(FORM_T1, true, s, n, GZ, A, B, C, Cbuf, N, M, K);
}
int cu32_matMulT2SK(const int64_t* s, int n, int GZ, const float* A, const float* B, float* C,
                    float* Cbuf, int N, int M, int K) {
  return matmul_any(FORM_T2, true, s, n, GZ, A, B, C, Cbuf, N, M, K);
}
// ---- product stored to several buffers at once (no counterpart in the reference, which runs on one GPU)
int cu32_matMul_replicated(const int64_t* s, int n, const float* A, const float* B, float* C, float* const* replicas,
                           int n_replicas, int N, int M, int K) {
  return matmul_any(FORM_AB, true, s, n, 1, A, B, C, nullptr, N, M, K, nullptr, 0, replicas, n_replicas);
}
int cu32_matMulT2_replicated(const int64_t* s, int n, const float* A, const float* B, float* C, float* const* replicas,
                             int n_replicas, int N, int M, int K) {
  return matmul_any(FORM_T2, true, s, n, 1, A, B, C, nullptr, N, M, K, nullptr, 0, replicas, n_replicas);
}
int cu32_matMul_mma(const int64_t* s, int n, const float* A, const float* B, float* C, int N, int M, int K) {
  return matmul_any(FORM_AB, false, s, n, 1, A, B, C, nullptr, N, M, K);
}
int cu32_matMulT1_mma(const int64_t* s, int n, const float* A, const float* B, float* C, int N, int M, int K) {
  return matmul_any(FORM_T1, false, s, n, 1, A, B, C, nullptr, N, M, K);
}
int cu32_matMulT2_mma(const int64_t* s, int n, const float* A, const float* B, float* C, int N, int M, int K) {
  return matmul_any(FORM_T2, false, s, n, 1, A, B, C, nullptr, N, M, K);
}

static int summary_any(int64_t stream, const float* dCbuf, float* dC, int part, int sizeC, const float* dBias,
                       int row_len, int width) {
  if (!dC || (part > 0 && !dCbuf)) return CU32_E_NULL;
  if (part < 0 || sizeC <= 0) return CU32_E_DIM;
  if (!aligned16(dC) || !aligned16(dCbuf) || (sizeC & 3)) return CU32_E_ALIGN;
  if (dBias) {
    if (row_len <= 0 || width <= 0 || width > row_len || sizeC % row_len) return CU32_E_DIM;
    if (!aligned16(dBias) || (row_len & 3)) return CU32_E_ALIGN;
  } else if (part == 0) {
    return CU32_OK;
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(static_cast<intptr_t>(stream));
  const int threads = 256;
  long long blocks = (static_cast<long long>(sizeC) / 4 + threads - 1) / threads;
  if (blocks > device_sm_count() * 16) blocks = device_sm_count() * 16;
  if (blocks < 1) blocks = 1;
  if (dBias)
    skbuf_summary_kernel<true><<<static_cast<unsigned>(blocks), threads, 0, st>>>(dCbuf, dC, part, sizeC, dBias,
                                                                                 row_len, width);
  else
    skbuf_summary_kernel<false><<<static_cast<unsigned>(blocks), threads, 0, st>>>(dCbuf, dC, part, sizeC, nullptr,
                                                                                  4, 4);
  return static_cast<int>(cudaPeekAtLastError());
}

int cu32_SKbuf_summary(int64_t stream, const float* dCbuf, float* dC, int part, int sizeC) {
  return summary_any(stream, dCbuf, dC, part, sizeC, nullptr, 0, 0);
}

// ---- Cuda_dconv3D_deltaW: weight gradient of the convolution (reference: the natives of the Java class
// z/dragon/engine/cuda/impl/math/Cuda_dconv3D_deltaW.java:288-640; their CUDA source is not published)
int cu32_dconv3D_deltaW(const int64_t* s, int n, const float* X, int IH, int IW, const float* dY, int OH, int OW,
                        float* dW, int FH, int FW, int N, int IC, int OC, int sh, int sw, int ph, int pw) {
  return deconvW_any(s, n, 1, X, IH, IW, dY, OH, OW, dW, nullptr, FH, FW, N, IC, OC, sh, sw, ph, pw);
}
int cu32_dconv3D_deltaW_W1(const int64_t* s, int n, const float* X, int IH, int IW, const float* dY, float* dW, int N,
                           int IC, int OC) {
  return deconvW_any(s, n, 1, X, IH, IW, dY, IH, IW, dW, nullptr, 1, 1, N, IC, OC, 1, 1, 0, 0);
}
int cu32_dconv3D_deltaW_buf_summary(int64_t stream, const float* dWbuf, float* dW, int part, int sizeW) {
  return summary_any(stream, dWbuf, dW, part, sizeW, nullptr, 0, 0);
}
int cu32_dconv3D_deltaW_GemmSK(const int64_t* s, int n, int GridZ, const float* X, int IH, int IW, const float* dY,
                               int OH, int OW, float* dW, float* dWbuf, int FH, int FW, int N, int IC, int OC,
                               int sh, int sw, int ph, int pw) {
  return deconvW_any(s, n, GridZ, X, IH, IW, dY, OH, OW, dW, dWbuf, FH, FW, N, IC, OC, sh, sw, ph, pw);
}
int cu32_dconv3D_deltaW_GemmV2SK(const int64_t* s, int n, int GridZ, const float* X, int IH, int IW, const float* dY,
                                 int OH, int OW, float* dW, float* dWbuf, int FH, int FW, int N, int IC, int OC,
                                 int sh, int sw, int ph, int pw) {
  return deconvW_any(s, n, GridZ, X, IH, IW, dY, OH, OW, dW, dWbuf, FH, FW, N, IC, OC, sh, sw, ph, pw);
}
int cu32_dconv3D_deltaW_GemmSK_W1(const int64_t* s, int n, int GridZ, const float* X, int IH, int IW, const float* dY,
                                  float* dW, float* dWbuf, int N, int IC, int OC) {
  return deconvW_any(s, n, GridZ, X, IH, IW, dY, IH, IW, dW, dWbuf, 1, 1, N, IC, OC, 1, 1, 0, 0);
}
// The Winograd natives (stride 1) are further names for the same contraction; the slice sizes and the
// transform's tile size n only steer the reference's own kernels.
#define CU32_DW_WINOGRAD(name, ...)                                                                              \
  int name(const int64_t* s, int n, int GridZ, int, int, __VA_ARGS__ const float* X, int IH, int IW, const float* dY, \
           int OH, int OW, float* dW, float* dWbuf, int FH, int FW, int N, int IC, int OC, int ph, int pw, int) {    \
    return deconvW_any(s, n, GridZ, X, IH, IW, dY, OH, OW, dW, dWbuf, FH, FW, N, IC, OC, 1, 1, ph, pw);            \
  }
CU32_DW_WINOGRAD(cu32_dconv3D_deltaW_Im2col_WinogradV2_SHW_s4_texture, )
CU32_DW_WINOGRAD(cu32_dconv3D_deltaW_Im2col_WinogradV2_SHW_s8_texture, )
CU32_DW_WINOGRAD(cu32_dconv3D_deltaW_Im2col_WinogradV2_SHW_s16_texture, int, )
#undef CU32_DW_WINOGRAD

// ---- contraction + bias row in one pass (no counterpart among the reference's natives: the Java
// engine runs Cuda_function.linear_dual2D_row(C, bias, 1, 1, 0) as a second kernel)
int cu32_matMul_biased(const int64_t* s, int n, const float* A, const float* B, float* C, const float* Bias,
                       int N, int M, int K, int width) {
  if (!Bias) return CU32_E_NULL;
  return matmul_any(FORM_AB, true, s, n, 1, A, B, C, nullptr, N, M, K, Bias, width);
}
int cu32_matMul_mma_biased(const int64_t* s, int n, const float* A, const float* B, float* C, const float* Bias,
                           int N, int M, int K, int width) {
  if (!Bias) return CU32_E_NULL;
  return matmul_any(FORM_AB, false, s, n, 1, A, B, C, nullptr, N, M, K, Bias, width);
}
int cu32_SKbuf_summary_biased(int64_t stream, const float* dCbuf, float* dC, const float* Bias, int part,
                              int sizeC, int M, int width) {
  if (!Bias) return CU32_E_NULL;
  return summary_any(stream, dCbuf, dC, part, sizeC, Bias, M, width);
}

// ---- batched
static int bmm_any(int form, bool x3, const int64_t* s, int n, const float* A, const float* B, float* C,
                   int Batch, int d0, int d1, int d2, int d3, bool scaled = false, float alpha = 1.0f) {
  cudaStream_t st;
  if (int rc = check_streams(s, n, &st)) return rc;
  if (Batch <= 0 || d0 <= 0 || d1 <= 0 || d2 <= 0 || d3 <= 0) return CU32_E_DIM;
  GemmCall c{};
  c.A = A; c.B = B; c.C = C; c.Cbuf = nullptr;
  c.batch = Batch; c.gz = 1; c.x3 = x3; c.stream = st;
  c.scale_on = scaled; c.alpha = alpha;
  if (form == FORM_AB) {            // (Batch, N, M, BK, AK)
    const int N = d0, M = d1, BK = d2, AK = d3;
    if (AK < BK) return CU32_E_DIM;
    c.M = N; c.N = M; c.K = BK; c.n_store = M;
    c.a_mn = false; c.lda = AK; c.sA = static_cast<long long>(N) * AK;
    c.b_mn = true;  c.ldb = M;  c.sB = static_cast<long long>(BK) * M;
    c.ldc = M; c.sC = static_cast<long long>(N) * M;
  } else if (form == FORM_T1) {     // (Batch, CN, AN, M, K)
    const int CN = d0, AN = d1, M = d2, K = d3;
    if (AN < CN) return CU32_E_DIM;
    c.M = CN; c.N = M; c.K = K; c.n_store = M;
    c.a_mn = true; c.lda = AN; c.sA = static_cast<long long>(K) * AN;
    c.b_mn = true; c.ldb = M;  c.sB = static_cast<long long>(K) * M;
    c.ldc = M; c.sC = static_cast<long long>(CN) * M;
  } else {                          // (Batch, N, CM, BM, K)
    const int N = d0, CM = d1, BM = d2, K = d3;
    if (CM < BM) return CU32_E_DIM;
    c.M = N; c.N = BM; c.K = K; c.n_store = CM;
    c.a_mn = false; c.lda = K; c.sA = static_cast<long long>(N) * K;
    c.b_mn = false; c.ldb = K; c.sB = static_cast<long long>(BM) * K;
    c.ldc = CM; c.sC = static_cast<long long>(N) * CM;
  }
  return run_gemm(c);
}

// ---- attention scores: batched A * B^T, scale and row softmax in one pass (no counterpart among the reference's
// natives: its attention block runs batchMatMulT2, linear2D (the 1/sqrt(d) scale), row_max, row_softmax and
// div2D_field as five kernels over the score tensor, nn/unit/complex/block/ImageMHA.java:67-68,
// CudaFloat32EngineBase.java:5738-5775)
}  // extern "C"
namespace dragon {
// Row softmax in place, one warp per row: y = exp(x - max) / sum over the first `width` columns of each row of
// `stride` floats, padding columns zeroed.  Used when a row does not fit the fused kernel.
__global__ void row_softmax_kernel(float* __restrict__ P, long long rows, int stride, int width) {
  const int lane = threadIdx.x & 31;
  const long long warps = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
  for (long long row = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); row < rows; row += warps) {
    float* x = P + row * stride;
    float m = -INFINITY;
    for (int c = lane; c < width; c += 32) m = fmaxf(m, x[c]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float sum = 0.f;
    for (int c = lane; c < width; c += 32) {
      const float e = expf(x[c] - m);
      x[c] = e;
      sum += e;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float rinv = 1.0f / sum;
    for (int c = lane; c < stride; c += 32) x[c] = c < width ? x[c] * rinv : 0.f;
  }
}
}  // namespace dragon
extern "C" {
int cu32_batchMatMulT2_softmax(const int64_t* s, int n, const float* A, const float* B, float* P, int Batch, int N,
                               int CM, int BM, int K, float alpha) {
  load_env_once();
  cudaStream_t st;
  if (int rc = check_streams(s, n, &st)) return rc;
  if (!A || !B || !P) return CU32_E_NULL;
  if (Batch <= 0 || N <= 0 || CM <= 0 || BM <= 0 || K <= 0 || CM < BM) return CU32_E_DIM;
  if ((K & 3) || (CM & 3) || !aligned16(A) || !aligned16(B) || !aligned16(P)) return CU32_E_ALIGN;
  if (static_cast<long long>(Batch) * N * CM >= (1LL << 40)) return CU32_E_DIM;
  const int nkb = (K + 31) / 32;
  if (CM > 512 || nkb > g_kc.load()) {
    // rows too long for the two TMEM buffers, or a reduction longer than one in-TMEM chunk (the softmax turns the
    // scores' absolute error into relative error of P, so the chunk is not stretched): scaled product, then a row
    // softmax in place
    if (int rc = bmm_any(FORM_T2, true, s, n, A, B, P, Batch, N, CM, BM, K, true, alpha)) return rc;
    const long long rows = static_cast<long long>(Batch) * N;
    long long blocks = (rows + 7) / 8;
    if (blocks > device_sm_count() * 16) blocks = device_sm_count() * 16;
    row_softmax_kernel<<<static_cast<unsigned>(blocks), 256, 0, st>>>(P, rows, CM, BM);
    return static_cast<int>(cudaPeekAtLastError());
  }
  if (!load_driver_entry_points()) return CU32_E_DRIVER;
  GemmParams p;
  std::memset(&p, 0, sizeof(p));
  const uint64_t nb = static_cast<uint64_t>(Batch);
  if (int rc = make_map3(&p.tmA, A, K, N, nb, K, static_cast<uint64_t>(N) * K, 32, 128, false)) return rc;
  if (int rc = make_map3(&p.tmB, B, K, BM, nb, K, static_cast<uint64_t>(BM) * K, 32, 128, false)) return rc;
  if (int rc = make_map3(&p.tmC, P, CM, N, nb, CM, static_cast<uint64_t>(N) * CM, 32, 32, false)) return rc;
  p.C = P; p.ldc = CM; p.c_stride = static_cast<long long>(N) * CM;
  p.M = N; p.N = CM;
  p.nkb_total = nkb;
  p.tiles_m = (N + 255) / 256;
  p.tiles_n = (CM + 255) / 256;
  p.unit_tiles = p.tiles_n;
  p.gz = 1;
  p.kc = nkb;            // the whole reduction is one chunk, so a tile's result is complete in TMEM
  choose_rings(&p);
  if (p.ring_raw == 0) { p.ring_raw = 3; p.ring_lo = 2; p.store_bufs = 1; }   // leaves room for the row statistics
  p.vec4_ok = 1; p.tma_store = 1;
  p.alpha = alpha; p.sm_width = BM;
  cudaError_t e;
  p.status = status_word_ptr(&e);
  if (!p.status) return static_cast<int>(e);
  g_last_tile = TILE_2x256;
  e = launch_gemm_kk_softmax(p, Batch, st);
  if (e != cudaSuccess) return static_cast<int>(e);
  return static_cast<int>(cudaPeekAtLastError());
}

// ---- data gradient / transposed convolution + bias row in one pass (no counterpart among the reference's natives:
// the Java engine's deconv3D_biased runs Cuda_function.linear_dual2D_row(Y, bias, 1, 1, 0) as a second kernel,
// CudaFloat32EngineBase.java:2620-2650).  Bias has IC entries (the channels of the output), width <= IC are real.
int cu32_dconv3D_deltaX_s1_biased(const int64_t* s, int n, const float* dY, int OH, int OW, const float* W, int FH,
                                  int FW, float* dX, int IH, int IW, int N, int IC, int OC, int ph, int pw,
                                  const float* Bias, int width) {
  if (!Bias) return CU32_E_NULL;
  return deconv_s1_any(s, n, dY, OH, OW, W, FH, FW, dX, IH, IW, N, IC, OC, ph, pw, Bias, width);
}
int cu32_dconv3D_deltaX_ksImsR_biased(const int64_t* s, int n, const float* dY, int OH, int OW, const float* CW, int FH,
                                      int FW, float* dX, int IH, int IW, int N, int IC, int OC, int sh, int sw, int ph,
                                      int pw, const float* Bias, int width) {
  if (!Bias) return CU32_E_NULL;
  return deconv_strided_any(s, n, dY, OH, OW, CW, true, FH, FW, dX, IH, IW, N, IC, OC, sh, sw, ph, pw, Bias, width);
}

// ---- batched contraction + scalar scale in one pass (no counterpart among the reference's natives: its
// attention block runs sdiv = linear2D(1/sqrt(d), X, 0) as a second kernel over the scores,
// nn/unit/complex/block/ImageMHA.java:67-68, Engine.java:4002, Cuda_function/type1_linear2D.cuh:40-58)
int cu32_batchMatMul_scaled(const int64_t* s, int n, const float* A, const float* B, float* C, int Batch, int N, int M,
                            int BK, int AK, float alpha) {
  return bmm_any(FORM_AB, true, s, n, A, B, C, Batch, N, M, BK, AK, true, alpha);
}
int cu32_batchMatMulT1_scaled(const int64_t* s, int n, const float* A, const float* B, float* C, int Batch, int CN,
                              int AN, int M, int K, float alpha) {
  return bmm_any(FORM_T1, true, s, n, A, B, C, Batch, CN, AN, M, K, true, alpha);
}
int cu32_batchMatMulT2_scaled(const int64_t* s, int n, const float* A, const float* B, float* C, int Batch, int N,
                              int CM, int BM, int K, float alpha) {
  return bmm_any(FORM_T2, true, s, n, A, B, C, Batch, N, CM, BM, K, true, alpha);
}

int cu32_batchMatMul(const int64_t* s, int n, const float* A, const float* B, float* C, int Batch, int N,
                     int M, int BK, int AK) {
  return bmm_any(FORM_AB, true, s, n, A, B, C, Batch, N, M, BK, AK);
}
int cu32_batchMatMul_texture(const int64_t* s, int n, const float* A, const float* B, float* C, int Batch,
                             int N, int M, int BK, int AK) {
  return bmm_any(FORM_AB, true, s, n, A, B, C, Batch, N, M, BK, AK);
}
int cu32_batchMatMulT1(const int64_t* s, int n, const float* A, const float* B, float* C, int Batch, int CN,
                       int AN, int M, int K) {
  return bmm_any(FORM_T1, true, s, n, A, B, C, Batch, CN, AN, M, K);
}
int cu32_batchMatMulT2(const int64_t* s, int n, const float* A, const float* B, float* C, int Batch, int N,
                       int CM, int BM, int K) {
  return bmm_any(FORM_T2, true, s, n, A, B, C, Batch, N, CM, BM, K);
}
int cu32_batchMatMulT2_texture(const int64_t* s, int n, const float* A, const float* B, float* C, int Batch,
                               int N, int CM, int BM, int K) {
  return bmm_any(FORM_T2, true, s, n, A, B, C, Batch, N, CM, BM, K);
}
int cu32_batchMatMul_mma(int useTexture, const int64_t* s, int n, const float* A, const float* B, float* C,
                         int Batch, int N, int M, int BK, int AK) {
  (void)useTexture;
  return bmm_any(FORM_AB, false, s, n, A, B, C, Batch, N, M, BK, AK);
}
int cu32_batchMatMulT1_mma(const int64_t* s, int n, const float* A, const float* B, float* C, int Batch,
                           int CN, int AN, int M, int K) {
  return bmm_any(FORM_T1, false, s, n, A, B, C, Batch, CN, AN, M, K);
}
int cu32_batchMatMulT2_mma(int useTexture, const int64_t* s, int n, const float* A, const float* B, float* C,
                           int Batch, int N, int CM, int BM, int K) {
  (void)useTexture;
  return bmm_any(FORM_T2, false, s, n, A, B, C, Batch, N, CM, BM, K);
}

// ---- convolution
int cu32_kernel_remode(int64_t stream, const float* dW, float* dCW, int FH, int FW, int OC, int IC) {
  if (!dW || !dCW) return CU32_E_NULL;
  if (FH <= 0 || FW <= 0 || OC <= 0 || IC <= 0) return CU32_E_DIM;
  const long long G = static_cast<long long>(FH) * FW * IC;
  if (G >= (1LL << 31) || G * OC >= (1LL << 31)) return CU32_E_DIM;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(static_cast<intptr_t>(stream));
  dim3 grid(static_cast<unsigned>((G + 31) / 32), static_cast<unsigned>((OC + 31) / 32));
  if (grid.y > 65535) return CU32_E_DIM;
  remode_kernel<<<grid, dim3(32, 8), 0, st>>>(dW, dCW, OC, static_cast<int>(G));
  return static_cast<int>(cudaPeekAtLastError());
}

int cu32_conv3D_GemmR(const int64_t* s, int n, const float* X, int IH, int IW, const float* W,
                      const float* CW, int FH, int FW, float* Y, int OH, int OW, int N, int IC, int OC,
                      int sh, int sw, int ph, int pw) {
  (void)CW;  // the tensor-map path reads W[OC][FH*FW*IC] directly; CW is the reference's operand layout
  return conv_any(true, s, n, X, IH, IW, W, FH, FW, Y, OH, OW, N, IC, OC, sh, sw, ph, pw);
}
int cu32_conv3D_GemmR_texture(const int64_t* s, int n, const float* X, int IH, int IW, const float* W,
                              const float* CW, int FH, int FW, float* Y, int OH, int OW, int N, int IC,
                              int OC, int sh, int sw, int ph, int pw) {
  (void)CW;
  return conv_any(true, s, n, X, IH, IW, W, FH, FW, Y, OH, OW, N, IC, OC, sh, sw, ph, pw);
}
int cu32_conv3D_GemmR_SGM(const int64_t* s, int n, const float* X, int IH, int IW, const float* W,
                          const float* CW, int FH, int FW, float* Y, int OH, int OW, int N, int IC, int OC,
                          int sh, int sw, int ph, int pw, int GM_slice) {
  (void)CW;
  if (GM_slice <= 0) return CU32_E_ARG;
  return conv_any(true, s, n, X, IH, IW, W, FH, FW, Y, OH, OW, N, IC, OC, sh, sw, ph, pw);
}
int cu32_conv3D_GemmR_texture_SGM(const int64_t* s, int n, const float* X, int IH, int IW, const float* W,
                                  const float* CW, int FH, int FW, float* Y, int OH, int OW, int N, int IC,
                                  int OC, int sh, int sw, int ph, int pw, int GM_slice) {
  (void)CW;
  if (GM_slice <= 0) return CU32_E_ARG;
  return conv_any(true, s, n, X, IH, IW, W, FH, FW, Y, OH, OW, N, IC, OC, sh, sw, ph, pw);
}
int cu32_conv3D_GemmR_biased(const int64_t* s, int n, const float* X, int IH, int IW, const float* W,
                             const float* CW, int FH, int FW, float* Y, int OH, int OW, int N, int IC, int OC,
                             int sh, int sw, int ph, int pw, const float* Bias, int width) {
  (void)CW;
  if (!Bias) return CU32_E_NULL;
  return conv_any(true, s, n, X, IH, IW, W, FH, FW, Y, OH, OW, N, IC, OC, sh, sw, ph, pw, Bias, width);
}
// The reference's V2 and Im2col-Winograd natives: same result through the same implicit GEMM.
int cu32_conv3DV2(int, const int64_t* s, int n, const float* X, int IH, int IW, const float* W, int FH, int FW,
                  float* Y, int OH, int OW, int N, int IC, int OC, int sh, int sw, int ph, int pw) {
  return conv_any(true, s, n, X, IH, IW, W, FH, FW, Y, OH, OW, N, IC, OC, sh, sw, ph, pw);
}
int cu32_conv3D_GemmV2R(int, const int64_t* s, int n, const float* X, int IH, int IW, const float* W,
                        const float* CW, int FH, int FW, float* Y, int OH, int OW, int N, int IC, int OC,
                        int sh, int sw, int ph, int pw) {
  (void)CW;
  return conv_any(true, s, n, X, IH, IW, W, FH, FW, Y, OH, OW, N, IC, OC, sh, sw, ph, pw);
}
#define DRAGON_WINOGRAD_ALIAS(name)                                                                        \
  int name(int, const int64_t* s, int n, const float* X, int IH, int IW, const float* W, const float* CW,  \
           int FH, int FW, float* Y, int OH, int OW, int N, int IC, int OC, int ph, int pw) {              \
    (void)CW;                                                                                              \
    return conv_any(true, s, n, X, IH, IW, W, FH, FW, Y, OH, OW, N, IC, OC, 1, 1, ph, pw);                 \
  }
#define DRAGON_WINOGRAD_ALIAS_SGM(name)                                                                    \
  int name(int, const int64_t* s, int n, const float* X, int IH, int IW, const float* W, const float* CW,  \
           int FH, int FW, float* Y, int OH, int OW, int N, int IC, int OC, int ph, int pw, int GM_slice) {\
    (void)CW;                                                                                              \
    if (GM_slice <= 0) return CU32_E_ARG;                                                                  \
    return conv_any(true, s, n, X, IH, IW, W, FH, FW, Y, OH, OW, N, IC, OC, 1, 1, ph, pw);                 \
  }
DRAGON_WINOGRAD_ALIAS(cu32_conv3D_Im2col_Winograd_s8_R_texture)
DRAGON_WINOGRAD_ALIAS_SGM(cu32_conv3D_Im2col_WinogradR_s8_texture_SGM)
DRAGON_WINOGRAD_ALIAS(cu32_conv3D_Im2col_Winograd_s16_R_texture)
DRAGON_WINOGRAD_ALIAS_SGM(cu32_conv3D_Im2col_WinogradR_s16_texture_SGM)
// ---- data gradient of the stride-1 convolution (the reference's Cuda_dconv3D_deltaX natives that
// need no stride handling); W is the forward filter W[OC][FH][FW][IC], read in place
int cu32_dconv3D_deltaX_s1(const int64_t* s, int n, const float* dY, int OH, int OW, const float* W, int FH, int FW,
                           float* dX, int IH, int IW, int N, int IC, int OC, int ph, int pw) {
  return deconv_s1_any(s, n, dY, OH, OW, W, FH, FW, dX, IH, IW, N, IC, OC, ph, pw);
}
int cu32_dconv3D_deltaX_s1_texture(const int64_t* s, int n, const float* dY, int OH, int OW, const float* W, int FH,
                                   int FW, float* dX, int IH, int IW, int N, int IC, int OC, int ph, int pw) {
  return deconv_s1_any(s, n, dY, OH, OW, W, FH, FW, dX, IH, IW, N, IC, OC, ph, pw);
}
int cu32_dconv3D_deltaX_s1_SGM(const int64_t* s, int n, const float* dY, int OH, int OW, const float* W, int FH,
                               int FW, float* dX, int IH, int IW, int N, int IC, int OC, int ph, int pw,
                               int GM_slice) {
  if (GM_slice <= 0) return CU32_E_ARG;
  return deconv_s1_any(s, n, dY, OH, OW, W, FH, FW, dX, IH, IW, N, IC, OC, ph, pw);
}
int cu32_dconv3D_deltaX_s1_texture_SGM(const int64_t* s, int n, const float* dY, int OH, int OW, const float* W,
                                       int FH, int FW, float* dX, int IH, int IW, int N, int IC, int OC, int ph,
                                       int pw, int GM_slice) {
  if (GM_slice <= 0) return CU32_E_ARG;
  return deconv_s1_any(s, n, dY, OH, OW, W, FH, FW, dX, IH, IW, N, IC, OC, ph, pw);
}
int cu32_dconv3D_deltaX_V2_s1(int, const int64_t* s, int n, const float* dY, int OH, int OW, const float* W, int FH,
                              int FW, float* dX, int IH, int IW, int N, int IC, int OC, int ph, int pw) {
  return deconv_s1_any(s, n, dY, OH, OW, W, FH, FW, dX, IH, IW, N, IC, OC, ph, pw);
}
int cu32_dconv3D_deltaX_W1(const int64_t* s, int n, const float* dY, const float* W, float* dX, int IH, int IW,
                           int N, int IC, int OC) {
  return deconv_s1_any(s, n, dY, IH, IW, W, 1, 1, dX, IH, IW, N, IC, OC, 0, 0);
}
int cu32_dconv3D_deltaX_W1_SGM(const int64_t* s, int n, const float* dY, const float* W, float* dX, int IH, int IW,
                               int N, int IC, int OC, int GM_slice) {
  if (GM_slice <= 0) return CU32_E_ARG;
  return deconv_s1_any(s, n, dY, IH, IW, W, 1, 1, dX, IH, IW, N, IC, OC, 0, 0);
}
// any stride, forward filter read in place (the reference's scatter-add formulation, A.cu:731-834)
int cu32_dconv3D_deltaX_crossAdd(const int64_t* s, int n, const float* dY, int OH, int OW, const float* W, int FH,
                                 int FW, float* dX, int IH, int IW, int N, int IC, int OC, int sh, int sw, int ph,
                                 int pw) {
  return deconv_strided_any(s, n, dY, OH, OW, W, false, FH, FW, dX, IH, IW, N, IC, OC, sh, sw, ph, pw);
}
int cu32_dconv3D_deltaX_crossAdd_SGM(const int64_t* s, int n, const float* dY, int OH, int OW, const float* W, int FH,
                                     int FW, float* dX, int IH, int IW, int N, int IC, int OC, int sh, int sw, int ph,
                                     int pw, int GM_slice) {
  if (GM_slice <= 0) return CU32_E_ARG;
  return deconv_strided_any(s, n, dY, OH, OW, W, false, FH, FW, dX, IH, IW, N, IC, OC, sh, sw, ph, pw);
}
int cu32_ks_remode(int64_t stream, const float* dW, int FH, int FW, float* dCW, int CFH, int CFW, int OC, int IC,
                   int sh, int sw) {
  return ks_remode_any(false, stream, dW, FH, FW, dCW, CFH, CFW, OC, IC, sh, sw);
}
int cu32_ks_remodev2(int64_t stream, const float* dW, int FH, int FW, float* dCW, int CFH, int CFW, int OC, int IC,
                     int sh, int sw) {
  return ks_remode_any(true, stream, dW, FH, FW, dCW, CFH, CFW, OC, IC, sh, sw);
}
// kernel-split natives: the filter arrives as the ks_remodev2 workspace
#define DRAGON_DX_KS(name)                                                                                       \
  int name(const int64_t* s, int n, const float* dY, int OH, int OW, const float* CW, int FH, int FW, float* dX, \
           int IH, int IW, int N, int IC, int OC, int sh, int sw, int ph, int pw) {                              \
    return deconv_strided_any(s, n, dY, OH, OW, CW, true, FH, FW, dX, IH, IW, N, IC, OC, sh, sw, ph, pw);        \
  }
#define DRAGON_DX_KS_SGM(name)                                                                                   \
  int name(const int64_t* s, int n, const float* dY, int OH, int OW, const float* CW, int FH, int FW, float* dX, \
           int IH, int IW, int N, int IC, int OC, int sh, int sw, int ph, int pw, int GM_slice) {                \
    if (GM_slice <= 0) return CU32_E_ARG;                                                                        \
    return deconv_strided_any(s, n, dY, OH, OW, CW, true, FH, FW, dX, IH, IW, N, IC, OC, sh, sw, ph, pw);        \
  }
#define DRAGON_DX_KS2(name)                                                                                      \
  int name(const int64_t* s, int n, const float* dY, int OH, int OW, const float* CW, int FH, int FW, float* dX, \
           int IH, int IW, int N, int IC, int OC, int ph, int pw) {                                              \
    return deconv_strided_any(s, n, dY, OH, OW, CW, true, FH, FW, dX, IH, IW, N, IC, OC, 2, 2, ph, pw);          \
  }
#define DRAGON_DX_KS2_SGM(name)                                                                                  \
  int name(const int64_t* s, int n, const float* dY, int OH, int OW, const float* CW, int FH, int FW, float* dX, \
           int IH, int IW, int N, int IC, int OC, int ph, int pw, int GM_slice) {                                \
    if (GM_slice <= 0) return CU32_E_ARG;                                                                        \
    return deconv_strided_any(s, n, dY, OH, OW, CW, true, FH, FW, dX, IH, IW, N, IC, OC, 2, 2, ph, pw);          \
  }
DRAGON_DX_KS(cu32_dconv3D_deltaX_kernelSplit)
DRAGON_DX_KS_SGM(cu32_dconv3D_deltaX_kernelSplit_SGM)
DRAGON_DX_KS(cu32_dconv3D_deltaX_ksImsR)
DRAGON_DX_KS_SGM(cu32_dconv3D_deltaX_ksImsR_SGM)
DRAGON_DX_KS(cu32_dconv3D_deltaX_ksImsR_texture)
DRAGON_DX_KS_SGM(cu32_dconv3D_deltaX_ksImsR_texture_SGM)
DRAGON_DX_KS2(cu32_dconv3D_deltaX_ksIms2R)
DRAGON_DX_KS2_SGM(cu32_dconv3D_deltaX_ksIms2R_SGM)
DRAGON_DX_KS2(cu32_dconv3D_deltaX_ksIms2R_texture)
DRAGON_DX_KS2_SGM(cu32_dconv3D_deltaX_ksIms2R_texture_SGM)
int cu32_dconv3D_deltaX_ksV2_Ims2R(int, const int64_t* s, int n, const float* dY, int OH, int OW, const float* CW,
                                   int FH, int FW, float* dX, int IH, int IW, int N, int IC, int OC, int ph, int pw) {
  return deconv_strided_any(s, n, dY, OH, OW, CW, true, FH, FW, dX, IH, IW, N, IC, OC, 2, 2, ph, pw);
}

#define DRAGON_DX_WINOGRAD(name)                                                                                \
  int name(int, const int64_t* s, int n, const float* dY, int OH, int OW, const float* W, int FH, int FW,       \
           float* dX, int IH, int IW, int N, int IC, int OC, int ph, int pw) {                                  \
    return deconv_s1_any(s, n, dY, OH, OW, W, FH, FW, dX, IH, IW, N, IC, OC, ph, pw);                           \
  }
#define DRAGON_DX_WINOGRAD_SGM(name)                                                                            \
  int name(int, const int64_t* s, int n, const float* dY, int OH, int OW, const float* W, int FH, int FW,       \
           float* dX, int IH, int IW, int N, int IC, int OC, int ph, int pw, int GM_slice) {                    \
    if (GM_slice <= 0) return CU32_E_ARG;                                                                       \
    return deconv_s1_any(s, n, dY, OH, OW, W, FH, FW, dX, IH, IW, N, IC, OC, ph, pw);                           \
  }
DRAGON_DX_WINOGRAD(cu32_dconv3D_deltaX_Im2col_Winograd_s8_texture)
DRAGON_DX_WINOGRAD_SGM(cu32_dconv3D_deltaX_Im2col_Winograd_s8_texture_SGM)
DRAGON_DX_WINOGRAD(cu32_dconv3D_deltaX_Im2col_Winograd_s16_texture)
DRAGON_DX_WINOGRAD_SGM(cu32_dconv3D_deltaX_Im2col_Winograd_s16_texture_SGM)

int cu32_conv3D_GemmR_W1(const int64_t* s, int n, const float* X, int IH, int IW, const float* W,
                         const float* CW, float* Y, int N, int IC, int OC) {
  (void)CW;
  return conv_any(true, s, n, X, IH, IW, W, 1, 1, Y, IH, IW, N, IC, OC, 1, 1, 0, 0);
}
int cu32_conv3D_GemmR_W1_SGM(const int64_t* s, int n, const float* X, int IH, int IW, const float* W,
                             const float* CW, float* Y, int N, int IC, int OC, int GM_slice) {
  (void)CW;
  if (GM_slice <= 0) return CU32_E_ARG;
  return conv_any(true, s, n, X, IH, IW, W, 1, 1, Y, IH, IW, N, IC, OC, 1, 1, 0, 0);
}
int cu32_conv3D(const int64_t* s, int n, const float* X, int IH, int IW, const float* W, int FH, int FW,
                float* Y, int OH, int OW, int N, int IC, int OC, int sh, int sw, int ph, int pw) {
  return conv_any(true, s, n, X, IH, IW, W, FH, FW, Y, OH, OW, N, IC, OC, sh, sw, ph, pw);
}
int cu32_conv3D_texture(const int64_t* s, int n, const float* X, int IH, int IW, const float* W, int FH,
                        int FW, float* Y, int OH, int OW, int N, int IC, int OC, int sh, int sw, int ph,
                        int pw) {
  return conv_any(true, s, n, X, IH, IW, W, FH, FW, Y, OH, OW, N, IC, OC, sh, sw, ph, pw);
}
int cu32_conv3D_np(const int64_t* s, int n, const float* X, int IH, int IW, const float* W, int FH, int FW,
                   float* Y, int OH, int OW, int N, int IC, int OC, int sh, int sw) {
  return conv_any(true, s, n, X, IH, IW, W, FH, FW, Y, OH, OW, N, IC, OC, sh, sw, 0, 0);
}
int cu32_conv3D_W1(const int64_t* s, int n, const float* X, int IH, int IW, const float* W, float* Y, int N,
                   int IC, int OC) {
  return conv_any(true, s, n, X, IH, IW, W, 1, 1, Y, IH, IW, N, IC, OC, 1, 1, 0, 0);
}

// ---- split-K without any allocation
// Partial products of cu32_matMulT1SK_noalloc live here instead of in a caller buffer.
// One instance per device that loads the library, held until the process exits.
static __device__ __align__(256) float g_splitk_scratch[CU32_NOALLOC_SCRATCH_FLOATS];

// In host code the array's name only stands for the symbol; the device address has to be
// asked for, once per device, while that device is current.
static float* splitk_scratch_ptr(cudaError_t* err) {
  static std::atomic<float*> cache[64];
  int dev = 0;
  *err = cudaGetDevice(&dev);
  if (*err != cudaSuccess) return nullptr;
  float* p = cache[dev & 63].load(std::memory_order_acquire);
  if (p) return p;
  float* sym = nullptr;
  *err = cudaGetSymbolAddress(reinterpret_cast<void**>(&sym), g_splitk_scratch);
  if (*err != cudaSuccess) return nullptr;
  cache[dev & 63].store(sym, std::memory_order_release);
  return sym;
}

int cu32_matMulT1SK_noalloc(const int64_t* s, int n, int GZ, const float* A, const float* B, float* C,
                            int N, int M, int K) {
  cudaStream_t st;
  if (int rc = check_streams(s, n, &st)) return rc;
  if (N <= 0 || M <= 0 || K <= 0) return CU32_E_DIM;
  if (GZ < 1) return CU32_E_ARG;
  const long long need = static_cast<long long>(GZ - 1) * N * M;
  if (need > CU32_NOALLOC_SCRATCH_FLOATS) return CU32_E_SCRATCH;
  // everything the two launches would refuse is refused before the first one writes into C
  if (!A || !B || !C) return CU32_E_NULL;
  if (!aligned16(A) || !aligned16(B) || !aligned16(C) || (N & 3) || (M & 3)) return CU32_E_ALIGN;
  cudaError_t e;
  float* scratch = splitk_scratch_ptr(&e);
  if (!scratch) return static_cast<int>(e);
  // Every slice overwrites its whole partial buffer (slices without k-blocks write zeros),
  // so nothing of an earlier call's contents is ever read.
  if (int rc = matmul_any(FORM_T1, true, s, n, GZ, A, B, C, GZ > 1 ? scratch : nullptr, N, M, K)) return rc;
  if (GZ == 1) return CU32_OK;
  return cu32_SKbuf_summary(s[0], scratch, C, GZ - 1, N * M);
}

// ---- self-test of the bounded waits
}  // extern "C"
namespace dragon {
// One warp waits on an mbarrier that nobody ever arrives at, with a short limit; the wait runs out, the
// kernel records its give-up code in the status word exactly as the contraction kernel's roles do, and
// returns normally.
__global__ void selftest_wait_kernel(int* status, long long limit_cycles) {
  __shared__ __align__(8) uint64_t bar;
  __shared__ volatile int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    ptx::mbar_init(ptx::smem_u32(&bar), 1);
    ptx::fence_mbar_init();
  }
  __syncthreads();
  const bool done = ptx::mbar_wait(ptx::smem_u32(&bar), 0u, &abort_flag, limit_cycles);
  if (!done && threadIdx.x == 0) atomicCAS(status, 0, (ROLE_SELFTEST << 24) | (1 << 16) | 42);
}
}  // namespace dragon
extern "C" {
int cu32_selftest_wait_giveup(int64_t stream, long long limit_cycles) {
  if (limit_cycles < 1 || limit_cycles > 100000000LL) return CU32_E_ARG;   // at most ~50 ms
  cudaError_t e;
  int* status = status_word_ptr(&e);
  if (!status) return static_cast<int>(e);
  selftest_wait_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(static_cast<intptr_t>(stream))>>>(status, limit_cycles);
  return static_cast<int>(cudaPeekAtLastError());
}

// ---- library control
int cu32_tune(const char* key, int value) {
  load_env_once();
  if (!key) return CU32_E_ARG;
  if (!std::strcmp(key, "kc")) { if (value < 1) return CU32_E_ARG; g_kc = value; return CU32_OK; }
  if (!std::strcmp(key, "kc_fast")) { if (value < 1) return CU32_E_ARG; g_kc_fast = value; return CU32_OK; }
  if (!std::strcmp(key, "tile")) { if (value < -1 || value >= TILE_COUNT) return CU32_E_ARG; g_tile = value; return CU32_OK; }
  if (!std::strcmp(key, "l2hint")) { if (value < 0 || value > 2) return CU32_E_ARG; g_l2hint = value; return CU32_OK; }
  if (!std::strcmp(key, "ring_raw")) { if (value < 0 || value > 8) return CU32_E_ARG; g_ring_raw = value; return CU32_OK; }
  if (!std::strcmp(key, "ring_lo")) { if (value < 0 || value > 8) return CU32_E_ARG; g_ring_lo = value; return CU32_OK; }
  if (!std::strcmp(key, "store_bufs")) { if (value < 0 || value > 2) return CU32_E_ARG; g_store_bufs = value; return CU32_OK; }
  if (!std::strcmp(key, "arrive_release")) { g_arrive_release = value ? 1 : 0; return CU32_OK; }
  if (!std::strcmp(key, "clock")) { g_clock_on = value ? 1 : 0; return CU32_OK; }
  if (!std::strcmp(key, "gather")) { g_force_gather = value ? 1 : 0; return CU32_OK; }
  if (!std::strcmp(key, "phase_overlap")) { g_phase_overlap = value ? 1 : 0; return CU32_OK; }
  if (!std::strcmp(key, "rep_lazy")) { g_rep_lazy = value ? 1 : 0; return CU32_OK; }
  if (!std::strcmp(key, "ring_paired")) { g_ring_paired = value ? 1 : 0; return CU32_OK; }
  if (!std::strcmp(key, "ring_fixed")) { g_ring_fixed = value ? 1 : 0; return CU32_OK; }
  if (!std::strcmp(key, "phase_fused")) { g_phase_fused = value ? 1 : 0; return CU32_OK; }
  if (!std::strcmp(key, "sm_reserve")) { if (value < 0 || value > 1024) return CU32_E_ARG; g_sm_reserve = value; return CU32_OK; }
  return CU32_E_ARG;
}
int cu32_get_tune(const char* key, int* value) {
  load_env_once();
  if (!key || !value) return CU32_E_ARG;
  if (!std::strcmp(key, "kc")) { *value = g_kc; return CU32_OK; }
  if (!std::strcmp(key, "kc_fast")) { *value = g_kc_fast; return CU32_OK; }
  if (!std::strcmp(key, "tile")) { *value = g_tile; return CU32_OK; }
  if (!std::strcmp(key, "l2hint")) { *value = g_l2hint; return CU32_OK; }
  if (!std::strcmp(key, "ring_raw")) { *value = g_ring_raw; return CU32_OK; }
  if (!std::strcmp(key, "ring_lo")) { *value = g_ring_lo; return CU32_OK; }
  if (!std::strcmp(key, "store_bufs")) { *value = g_store_bufs; return CU32_OK; }
  if (!std::strcmp(key, "arrive_release")) { *value = g_arrive_release; return CU32_OK; }
  if (!std::strcmp(key, "clock")) { *value = g_clock_on; return CU32_OK; }
  if (!std::strcmp(key, "gather")) { *value = g_force_gather; return CU32_OK; }
  if (!std::strcmp(key, "phase_overlap")) { *value = g_phase_overlap; return CU32_OK; }
  if (!std::strcmp(key, "rep_lazy")) { *value = g_rep_lazy; return CU32_OK; }
  if (!std::strcmp(key, "ring_paired")) { *value = g_ring_paired; return CU32_OK; }
  if (!std::strcmp(key, "ring_fixed")) { *value = g_ring_fixed; return CU32_OK; }
  if (!std::strcmp(key, "phase_fused")) { *value = g_phase_fused; return CU32_OK; }
  if (!std::strcmp(key, "sm_reserve")) { *value = g_sm_reserve; return CU32_OK; }
  if (!std::strcmp(key, "last_tile")) { *value = g_last_tile; return CU32_OK; }
  return CU32_E_ARG;
}
int cu32_read_status(int* status) {
  if (!status) return CU32_E_NULL;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return static_cast<int>(e);
  e = cudaMemcpyFromSymbol(status, g_status_word, sizeof(int));
  if (e != cudaSuccess) return static_cast<int>(e);
  const int zero = 0;
  e = cudaMemcpyToSymbol(g_status_word, &zero, sizeof(int));
  return static_cast<int>(e);
}
int cu32_read_clock(unsigned long long* out3) {
  if (!out3) return CU32_E_NULL;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return static_cast<int>(e);
  unsigned long long v[4] = {0, 0, 0, 0};
  e = cudaMemcpyFromSymbol(v, g_clock_acc, sizeof(v));
  if (e != cudaSuccess) return static_cast<int>(e);
  out3[0] = v[0]; out3[1] = v[1]; out3[2] = v[2];
  const unsigned long long zero[4] = {0, 0, 0, 0};
  return static_cast<int>(cudaMemcpyToSymbol(g_clock_acc, zero, sizeof(zero)));
}
const char* cu32_version(void) { return "dragon_cu32 0.1 sm_100a"; }

}  // extern "C"
