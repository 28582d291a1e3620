// FP32-accurate dense contraction on Blackwell tensor cores.
//
//   C[M,N] = A[M,K] * B[K,N]      (FP32 in, FP32 out, BLAS letters)
//
// One kernel template covers every entry point of the Cu32 matMul / batchMatMul /
// implicit-GEMM convolution family: the operand "major-ness" (which axis is
// contiguous in memory) is a template flag per operand, the batch index or the
// split-K slice rides on the tile index, and one operand can be gathered from an
// NHWC feature map by an im2col-mode tensor map: the A operand for the convolution and
// its data gradient (rows = output pixels, K = filter taps x channels), the B operand
// for its weight gradient (K = output pixels, one filter tap per z index).  Output rows
// may be strided pixels of an image (one phase of a strided data gradient).
//
// Arithmetic.  Each FP32 input x is used as
//     hi = tf32_trunc(x)          lo = tf32_round(x - hi)
// where hi is what the tensor core itself makes of an FP32 operand (it ignores the low
// 13 mantissa bits), so the tile as TMA wrote it serves as hi and only lo is written, next
// to it in shared memory.  The product is formed as  lo*hi + hi*lo + hi*hi  on
// tcgen05.mma kind::tf32 (the lo*lo term, below 2^-20 relative, is dropped).  The tensor
// core accumulates in FP32 inside TMEM, but truncates the accumulator after every
// instruction; it is therefore only trusted for `kc` k-blocks (one "chunk"):
// drain warps then add the chunk to FP32 register accumulators with
// round-to-nearest adds, so the length of any truncating accumulation chain is
// bounded regardless of K.
//
// The kernel is persistent: the grid is one CTA (or CTA pair) per SM and each walks
// the tile list with a fixed stride, so the drain and store of one tile overlap
// the loads and MMAs of the next; pipeline-stage and TMEM-buffer phases simply
// keep counting across tiles.
//
// Roles inside a CTA of 16 warps:
//   warp 0        TMA producer      global -> shared (raw FP32 tiles, 128B swizzle)
//   warp 1        MMA issuer        one thread issues tcgen05.mma, commits to mbarriers
//   warps 2..7    splitters         shared -> shared: raw tile -> lo tile beside it
//   warps 8..15   drainers          TMEM -> registers (sum of chunks) -> global
// With CTAS == 2 two CTAs of a cluster form one 256-row tile: each loads and
// splits its own half of A and of B, the even CTA issues cta_group::2 MMAs, and
// each CTA drains its own 128 TMEM lanes.
//
// Every mbarrier wait is bounded (see sm100_ptx.cuh).  A role that gives up
// records (role, stage, iteration) in the status word, raises the CTA's abort
// flag, and all roles fall through to the common exit, which frees TMEM.
#pragma once
#include "sm100_ptx.cuh"

namespace dragon {

// One further phase of a strided data gradient (GemmParams::phx): what differs from phase 0, whose values are the
// GemmParams fields of the same meaning.
struct alignas(64) GemmPhase {
  CUtensorMap tmA;   // im2col map over deltaY with this phase's window corners
  CUtensorMap tmB;   // this phase's filter slot (or the filter itself)
  float* C;          // first pixel of the phase in deltaX
  int M;             // output pixels of the phase (rows)
  int nkb;           // k-blocks of its reduction
  int OH, OW, FW;    // conv_OH, conv_OW, conv_FW of the phase
  int pw, ph;        // conv_pw, conv_ph
  int tap_base, tap_sy, tap_sx;
  int os_uv, os_v;
};

struct GemmParams {
  CUtensorMap tmA;      // K-major A: dims (K, M, batch), box (32, 128, 1)
                        // MN-major A: dims (M, K, batch), box (32, 32, 1)
                        // im2col A: NHWC dims (C, W, H, N), 32 channels x 128 pixels
  CUtensorMap tmB;      // K-major B: dims (K, N, batch), box (32, BN/CTAS, 1)
                        // MN-major B: dims (N, K, batch), box (32, 32, 1)
  CUtensorMap tmC;      // output C: dims (N, M, batches), box (32, 32, 1), 128B swizzle
  CUtensorMap tmCbuf;   // split-K partial buffers: dims (N, M, gz-1), same box
  CUtensorMap tmRep[7];  // further copies of the output (same dims and box as tmC), e.g. the same rows of a gathered
                         // output in the memory of the other GPUs of an NVLink domain, mapped into this process
  int n_rep;             // how many of them are valid: every store to C is repeated to each (stores only, never loads)
  float* rep_ptr[7];     // the same copies as plain pointers (same pitch as C), for the lazy mode below
  int rep_lazy;          // 1: the drain warps store a finished block to C only and carry it to the copies while the
                         // next tile is being multiplied - 16-byte loads of C from L2, 16-byte stores to every
                         // copy, a row segment at a time between two drains - so that the links to the other GPUs
                         // see a steady stream instead of every CTA's whole tile at once (one batch, no split-K)
  float* C;             // output of batch 0 / split-K slice 0
  const float* bias;    // optional row vector added to every output row before the store (gz == 1 only)
  int bias_width;       // columns < bias_width get acc + bias[col]; columns >= bias_width are stored as 0
  float* Cbuf;          // split-K: outputs of slices 1..gz-1, c_stride floats apart
  long long ldc;        // row pitch of C in floats
  long long c_stride;   // floats between consecutive batches (or Cbuf slices)
  int M, N;             // rows / columns of C to store
  int nkb_total;        // k-blocks of 32 in the whole reduction (before split-K)
  int tiles_m, tiles_n; // tile grid; a tile is (128*CTAS) x BN
  int gz;               // > 1: tiles run over gz split-K slices; else over zcount batches
  int zcount;           // batches (gz == 1) or slices (= gz) folded into the tile index
  int kc;               // k-blocks accumulated in TMEM before a drain (>= 1)
  int flush_chunks;     // chunks summed in registers before the sums go to memory (>= 1): the first flush of a
                        // tile stores, later ones add to what is there, so no FP32 register sum grows longer
  int vec4_ok;          // C, ldc and c_stride allow 16-byte stores
  int tma_store;        // tmC / tmCbuf are valid: store through shared memory + TMA
  int l2_hints;         // load A with evict-last and B with evict-first L2 priority
  int* status;          // device word, 0 = ok; first give-up code otherwise
  unsigned long long* clock_acc;   // optional: {SM cycles, nanoseconds, launches} summed by CTA 0 of every launch
  // Shared-memory rings (sized by the host within the 227 KB a CTA may use).  A k-block's raw tiles
  // occupy a slot of the raw ring from the TMA issue until its MMAs have completed; its lo tiles
  // occupy a slot of the (shorter or equal) lo ring only from the split until then.  Memory-bound
  // shapes trade lo slots for raw slots: more loads in flight against the HBM latency.
  int ring_raw;         // raw slots, 2..8
  int ring_lo;          // lo slots, 1..ring_raw (FP32-accurate mode only)
  int store_bufs;       // 4 KB store-staging tiles per drain warp, 1 or 2
  int ring_paired;      // equally long rings: lo tiles interleaved with the raw tiles (1) or in a ring of their own (0)
  int ring_fixed;       // set by the launcher: 1 = the rings are the configuration's default, 2 = its below-ridge
                        // geometry (GemmCfg::ALT_*): use that compile-time path; 0 = the launch parameters
  int arrive_release;   // debugging aid: remote mbarrier arrives carry a cluster-scope release
  int overlap_prev;     // host side only: this launch may start while the previous launch on the stream is still
                        // running (it does not depend on its results - the phases of a strided data gradient)
  int sm_reserve;       // SMs the persistent grid leaves free (for a collective's kernels running beside it)
  // im2col geometry (A gathered from an NHWC feature map); unused otherwise.
  // The reduction index runs over (fh, fw, ic) with every filter tap padded to
  // conv_icb blocks of 32 channels, so a k-block never straddles two taps.
  int conv_OW, conv_OH, conv_FW, conv_IC, conv_icb, conv_sw, conv_sh, conv_pw, conv_ph;
  // Data-gradient forms (im2col A, MN-major B): the filter is a stack of [K x N] matrices, one per tap.
  // The tap a k-block needs is tap_base + tap_sy * fh + tap_sx * fw (fh, fw: the tap of the im2col load), which
  // expresses reversed and strided tap orders over a filter that stays where it is.
  int tap_base, tap_sy, tap_sx;
  // Geometries no im2col tensor map can express (strides above 8, window corners outside +-128, taps above 255):
  // the producer warp gathers the image operand itself with plain loads into the same swizzled tile.
  int gather;           // 1: gather instead of the im2col-mode tensor map
  const float* g_img;   // the NHWC tensor the walk runs over (X, or deltaY for the data gradient)
  int g_H, g_W, g_N;    // its spatial extents and image count; its channel count is conv_IC
  int bmap_order;       // 0: B map coordinates (n, tap, k) - filter W[k][tap][n];  1: (n, k, tap) - filter CW[tap][k][n]
  // Strided output rows (data gradient for strides > 1): row -> (image, u, v) -> element offset
  // image * os_sn + u * os_su + v * os_sv; stores go straight from registers.
  int scale_on;         // multiply every output element by alpha on its way out (one FP32 rounding)
  float alpha;
  int unit_tiles;       // tiles a CTA (pair) takes in a row before moving on: 1, or tiles_n in the softmax mode
  int sm_width;         // softmax mode: columns < sm_width take part, the others (pitch padding) are stored as 0
  int ztaps;            // > 0: weight gradient, the z index is slice * ztaps + filter tap
  int os_on, os_uv, os_v;
  long long os_sn, os_su, os_sv;
  // Strided data gradient in one launch: n_phases > 1 phases (at most 4) whose tiles are taken in turn - a CTA (pair)
  // works through tile j of every phase before it moves to its next j - so the drain and stores of a short
  // phase's tile run under the MMAs of the next, longer one.  Phase 0 is described by the fields above.
  int n_phases;
  GemmPhase phx[3];
};

enum GemmRole : int { ROLE_TMA = 1, ROLE_SPLIT = 2, ROLE_MMA = 3, ROLE_MMA_TMEM = 4, ROLE_DRAIN = 5, ROLE_SELFTEST = 7 };

template <int BN_, int CTAS_, bool A_MN_, bool B_MN_, bool X3_, bool IM2COL_ = false, bool SOFTMAX_ = false,
          bool REP_ = false>
struct GemmCfg {
  static constexpr int BN = BN_, CTAS = CTAS_;
  static constexpr bool A_MN = A_MN_, B_MN = B_MN_, X3 = X3_, IM2COL = IM2COL_;
  // SOFTMAX: the rows of the product (at most 512 columns: the two TMEM buffers side by side) are normalised
  // with a softmax before they leave the SM - the attention scores never exist in memory.
  static constexpr bool SOFTMAX = SOFTMAX_;
  // REP: the output is kept in up to seven further copies (GemmParams::tmRep / rep_ptr); the other
  // instantiations carry none of that code.
  static constexpr bool REP = REP_;
  static_assert(!SOFTMAX_ || (BN_ == 256 && CTAS_ == 2 && X3_ && !A_MN_ && !B_MN_ && !IM2COL_),
                "the row softmax is built on the 256x256 pair tile of the A * B^T form");
  static constexpr int BM = 128;            // rows of A (and TMEM lanes) per CTA
  static constexpr int BK = 32;             // one 128-byte swizzle row of FP32
  static constexpr int BN_CTA = BN / CTAS;  // B columns staged per CTA
  static constexpr int A_BYTES = BM * BK * 4;
  static constexpr int B_BYTES = BN_CTA * BK * 4;
  static constexpr int HI_BYTES = A_BYTES + B_BYTES;   // bytes one k-block brings in by TMA: a raw slot [A][B]
  // Shared memory: [raw ring][lo ring (FP32-accurate mode)][store staging]; the ring lengths are launch
  // parameters.  MAX_DYN_SMEM leaves room for the static barriers inside the 227 KB a CTA may use.
  static constexpr int MAX_DYN_SMEM = (SOFTMAX_ ? 216 : 226) * 1024;   // the softmax mode keeps 4 KB of row statistics in static shared memory (once per compiled ring geometry)
  static constexpr int MAX_RING = 8;
  static constexpr int STAGING_TILE = 4096;   // one 32x32 FP32 piece
  // the default, balanced rings: as many (raw + lo) pairs as fit beside one staging tile per drain warp
  static constexpr int PAIR_BYTES = HI_BYTES * (X3 ? 2 : 1);
  static constexpr int STAGES_RAW = (MAX_DYN_SMEM - 1024 - 8 * STAGING_TILE) / PAIR_BYTES;
  static constexpr int STAGES = STAGES_RAW > MAX_RING ? MAX_RING : STAGES_RAW;
  // the below-ridge geometry (measured on the attention-shaped batched products): 128x64 one-CTA tile 6 raw + 2 lo
  // slots, 256x256 pair tile 3 + 2 with two staging tiles per drain warp (3 + 2 + 1 with the fused softmax, which
  // needs the room for its row statistics); 0 = the configuration has none
  static constexpr bool ALT_OK = X3 && !IM2COL_ && ((BN == 64 && CTAS == 1) || (BN == 256 && CTAS == 2));
  static constexpr int ALT_RAW = !ALT_OK ? 0 : (BN == 64 ? 6 : 3);
  static constexpr int ALT_LO = !ALT_OK ? 0 : 2;
  static constexpr int ALT_BUFS = !ALT_OK ? 0 : (BN == 64 || SOFTMAX_ ? 1 : 2);
  static constexpr int TMEM_NEED = 2 * BN;
  static constexpr int TMEM_COLS = TMEM_NEED <= 32 ? 32 : TMEM_NEED <= 64 ? 64 : TMEM_NEED <= 128 ? 128
                                   : TMEM_NEED <= 256 ? 256 : 512;
  static constexpr int THREADS = 512;
  static constexpr int SPLIT_WARP0 = 2, SPLIT_WARPS = 6;
  static constexpr int DRAIN_WARP0 = 8, DRAIN_WARPS = 8;
  static constexpr int CW = BN / 2;          // columns per drain warp
  static constexpr bool REALLOC = CW >= 64;  // drainers need more than the 128 registers a 512-thread CTA starts with
  // register budgets after reallocation (256 threads each side, 64 K registers per SM)
  static constexpr int REGS_MOVERS = 72;
  static constexpr int REGS_DRAINERS = 184;
  static_assert(BN == 64 || BN == 128 || BN == 256, "BN");
  static_assert(TMEM_NEED <= 512, "TMEM");
  static_assert(STAGES >= 2, "stages");
  // IM2COL with a K-major A: the A tile is an im2col walk over the image (convolution, data gradient).
  // IM2COL with an MN-major A: the B tile is the walk and the reduction runs over output pixels
  // (weight gradient: deltaW = deltaY^T * im2col(X), one filter tap per z index).
  static constexpr bool IM2COL_A = IM2COL && !A_MN;
  static constexpr bool IM2COL_B = IM2COL && A_MN;
  static_assert(!IM2COL_B || B_MN, "an im2col B tile is MN-major (channels contiguous)");

  // Dynamic shared memory a launch with the given rings needs (1024: manual alignment of the tiles).
  static constexpr int dyn_smem(int ring_raw, int ring_lo, int store_bufs) {
    return 1024 + ring_raw * HI_BYTES + (X3 ? ring_lo * HI_BYTES : 0) + 8 * store_bufs * STAGING_TILE;
  }
};

__device__ __forceinline__ float4 lds128(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(addr));
  return v;
}
// The split's accesses: a thread's 16 bytes as two 8-byte accesses 256 bytes apart, so that a warp still covers 512
// contiguous bytes (chunk = first byte of the warp's 512).  Measured against one 16-byte access per thread: 3-7 %
// on the shared-memory-bound narrower tiles, nothing on the 256x256 tile; which element a thread holds is
// irrelevant to the split, which is elementwise.
__device__ __forceinline__ float4 lds2x64(uint32_t chunk, int lane) {
  float4 v;
  asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(chunk + lane * 8));
  asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v.z), "=f"(v.w) : "r"(chunk + 256 + lane * 8));
  return v;
}
__device__ __forceinline__ void sts2x64(uint32_t chunk, int lane, float4 v) {
  asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(chunk + lane * 8), "f"(v.x), "f"(v.y) : "memory");
  asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(chunk + 256 + lane * 8), "f"(v.z), "f"(v.w) : "memory");
}
__device__ __forceinline__ void sts128(uint32_t addr, float4 v) {
  asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(v.x), "f"(v.y),
               "f"(v.z), "f"(v.w)
               : "memory");
}

// Work of one CTA for one output tile.
struct TileWork {
  int row0;    // first row of A / C handled by this CTA
  int col0;    // first column of C of the tile
  int bcol0;   // first column of B staged by this CTA
  int batch;   // batch coordinate of the tensor maps
  int kb0;     // first k-block
  int nkb;     // number of k-blocks (0 for a split-K slice that got none)
  float* out;  // output base for this batch / slice
  int zc;      // batch / slice coordinate in the output tensor map
  int tap;     // weight gradient: filter tap this tile belongs to
  int phase;   // strided data gradient in one launch: which phase the tile belongs to
  bool to_cbuf;  // this tile's output goes to the split-K partial buffers
};

// RINGS = 1: the rings are the configuration's balanced default (Cfg::STAGES raw slots, as many lo slots, each lo
// tile right behind its raw tile), known at compile time - slot addresses and wrap-arounds fold into constants,
// which the shared-memory-bound narrower tiles need (measured: 12-15 % on the 256x128 pair tile).  Otherwise the
// ring geometry comes from the launch parameters.
// A second compile-time geometry serves the shapes below the roofline's ridge (short reductions paced by loads and
// stores): a long raw ring against the HBM latency with a short lo ring.
//   RINGS 0 = launch parameters, 1 = balanced default, 2 = the configuration's below-ridge geometry (ALT_*)
template <class Cfg, int RINGS>
__device__ __forceinline__ void gemm_tf32_body(const GemmParams& p) {
  using namespace ptx;
  constexpr int BN = Cfg::BN, CTAS = Cfg::CTAS, CW = Cfg::CW;
  constexpr bool X3 = Cfg::X3;
  constexpr bool RELAY = X3 || CTAS == 2;  // MMA waits on the splitters' barrier

  extern __shared__ uint8_t smem_dyn[];
  __shared__ __align__(8) uint64_t bar_full_tma[8];
  __shared__ __align__(8) uint64_t bar_full_split[8];
  __shared__ __align__(8) uint64_t bar_full_split_peer[8];   // CTA pairs: the odd CTA's splitters arrive here
  __shared__ __align__(8) uint64_t bar_empty[8];
  __shared__ __align__(8) uint64_t bar_tmem_full[2];
  __shared__ __align__(8) uint64_t bar_tmem_empty[2];
  __shared__ __align__(8) uint64_t bar_red[2];       // softmax: the drain warps have published their row maxima / sums
  __shared__ float red[Cfg::SOFTMAX ? 2 : 1][2][2][Cfg::SOFTMAX ? Cfg::BM : 1];   // softmax: [parity][max, sum][column half][row]
  __shared__ uint32_t tmem_base_slot;
  __shared__ volatile int abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = (CTAS == 2) ? cluster_ctarank() : 0u;

  // ring geometry (launch parameters, uniform over the grid)
  const uint32_t R = RINGS == 1 ? static_cast<uint32_t>(Cfg::STAGES) : RINGS == 2 ? static_cast<uint32_t>(Cfg::ALT_RAW)
                                                                    : static_cast<uint32_t>(p.ring_raw);
  const uint32_t L = RINGS == 1 ? R : RINGS == 2 ? static_cast<uint32_t>(Cfg::ALT_LO)
                                                 : (X3 ? static_cast<uint32_t>(p.ring_lo) : R);
  const uint32_t raw_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  // With equally long rings a k-block's lo tiles sit right behind its raw tiles ([raw 0][lo 0][raw 1][lo 1]...);
  // with a shorter lo ring the two rings are separate ([raw 0..R-1][lo 0..L-1]).
  const bool paired = RINGS == 1 ? X3 : RINGS == 2 ? false : (X3 && L == R && p.ring_paired);
  const uint32_t raw_stride = paired ? 2u * Cfg::HI_BYTES : static_cast<uint32_t>(Cfg::HI_BYTES);
  const uint32_t lo_stride = raw_stride;
  const uint32_t lo_base = paired ? raw_base + Cfg::HI_BYTES : raw_base + R * Cfg::HI_BYTES;
  const uint32_t stg_base = raw_base + R * Cfg::HI_BYTES + (X3 ? L * Cfg::HI_BYTES : 0u);

  // ---- persistent tile loop: this CTA (pair) takes tiles first, first + step, ...
  // Tile ids run over (z, m-group, n, m-in-group); concurrently resident tiles are
  // consecutive ids, i.e. a GROUP x n patch of the output that shares operands in L2.
  constexpr bool DG = Cfg::IM2COL_A && Cfg::B_MN;     // the data-gradient instantiation
  const bool phased = DG && p.n_phases > 1;
  const int tiles_mn = p.tiles_m * p.tiles_n;
  const long long total_tiles = static_cast<long long>(tiles_mn) * p.zcount * (phased ? p.n_phases : 1);
  const long long tile_first = (CTAS == 2) ? (blockIdx.x >> 1) : blockIdx.x;
  const long long tile_step = (CTAS == 2) ? (gridDim.x >> 1) : gridDim.x;
  const int kc = p.kc;
  // The i-th tile of this CTA (pair), or -1 past the end.  A unit is one tile, except in the softmax mode,
  // where it is the tiles_n tiles that hold whole rows: those are taken one after the other.
  // In the phased mode a unit is tile j of every phase, taken one after the other.
  const int subs = Cfg::SOFTMAX ? p.unit_tiles : (phased ? p.n_phases : 1);
  const long long total_units = total_tiles / subs;
  const bool grouped = Cfg::SOFTMAX || phased;
  auto tile_at = [&](long long i) -> long long {
    const long long u = tile_first + (grouped ? i / subs : i) * tile_step;
    if (u >= total_units) return -1;
    return grouped ? u * subs + i % subs : u;
  };
  // What a tile's phase changes (phase 0 and every launch without phases: the GemmParams fields themselves).
  struct PhaseView {
    const CUtensorMap* tmA; const CUtensorMap* tmB;
    int M, OH, OW, FW, pw, ph, tap_base, tap_sy, tap_sx, os_uv, os_v;
  };
  auto phase_view = [&](int ph) -> PhaseView {
    PhaseView v;
    if (DG && ph > 0) {
      const GemmPhase& x = p.phx[ph - 1];
      v.tmA = &x.tmA; v.tmB = &x.tmB; v.M = x.M; v.OH = x.OH; v.OW = x.OW; v.FW = x.FW; v.pw = x.pw; v.ph = x.ph;
      v.tap_base = x.tap_base; v.tap_sy = x.tap_sy; v.tap_sx = x.tap_sx; v.os_uv = x.os_uv; v.os_v = x.os_v;
    } else {
      v.tmA = &p.tmA; v.tmB = &p.tmB; v.M = p.M; v.OH = p.conv_OH; v.OW = p.conv_OW; v.FW = p.conv_FW;
      v.pw = p.conv_pw; v.ph = p.conv_ph; v.tap_base = p.tap_base; v.tap_sy = p.tap_sy; v.tap_sx = p.tap_sx;
      v.os_uv = p.os_uv; v.os_v = p.os_v;
    }
    return v;
  };

  auto decode = [&](long long t) -> TileWork {
    constexpr int GROUP = 8;
    int phase = 0;
    if (phased) {   // t = (tile inside the phase) * n_phases + phase
      phase = static_cast<int>(t % p.n_phases);
      t /= p.n_phases;
    }
    const int z = static_cast<int>(t / tiles_mn);
    const int r = static_cast<int>(t - static_cast<long long>(z) * tiles_mn);
    const int per_group = GROUP * p.tiles_n;
    const int g_first = (r / per_group) * GROUP;
    const int g_size = min(p.tiles_m - g_first, GROUP);
    const int tm = Cfg::SOFTMAX ? r / p.tiles_n : g_first + (r % per_group) % g_size;
    const int tn = Cfg::SOFTMAX ? r % p.tiles_n : (r % per_group) / g_size;
    TileWork w;
    w.row0 = (tm * CTAS + static_cast<int>(rank)) * Cfg::BM;
    w.col0 = tn * BN;
    w.bcol0 = w.col0 + static_cast<int>(rank) * Cfg::BN_CTA;
    w.tap = 0;
    w.phase = phase;
    if (phased) {
      // phases differ in size: a tile past the end of its phase has no work (the test is on the pair's first
      // row, so both CTAs of a pair agree) and stores nothing (every row is clipped)
      const int m_ph = phase == 0 ? p.M : p.phx[phase - 1].M;
      w.kb0 = 0;
      w.nkb = (tm * CTAS * Cfg::BM < m_ph) ? (phase == 0 ? p.nkb_total : p.phx[phase - 1].nkb) : 0;
      w.batch = 0;
      w.out = phase == 0 ? p.C : p.phx[phase - 1].C;
      w.to_cbuf = false;
      w.zc = 0;
      return w;
    }
    if (p.ztaps > 0) {
      // weight gradient: z = slice * taps + tap; a tap owns p.N (= IC) columns of each output row
      const int slice = z / p.ztaps;
      w.tap = z - slice * p.ztaps;
      w.kb0 = static_cast<int>((static_cast<long long>(slice) * p.nkb_total) / p.gz);
      w.nkb = static_cast<int>((static_cast<long long>(slice + 1) * p.nkb_total) / p.gz) - w.kb0;
      w.batch = 0;
      w.out = ((slice == 0) ? p.C : p.Cbuf + static_cast<long long>(slice - 1) * p.c_stride) +
              static_cast<long long>(w.tap) * p.N;
      w.to_cbuf = slice > 0;
      w.zc = slice > 0 ? slice - 1 : 0;
    } else if (p.gz > 1) {
      w.kb0 = static_cast<int>((static_cast<long long>(z) * p.nkb_total) / p.gz);
      w.nkb = static_cast<int>((static_cast<long long>(z + 1) * p.nkb_total) / p.gz) - w.kb0;
      w.batch = 0;
      w.out = (z == 0) ? p.C : p.Cbuf + static_cast<long long>(z - 1) * p.c_stride;
      w.to_cbuf = z > 0;
      w.zc = z > 0 ? z - 1 : 0;
    } else {
      w.kb0 = 0;
      w.nkb = p.nkb_total;
      w.batch = z;
      w.out = p.C + static_cast<long long>(z) * p.c_stride;
      w.to_cbuf = false;
      w.zc = z;
    }
    return w;
  };

  auto give_up = [&](int role, int a, int b) {
    abort_flag = 1;
    atomicCAS(p.status, 0, (role << 24) | ((a & 0xFF) << 16) | (b & 0xFFFF));
  };

  // ---- one-time setup
  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < 8; ++s) {
      mbar_init(smem_u32(&bar_full_tma[s]), 1);
      mbar_init(smem_u32(&bar_full_split[s]), Cfg::SPLIT_WARPS);
      mbar_init(smem_u32(&bar_full_split_peer[s]), Cfg::SPLIT_WARPS);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&bar_tmem_full[b]), 1);
      mbar_init(smem_u32(&bar_tmem_empty[b]), Cfg::DRAIN_WARPS * CTAS);
      mbar_init(smem_u32(&bar_red[b]), Cfg::DRAIN_WARPS);
    }
    fence_mbar_init();
    tma_prefetch_desc(&p.tmA);
    tma_prefetch_desc(&p.tmB);
  }
  if (warp == 2) {
    tmem_alloc<CTAS>(smem_u32(&tmem_base_slot), Cfg::TMEM_COLS);
    tmem_relinquish<CTAS>();
  }
  tc_fence_before();
  __syncthreads();
  if (CTAS == 2) cluster_sync();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  // A launch that declared itself independent of this one (GemmParams::overlap_prev) may be scheduled from here on;
  // its CTAs then take over SMs as this grid's CTAs retire, instead of waiting for the whole grid.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // CTA 0 times itself in SM cycles and in nanoseconds: summed over launches, cycles / ns is the clock the
  // kernel really ran at (the management library's reading is a coarse sample and can miss short runs).
  long long clk_t0 = 0;
  unsigned long long clk_g0 = 0;
  if (p.clock_acc != nullptr && blockIdx.x == 0 && threadIdx.x == 0) {
    clk_t0 = clock64();
    clk_g0 = globaltimer_ns();
  }

  // Barrier addresses on the CTA that issues the MMAs (rank 0).
  auto leader_addr = [&](const uint64_t* bar) -> uint32_t {
    return (CTAS == 2) ? mapa(smem_u32(bar), 0u) : smem_u32(bar);
  };
  auto arrive_remote = [&](uint32_t bar) {
    if (p.arrive_release) mbar_arrive_cluster_release(bar);
    else mbar_arrive_cluster(bar);
  };

  // Warps 0..7 (two warpgroups) run the data-movement roles on a small register
  // budget; warps 8..15 hold the FP32 accumulators.  With 256-column tiles the
  // accumulators alone need 128 registers per thread, so registers are moved
  // from the first two warpgroups to the last two.
  if (warp < Cfg::DRAIN_WARP0) {
  if (Cfg::REALLOC) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(Cfg::REGS_MOVERS));
  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    // The whole warp walks the loop so that addresses, coordinates and descriptors are
    // computed once per warp in the uniform datapath (TMA and MMA instructions take their
    // operands from uniform registers); only the instructions themselves are single-lane.
    {
      const bool leader = lane == 0;
      uint32_t it = 0;  // k-blocks issued so far, over all tiles
      uint32_t s = 0, ph = 0;  // raw slot = it % R and its phase parity, carried as counters
      bool alive = true;
      // Tiles are walked in groups of 8 row-tiles across all column-tiles, so an A panel is
      // re-used by every column-tile of the sweep while B streams through once per group:
      // keep A in L2, let B go first (without this the two panels, together larger than
      // L2, evict each other in exactly the order they are needed again).
      const uint64_t pol_a = p.l2_hints ? l2_policy_evict_last() : 0ull;
      const uint64_t pol_b = p.l2_hints == 1 ? l2_policy_evict_first() : 0ull;
      for (long long i_tile = 0, t; alive && (t = tile_at(i_tile)) >= 0; ++i_tile) {
        const TileWork w = decode(t);
        const PhaseView pv = phase_view(w.phase);
        for (int i = 0; i < w.nkb; ++i, ++it, s = (s + 1 == R) ? 0u : s + 1, ph ^= (s == 0)) {
          if (!mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1u, &abort_flag)) {
            if (leader) give_up(ROLE_TMA, s, i);
            alive = false;
            break;
          }
          const uint32_t full = smem_u32(&bar_full_tma[s]);
          int k0 = (w.kb0 + i) * Cfg::BK;
          const uint32_t a_dst = raw_base + s * raw_stride;
          const uint32_t b_dst = a_dst + Cfg::A_BYTES;
          // im2col coordinates: k-block -> (filter tap, block of 32 channels inside the tap);
          // row0 addresses output pixel (n, oh, ow), and the run of 128 pixels wraps over
          // rows and images inside the tensor map's traversal box.
          int ic0 = 0, fh = 0, fw = 0, n = 0, oh = 0, ow = 0;
          if (Cfg::IM2COL_A) {
            const int tap = (w.kb0 + i) / p.conv_icb;
            ic0 = ((w.kb0 + i) - tap * p.conv_icb) * Cfg::BK;
            fh = tap / pv.FW;
            fw = tap - fh * pv.FW;
            k0 = tap * p.conv_IC + ic0;  // position in the filter's (fh, fw, ic) axis
            const int ohw = pv.OH * pv.OW;
            n = w.row0 / ohw;
            const int r = w.row0 - n * ohw;
            oh = r / pv.OW;
            ow = r - oh * pv.OW;
          }
          if (Cfg::IM2COL_B) {
            // the k-block is a run of 32 output pixels starting at pixel k0 = (n, oh, ow); runs wrap over
            // rows and images inside the tensor map's traversal box and read zeros past the last image
            fh = w.tap / p.conv_FW;
            fw = w.tap - fh * p.conv_FW;
            const int ohw = p.conv_OH * p.conv_OW;
            n = k0 / ohw;
            const int r = k0 - n * ohw;
            oh = r / p.conv_OW;
            ow = r - oh * p.conv_OW;
          }
          uint32_t tx_bytes = Cfg::HI_BYTES;
          if (Cfg::IM2COL && p.gather) {
            // Slow path: the whole warp builds the im2col tile with 16-byte loads, zero outside the image, in the
            // layout the tensor map would have produced, then publishes it to the async proxy; only the other
            // operand still arrives by TMA.
            const int ohw = p.conv_OH * p.conv_OW;
            const int chunk = lane & 7, sub = lane >> 3;
            if (Cfg::IM2COL_A) {
              // K-major A tile: row r = output pixel row0 + r, 32 channels = 8 chunks at r*128 + ((c ^ (r & 7)) * 16)
#pragma unroll 1
              for (int rr = 0; rr < Cfg::BM / 4; ++rr) {
                const int r = rr * 4 + sub;
                const int pix = w.row0 + r;
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (pix < p.M && ic0 + chunk * 4 < p.conv_IC) {
                  const int pn = pix / ohw, pr = pix - pn * ohw;
                  const int poh = pr / p.conv_OW, pow_ = pr - poh * p.conv_OW;
                  const int ih = poh * p.conv_sh - p.conv_ph + fh, iw = pow_ * p.conv_sw - p.conv_pw + fw;
                  if (ih >= 0 && ih < p.g_H && iw >= 0 && iw < p.g_W)
                    v = __ldg(reinterpret_cast<const float4*>(
                        p.g_img + ((static_cast<long long>(pn) * p.g_H + ih) * p.g_W + iw) * p.conv_IC + ic0 + chunk * 4));
                }
                sts128(a_dst + r * 128 + ((chunk ^ (r & 7)) * 16), v);
              }
              tx_bytes = Cfg::B_BYTES;
            } else {
              // MN-major B slabs of [32 pixels][32 channels], 32-byte-unit swizzle: 16-byte chunk c of pixel row k at
              // k*128 + (((c >> 1) ^ (k & 3)) << 5) + (c & 1) * 16
              const long long gk = static_cast<long long>(p.nkb_total) * Cfg::BK;   // >= the true pixel count; rows beyond the images read zeros below
#pragma unroll 1
              for (int j = 0; j < Cfg::BN_CTA / 32; ++j) {
                const int ch0 = w.bcol0 + 32 * j + chunk * 4;
#pragma unroll 1
                for (int kk2 = 0; kk2 < 8; ++kk2) {
                  const int k = kk2 * 4 + sub;
                  const long long pix = static_cast<long long>(k0) + k;
                  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                  if (pix < gk && ch0 < p.N) {
                    const int pn = static_cast<int>(pix / ohw), pr = static_cast<int>(pix - static_cast<long long>(pn) * ohw);
                    const int poh = pr / p.conv_OW, pow_ = pr - poh * p.conv_OW;
                    const int ih = poh * p.conv_sh - p.conv_ph + fh, iw = pow_ * p.conv_sw - p.conv_pw + fw;
                    if (pn < p.g_N && ih >= 0 && ih < p.g_H && iw >= 0 && iw < p.g_W)
                      v = __ldg(reinterpret_cast<const float4*>(
                          p.g_img + ((static_cast<long long>(pn) * p.g_H + ih) * p.g_W + iw) * p.conv_IC + ch0));
                  }
                  sts128(b_dst + j * 4096 + k * 128 + ((((chunk >> 1) ^ (k & 3)) << 5) | ((chunk & 1) << 4)), v);
                }
              }
              tx_bytes = Cfg::A_BYTES;
            }
            fence_proxy_async_smem();
            __syncwarp();
          }
          // one single-thread region for all copies of the k-block
          if (elect_one()) {
            mbar_arrive_expect_tx(full, tx_bytes);
            if (Cfg::IM2COL_A && p.gather) {
              // the A tile is in place already
            } else if (Cfg::IM2COL_A) {
              tma_load_im2col_4d(a_dst, pv.tmA, full, ic0, ow * p.conv_sw - pv.pw,
                                 oh * p.conv_sh - pv.ph, n, static_cast<uint16_t>(fw),
                                 static_cast<uint16_t>(fh), pol_a);
            } else if (Cfg::A_MN) {
#pragma unroll
              for (int j = 0; j < Cfg::BM / 32; ++j)
                tma_load_3d(a_dst + j * 4096, &p.tmA, full, w.row0 + 32 * j, k0, w.batch, pol_a);
            } else {
              tma_load_3d(a_dst, &p.tmA, full, k0, w.row0, w.batch, pol_a);
            }
            if (Cfg::IM2COL_B && p.gather) {
              // the B slabs are in place already
            } else if (Cfg::IM2COL_B) {
              // 32 pixels x 32 channels of tap (fh, fw) per slab; slabs that would start past the last
              // channel re-read the last block instead (their output columns are never stored)
              const int cmax = ((p.N - 1) >> 5) << 5;
#pragma unroll
              for (int j = 0; j < Cfg::BN_CTA / 32; ++j)
                tma_load_im2col_4d(b_dst + j * 4096, &p.tmB, full, min(w.bcol0 + 32 * j, cmax),
                                   ow * p.conv_sw - p.conv_pw, oh * p.conv_sh - p.conv_ph, n,
                                   static_cast<uint16_t>(fw), static_cast<uint16_t>(fh), pol_b);
            } else if (Cfg::B_MN && Cfg::IM2COL) {
              // data gradient: this k-block is 32 input channels of tap (fh, fw) of the im2col walk;
              // the filter matrix that multiplies it sits at a tap index given by the host
              const int btap = pv.tap_base + pv.tap_sy * fh + pv.tap_sx * fw;
#pragma unroll
              for (int j = 0; j < Cfg::BN_CTA / 32; ++j)
                if (p.bmap_order == 0) tma_load_3d(b_dst + j * 4096, pv.tmB, full, w.bcol0 + 32 * j, btap, ic0, pol_b);
                else                   tma_load_3d(b_dst + j * 4096, pv.tmB, full, w.bcol0 + 32 * j, ic0, btap, pol_b);
            } else if (Cfg::B_MN) {
#pragma unroll
              for (int j = 0; j < Cfg::BN_CTA / 32; ++j)
                tma_load_3d(b_dst + j * 4096, &p.tmB, full, w.bcol0 + 32 * j, k0, w.batch, pol_b);
            } else {
              tma_load_3d(b_dst, &p.tmB, full, k0, w.bcol0, w.batch, pol_b);
            }
          }
          __syncwarp();
        }
      }
      if (leader && abort_flag) {
        // Let copies already in flight land before shared memory is released:
        // wait (bounded) for the barrier of every slot still outstanding.
        const uint32_t first = it > R ? it - R : 0u;
        for (uint32_t i = first; i < it; ++i) {
          const uint32_t slot = i % R;
          const uint32_t par = (i / R) & 1u;
          const long long t0 = clock64();
          while (!mbar_try_wait(smem_u32(&bar_full_tma[slot]), par) && clock64() - t0 < 20000000LL) {
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    // Measured cost to this thread, per k-block of 12 MMAs (1536 cycles of execution on the
    // 256-column pair tile): about 390 cycles to issue them from one elect.sync region, about
    // 100 for the commits (one paired commit instead of two for a CTA pair); the rest of the
    // time it waits for operands.
    if (rank == 0) {
      const bool leader = lane == 0;   // the one thread that issues (and whose commits track) the MMAs
      constexpr uint32_t idesc = make_idesc_tf32(Cfg::BM * CTAS, BN, Cfg::A_MN, Cfg::B_MN);
      constexpr uint32_t A_LBO = Cfg::A_MN ? 4096u : 16u;
      constexpr uint32_t B_LBO = Cfg::B_MN ? 4096u : 16u;
      constexpr uint32_t A_SBO = Cfg::A_MN ? 512u : 1024u;
      constexpr uint32_t B_SBO = Cfg::B_MN ? 512u : 1024u;
      constexpr uint32_t A_LT = Cfg::A_MN ? SMEM_LAYOUT_SW128_32B : SMEM_LAYOUT_SW128;
      constexpr uint32_t B_LT = Cfg::B_MN ? SMEM_LAYOUT_SW128_32B : SMEM_LAYOUT_SW128;
      constexpr uint32_t A_KSTEP = Cfg::A_MN ? 1024u : 32u;  // bytes per 8 elements of K
      constexpr uint32_t B_KSTEP = Cfg::B_MN ? 1024u : 32u;
      // This loop's scalar bookkeeping is on the critical path (one warp, dependent
      // instructions, ~8 cycles each): ring positions are carried as counters instead of
      // being re-derived with divisions every k-block.
      uint32_t it = 0;    // k-blocks consumed so far, over all tiles
      uint32_t ch = 0;    // chunks started so far: TMEM buffer = ch & 1
      uint32_t s = 0, ph = 0;   // raw slot and its phase parity
      uint32_t l = 0;     // lo slot = it % L
      uint32_t kk = 0;    // k-blocks already in the current chunk
      bool alive = true;
      for (long long i_tile = 0, t; alive && (t = tile_at(i_tile)) >= 0; ++i_tile) {
        const TileWork w = decode(t);
        kk = 0;
        for (int i = 0; i < w.nkb; ++i, ++it) {
          const bool chunk_start = kk == 0;
          ++kk;
          const bool chunk_end = kk == static_cast<uint32_t>(kc) || i + 1 == w.nkb;
          if (chunk_end) kk = 0;
          const uint32_t ready = (RELAY ? smem_u32(&bar_full_split[0]) : smem_u32(&bar_full_tma[0])) + s * 8u;
          if (!mbar_wait(ready, ph, &abort_flag)) {
            if (leader) give_up(ROLE_MMA, s, i);
            alive = false;
            break;
          }
          if (CTAS == 2 && !mbar_wait<true>(smem_u32(&bar_full_split_peer[0]) + s * 8u, ph, &abort_flag)) {
            if (leader) give_up(ROLE_MMA, 50 + s, i);
            alive = false;
            break;
          }
          const uint32_t buf = ch & 1u;
          if (chunk_start) {
            // the n-th use of a buffer waits for the (n-1)-th drain; the first use passes
            if (!mbar_wait<CTAS == 2>(smem_u32(&bar_tmem_empty[0]) + buf * 8u, ((ch >> 1) & 1u) ^ 1u, &abort_flag)) {
              if (leader) give_up(ROLE_MMA_TMEM, buf, i);
              alive = false;
              break;
            }
          }
          tc_fence_after();
          const uint32_t a_hi = raw_base + s * raw_stride;
          const uint32_t b_hi = a_hi + Cfg::A_BYTES;
          const uint32_t a_lo = lo_base + l * lo_stride;
          const uint32_t b_lo = a_lo + Cfg::A_BYTES;
          const uint32_t d = tmem_base + buf * BN;
          // The tensor core truncates (rounds toward zero) its FP32 accumulator after every
          // instruction, an error of up to one ulp of the *accumulator*.  Issuing all the
          // small lo*hi / hi*lo products of the k-block first, while the accumulator of a
          // fresh chunk is still small, keeps those truncations negligible; only the four
          // hi*hi instructions then round at full magnitude.
          //
          // All instructions of the k-block sit in ONE elect.sync region: the compiler then
          // knows a single thread runs it and feeds the MMAs from uniform registers - measured
          // 24 cycles per issued MMA against 50-60 with a (lane == 0) test on each.  Successive
          // descriptors differ only in the start-address field (low word, 16-byte units).
          if (elect_one()) {
            constexpr uint64_t A_STEP = A_KSTEP >> 4, B_STEP = B_KSTEP >> 4;
            const uint64_t db_hi0 = make_smem_desc(b_hi, B_LBO, B_SBO, B_LT);
            const uint32_t first = chunk_start ? 0u : 1u;
            const uint64_t da_hi0 = make_smem_desc(a_hi, A_LBO, A_SBO, A_LT);
            if (X3) {
              const uint64_t da_lo0 = make_smem_desc(a_lo, A_LBO, A_SBO, A_LT);
              const uint64_t db_lo0 = make_smem_desc(b_lo, B_LBO, B_SBO, B_LT);
#pragma unroll
              for (int j = 0; j < Cfg::BK / 8; ++j) {
                umma_tf32<CTAS>(d, da_lo0 + j * A_STEP, db_hi0 + j * B_STEP, idesc, j == 0 ? first : 1u);
                umma_tf32<CTAS>(d, da_hi0 + j * A_STEP, db_lo0 + j * B_STEP, idesc, 1u);
              }
            }
#pragma unroll
            for (int j = 0; j < Cfg::BK / 8; ++j)
              umma_tf32<CTAS>(d, da_hi0 + j * A_STEP, db_hi0 + j * B_STEP, idesc, (!X3 && j == 0) ? first : 1u);
            // The raw slot (and with it the lo slot) may be refilled once these MMAs have read it.
            if (CTAS == 2) umma_commit_pair(smem_u32(&bar_empty[0]) + s * 8u);
            else umma_commit<CTAS>(smem_u32(&bar_empty[0]) + s * 8u);
            if (chunk_end) {
              if (CTAS == 2) umma_commit_pair(smem_u32(&bar_tmem_full[0]) + buf * 8u);
              else umma_commit<CTAS>(smem_u32(&bar_tmem_full[0]) + buf * 8u);
            }
          }
          __syncwarp();
          if (++s == R) { s = 0; ph ^= 1u; }
          if (++l == L) l = 0;
          if (chunk_end) ++ch;
        }
      }
    }
  } else {
    // ------------------------------------------------------------ splitters
    if (RELAY) {
      // which 16-byte vectors of the slot this thread handles
      const int st = (warp - Cfg::SPLIT_WARP0) * 32 + lane;
      constexpr int NST = Cfg::SPLIT_WARPS * 32;
      constexpr int NVEC = Cfg::HI_BYTES / 16;
      static_assert(NVEC % 32 == 0, "a warp's 32 vectors of the split are 512 contiguous bytes inside the slot");
      uint32_t it = 0;
      uint32_t s = 0, ph = 0;     // raw slot = it % R and its phase parity, carried as counters
      uint32_t l = 0;             // lo slot = it % L
      uint32_t sp = 0, php = 0;   // raw slot and phase parity of k-block it - L, the previous user of lo slot l
      bool alive = true;
      for (long long i_tile = 0, t; alive && (t = tile_at(i_tile)) >= 0; ++i_tile) {
        const TileWork w = decode(t);
        for (int i = 0; i < w.nkb; ++i, ++it, s = (s + 1 == R) ? 0u : s + 1, ph ^= (s == 0)) {
          if (!mbar_wait(smem_u32(&bar_full_tma[s]), ph, &abort_flag)) {
            if (lane == 0) give_up(ROLE_SPLIT, s, i);
            alive = false;
            break;
          }
          if (X3 && L != R && it >= L) {
            // The lo slot is free once the MMAs of k-block it - L have completed, which is what frees
            // that k-block's raw slot: wait on its "empty" barrier.  (With L == R that is this raw slot's
            // own previous use, which the producer has waited for already.)  No later phase of that
            // barrier can complete before this k-block has been split, so the parity is unambiguous.
            if (!mbar_wait(smem_u32(&bar_empty[sp]), php, &abort_flag)) {
              if (lane == 0) give_up(ROLE_SPLIT, 100 + sp, i);
              alive = false;
              break;
            }
          }
          const uint32_t hi_base = raw_base + s * raw_stride;
          const uint32_t lo_slot = lo_base + l * lo_stride;
          if (X3) {
            // lo = tf32(x - trunc(x)); x itself stays where TMA put it (the tensor core drops the low
            // 13 mantissa bits of an FP32 operand by itself, so the raw tile already is the hi operand).
            // The loads of the next group of vectors are in flight while this group is converted and stored.
            constexpr int PER = (NVEC + NST - 1) / NST;
            constexpr int G = 3;
            float4 x[2][G];
#pragma unroll
            for (int u = 0; u < G; ++u) {
              const int v = st + u * NST;
              if (u < PER && v < NVEC) x[0][u] = lds2x64(hi_base + (v - lane) * 16, lane);
            }
#pragma unroll
            for (int b = 0; b < PER; b += G) {
              const int cur = (b / G) & 1;
#pragma unroll
              for (int u = 0; u < G; ++u) {
                const int v = st + (b + G + u) * NST;
                if (b + G + u < PER && v < NVEC) x[cur ^ 1][u] = lds2x64(hi_base + (v - lane) * 16, lane);
              }
#pragma unroll
              for (int u = 0; u < G; ++u) {
                const int v = st + (b + u) * NST;
                if (b + u < PER && v < NVEC) {
                  const float4 xv = x[cur][u];
                  float4 lv;
                  lv.x = rn_tf32(xv.x - trunc_tf32(xv.x)); lv.y = rn_tf32(xv.y - trunc_tf32(xv.y));
                  lv.z = rn_tf32(xv.z - trunc_tf32(xv.z)); lv.w = rn_tf32(xv.w - trunc_tf32(xv.w));
                  sts2x64(lo_slot + (v - lane) * 16, lane, lv);
                }
              }
            }
            // the tensor core reads these tiles through the async proxy: without this fence a
            // store can still be in flight when the MMA that the arrive below releases reads it
            fence_proxy_async_smem();
          }
          __syncwarp();
          if (lane == 0) {
            if (CTAS == 2 && rank != 0)
              arrive_remote(leader_addr(&bar_full_split_peer[s]));
            else
              mbar_arrive(smem_u32(&bar_full_split[s]));
          }
          if (++l == L) l = 0;
          // (sp, php) follow k-block (it + 1) - L: it sits at raw slot 0, phase 0 when it + 1 == L
          if (it + 1 > L && ++sp == R) { sp = 0; php ^= 1u; }
        }
      }
    }
  }
  } else {
    // ------------------------------------------------------------ drainers
    if (Cfg::REALLOC) asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(Cfg::REGS_DRAINERS));
    const int q = warp & 3;                              // TMEM lane quarter this warp may read
    const int h = (warp - Cfg::DRAIN_WARP0) >> 2;        // which half of the columns
    uint32_t ch = 0;                                     // chunks drained so far, over all tiles
    uint32_t pc = 0;                                     // 32x32 pieces this warp has sent through TMA stores
    const uint32_t sbufs = RINGS == 1 ? 1u : RINGS == 2 ? static_cast<uint32_t>(Cfg::ALT_BUFS) : static_cast<uint32_t>(p.store_bufs);
    const uint32_t stg0 = stg_base + (warp - Cfg::DRAIN_WARP0) * sbufs * Cfg::STAGING_TILE;
    bool alive = true;
    // Lazy copies: the block this warp stored last (32 rows x CW columns of C) is carried to the further copies
    // in FW_STEPS steps of one 16-byte vector per lane.
    constexpr int FW_VPR = CW / 4;                 // vectors per row segment
    constexpr int FW_RPS = 32 / FW_VPR > 0 ? 32 / FW_VPR : 1;   // rows per step
    constexpr int FW_STEPS = 32 / FW_RPS;
    static_assert(CW <= 128 && (CW % 4) == 0, "a row segment of a drain warp is at most 32 vectors");
    int fw_step = FW_STEPS, fw_r0 = 0, fw_c0 = 0;   // nothing pending
    bool fw_fresh = false;                          // the block's own stores to C have not been waited for yet
    auto forward_until = [&](int target, bool batched) {
      if (fw_step >= target) return;
      if (fw_fresh) {   // the TMA stores of the block (issued by lane 0) have completed before anyone reads C
        if (lane == 0) { tma_store_wait_all(); fence_proxy_async_all(); }
        __syncwarp();
        fw_fresh = false;
      }
      const int cc = fw_c0 + (lane % FW_VPR) * 4;
      const bool col_ok = cc < p.N;               // p.N is a multiple of 4 on this path
      auto off_of = [&](int step) -> long long {
        const int r = fw_r0 + step * FW_RPS + lane / FW_VPR;
        return (col_ok && r < p.M) ? static_cast<long long>(r) * p.ldc + cc : -1;
      };
      // four loads in flight where the registers are free for them (between tiles and at the end)
      if (batched) for (; fw_step + 4 <= target; fw_step += 4) {
        long long o[4];
        float4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          o[u] = off_of(fw_step + u);
          if (o[u] >= 0) v[u] = ldg128_l2(p.C + o[u]);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (o[u] >= 0)
            for (int i = 0; i < p.n_rep; ++i) *reinterpret_cast<float4*>(p.rep_ptr[i] + o[u]) = v[u];
      }
      for (; fw_step < target; ++fw_step) {
        const long long o = off_of(fw_step);
        if (o >= 0) {
          const float4 v = ldg128_l2(p.C + o);
          for (int i = 0; i < p.n_rep; ++i) *reinterpret_cast<float4*>(p.rep_ptr[i] + o) = v;
        }
      }
    };
    for (long long i_tile = 0, t; alive && (t = tile_at(Cfg::SOFTMAX ? i_tile * subs : i_tile)) >= 0; ++i_tile) {
      const TileWork w = decode(t);
      if constexpr (Cfg::SOFTMAX) {
        // ---------------------------------------------------------------- row softmax of the finished products
        // The unit's tiles (one chunk each: the host makes kc cover the whole reduction) sit side by side in the
        // TMEM buffers: this thread owns row q*32 + lane and, in each buffer, the CW columns of its half h.
        //   pass 1  x' = fma(x, alpha, 0), row maximum     (the two halves exchange through shared memory)
        //   pass 2  e = exp(x' - max) written back to TMEM, row sum (exchanged likewise)
        //   pass 3  e * (1 / sum) -> staging tile -> TMA store; a buffer is handed back after its last load
        // Same values as the engine's sequence scale -> row_max -> row_softmax -> div2D_field up to the order of
        // the row sum and the reciprocal (one rounding each).
        const uint32_t upar = static_cast<uint32_t>(i_tile) & 1u;
        bool ok = true;
        for (int b = 0; ok && b < subs; ++b) {
          const uint32_t cb = ch + b;
          if (!mbar_wait(smem_u32(&bar_tmem_full[cb & 1u]), (cb >> 1) & 1u, &abort_flag)) {
            if (lane == 0) give_up(ROLE_DRAIN, static_cast<int>(cb & 1u), b);
            ok = false;
          }
        }
        if (!ok) { alive = false; break; }
        tc_fence_after();
        const int myrow = q * 32 + lane;
        const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
        static_assert(CW == 128, "the passes below read a warp's 128 columns as two loads of 64");
        float va[64], vb[64];
        // fl(x * alpha) is monotonic in x, so the maximum of x' is the scaled maximum (minimum for alpha < 0) of x
        const bool up = p.alpha >= 0.0f;
        // ---- pass 1
        float m = up ? -INFINITY : INFINITY;
        for (int b = 0; b < subs; ++b) {
          const uint32_t t0 = lane_addr + static_cast<uint32_t>(((ch + b) & 1u) * BN + h * CW);
          const int c_first = b * BN + h * CW;
          if (c_first >= p.sm_width) break;   // warp-uniform: nothing but pitch padding from here on
          tmem_ld_32x64(t0, va);
          tmem_ld_32x64(t0 + 64, vb);
          tmem_wait_ld();
          if (c_first + CW <= p.sm_width) {
#pragma unroll
            for (int j = 0; j < 64; ++j) m = up ? fmaxf(m, fmaxf(va[j], vb[j])) : fminf(m, fminf(va[j], vb[j]));
          } else {
#pragma unroll
            for (int j = 0; j < 64; ++j) {
              if (c_first + j < p.sm_width) m = up ? fmaxf(m, va[j]) : fminf(m, va[j]);
              if (c_first + 64 + j < p.sm_width) m = up ? fmaxf(m, vb[j]) : fminf(m, vb[j]);
            }
          }
        }
        red[upar][0][h][myrow] = fmaf(m, p.alpha, 0.0f);   // +-inf stays: a half without valid columns never wins
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_red[0]));
        if (!mbar_wait(smem_u32(&bar_red[0]), upar, &abort_flag)) {
          if (lane == 0) give_up(ROLE_DRAIN, 20, 0);
          alive = false;
          break;
        }
        m = fmaxf(red[upar][0][0][myrow], red[upar][0][1][myrow]);
        // ---- pass 2
        float sum = 0.0f;
        for (int b = 0; b < subs; ++b) {
          const uint32_t t0 = lane_addr + static_cast<uint32_t>(((ch + b) & 1u) * BN + h * CW);
          const int c_first = b * BN + h * CW;
          tmem_ld_32x64(t0, va);
          tmem_ld_32x64(t0 + 64, vb);
          tmem_wait_ld();
          const bool whole = c_first + CW <= p.sm_width;   // warp-uniform
          float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;   // partial sums: shorter chains, smaller rounding error
#pragma unroll
          for (int j = 0; j < 64; j += 2) {
            float e0 = expf(fmaf(va[j], p.alpha, 0.0f) - m), e1 = expf(fmaf(va[j + 1], p.alpha, 0.0f) - m);
            float e2 = expf(fmaf(vb[j], p.alpha, 0.0f) - m), e3 = expf(fmaf(vb[j + 1], p.alpha, 0.0f) - m);
            if (!whole) {
              if (c_first + j >= p.sm_width) e0 = 0.0f;
              if (c_first + j + 1 >= p.sm_width) e1 = 0.0f;
              if (c_first + 64 + j >= p.sm_width) e2 = 0.0f;
              if (c_first + 64 + j + 1 >= p.sm_width) e3 = 0.0f;
            }
            va[j] = e0; va[j + 1] = e1; vb[j] = e2; vb[j + 1] = e3;
            s0 += e0; s1 += e1; s2 += e2; s3 += e3;
          }
          sum += (s0 + s1) + (s2 + s3);
          tmem_st_32x64(t0, va);
          tmem_st_32x64(t0 + 64, vb);
          tmem_wait_st();
        }
        red[upar][1][h][myrow] = sum;
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_red[1]));
        if (!mbar_wait(smem_u32(&bar_red[1]), upar, &abort_flag)) {
          if (lane == 0) give_up(ROLE_DRAIN, 21, 0);
          alive = false;
          break;
        }
        const float rinv = 1.0f / (red[upar][1][0][myrow] + red[upar][1][1][myrow]);
        // ---- pass 3
        for (int b = 0; b < subs; ++b) {
          const uint32_t t0 = lane_addr + static_cast<uint32_t>(((ch + b) & 1u) * BN + h * CW);
          const uint32_t buf = (ch + b) & 1u;
          tmem_ld_32x64(t0, va);
          tmem_ld_32x64(t0 + 64, vb);
          tmem_wait_ld();
          // this buffer's values have left TMEM: hand it back to the MMA issuer
          tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            if (rank != 0) arrive_remote(leader_addr(&bar_tmem_empty[buf]));
            else mbar_arrive(smem_u32(&bar_tmem_empty[buf]));
          }
#pragma unroll
          for (int g = 0; g < CW / 32; ++g) {
            const int c0 = b * BN + h * CW + g * 32;
            const int r0 = w.row0 + q * 32;
            if (c0 < p.N && r0 < p.M) {   // warp-uniform
              const uint32_t stg = stg0 + ((sbufs == 2u) ? (pc & 1u) : 0u) * Cfg::STAGING_TILE;
              if (lane == 0) {   // the store that last used this staging tile has read it
                if (sbufs == 2u) tma_store_wait_read_1(); else tma_store_wait_read();
              }
              __syncwarp();
#pragma unroll
              for (int cq = 0; cq < 8; ++cq) {
                const int j = (g & 1) * 32 + cq * 4;
                const float (&src)[64] = (g < 2) ? va : vb;
                sts128(stg + lane * 128 + ((cq ^ (lane & 7)) * 16),
                       make_float4(src[j] * rinv, src[j + 1] * rinv, src[j + 2] * rinv, src[j + 3] * rinv));
              }
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0) {
                tma_store_3d(&p.tmC, stg, c0, r0, w.zc);
                tma_store_commit();
              }
              ++pc;
            }
          }
        }
        ch += static_cast<uint32_t>(subs);
        continue;
      }
      float acc[CW];
#pragma unroll
      for (int j = 0; j < CW; ++j) acc[j] = 0.0f;
      const int nchunks = (w.nkb + kc - 1) / kc;
      // Long reductions leave the registers more than once: after every flush_chunks chunks the sums are
      // stored (first time) or added to the output (later), which bounds the length of any FP32 register
      // sum and with it the rounding error of non-negative data, whatever K is.  The additions to memory
      // are one per element and flush, in a fixed order, so results stay reproducible.
      const bool multi = nchunks > p.flush_chunks;
      // a fused bias / scale is applied to the complete sum, so with several flushes the last one must read
      // the output back: those tiles take the register path
      const bool use_tma = p.tma_store && !(multi && (p.bias != nullptr || p.scale_on));
      bool first = true;
      int since = 0;
      for (int c = 0;; ++c) {
        if (c < nchunks) {
          // the previous block's way to the copies is spread evenly over this tile's chunks
          if constexpr (Cfg::REP)
            if (fw_step < FW_STEPS) forward_until(((c + 1) * FW_STEPS + nchunks - 1) / nchunks, false);
          const int buf = ch & 1;
          const uint32_t par = (ch >> 1) & 1;
          if (!mbar_wait(smem_u32(&bar_tmem_full[buf]), par, &abort_flag)) {
            if (lane == 0) give_up(ROLE_DRAIN, buf, c);
            alive = false;
            break;
          }
          tc_fence_after();
          const uint32_t t0 = tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                              static_cast<uint32_t>(buf * BN + h * CW);
          // 16-column pieces, the load of piece g+1 in flight while piece g is added; the
          // buffer goes back to the MMA issuer as soon as the last piece has left TMEM.
          constexpr int PIECES = CW / 16;
          float va[16], vb[16];
          tmem_ld_32x16(t0, va);
#pragma unroll
          for (int g = 0; g < PIECES; ++g) {
            tmem_wait_ld();
            float (&cur)[16] = (g & 1) ? vb : va;
            float (&nxt)[16] = (g & 1) ? va : vb;
            if (g + 1 < PIECES) {
              tmem_ld_32x16(t0 + (g + 1) * 16, nxt);
            } else {
              tc_fence_before();
              __syncwarp();
              if (lane == 0) {
                if (CTAS == 2 && rank != 0)
                  arrive_remote(leader_addr(&bar_tmem_empty[buf]));
                else
                  mbar_arrive(smem_u32(&bar_tmem_empty[buf]));
              }
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) acc[g * 16 + j] += cur[j];
          }
          ++ch;
        }
        const bool last = c + 1 >= nchunks;
        if (!last && ++since < p.flush_chunks) continue;
        // ---- fused bias row (optional): what the engine's linear_dual2D_row(C, bias, 1, 1, 0) does right
        // after the product - one FP32 add per element, padding columns forced to zero.  Applied to
        // each 4-column vector of the complete sum on its way out, so that no more than a few bias values are live.
        auto with_bias = [&](int j, float4 v) -> float4 {
          if (!last) return v;
          if (p.scale_on) {   // what a separate y = alpha*x + 0 kernel would store: one fused multiply-add per element
            v.x = fmaf(v.x, p.alpha, 0.0f); v.y = fmaf(v.y, p.alpha, 0.0f);
            v.z = fmaf(v.z, p.alpha, 0.0f); v.w = fmaf(v.w, p.alpha, 0.0f);
          }
          if (p.bias == nullptr) return v;
          const int cc = w.col0 + h * CW + j;   // a multiple of 4, like p.N: all four columns exist or none
          if (cc >= p.N) return v;
          const float4 b = __ldg(reinterpret_cast<const float4*>(p.bias + cc));
          v.x = (cc + 0 < p.bias_width) ? v.x + b.x : 0.0f;
          v.y = (cc + 1 < p.bias_width) ? v.y + b.y : 0.0f;
          v.z = (cc + 2 < p.bias_width) ? v.z + b.z : 0.0f;
          v.w = (cc + 3 < p.bias_width) ? v.w + b.w : 0.0f;
          return v;
        };
        // The common case has neither: keep its loops free of the per-vector tests (measured: the tests cost more
        // than the stores they guard).
        const bool plain = !(last && (p.bias != nullptr || p.scale_on));
        // what is already in memory for this vector (later flushes of a tile)
        auto plus_old = [&](float4 v, const float* src) -> float4 {
          if (first) return v;
          const float4 o = *reinterpret_cast<const float4*>(src);
          v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
          return v;
        };
        // ---- store; the MMA warp is already filling the TMEM buffers with the next chunks meanwhile
        if (use_tma) {
          // Each drain warp owns a 32-row x CW-column block.  32x32 pieces go through a
          // swizzled 4 KB staging tile (row r, 16-byte chunk c at r*128 + ((c ^ (r & 7)) * 16):
          // conflict-free for the row-per-lane writes) and leave as one TMA store each, which
          // writes whole 128-byte row segments and clips rows >= M and columns >= N.  With two
          // staging tiles per warp a piece is staged while the previous one is still being read.
          // Later flushes of a tile leave as TMA add-reductions, after the earlier ones have completed.
          const CUtensorMap* cmap = w.to_cbuf ? &p.tmCbuf : &p.tmC;
          if (!first) {
            if (lane == 0) tma_store_wait_all();
            __syncwarp();
          }
#pragma unroll
          for (int g = 0; g < CW / 32; ++g) {
            const int c0 = w.col0 + h * CW + g * 32;
            const int r0 = w.row0 + q * 32;
            if (c0 < p.N && r0 < p.M) {   // warp-uniform
              const uint32_t stg = stg0 + ((sbufs == 2u) ? (pc & 1u) : 0u) * Cfg::STAGING_TILE;
              if (lane == 0) {   // the store that last used this staging tile has read it
                if (sbufs == 2u) tma_store_wait_read_1(); else tma_store_wait_read();
              }
              __syncwarp();
              if (plain) {
#pragma unroll
                for (int cq = 0; cq < 8; ++cq)
                  sts128(stg + lane * 128 + ((cq ^ (lane & 7)) * 16),
                         make_float4(acc[g * 32 + cq * 4], acc[g * 32 + cq * 4 + 1], acc[g * 32 + cq * 4 + 2],
                                     acc[g * 32 + cq * 4 + 3]));
              } else {
#pragma unroll
                for (int cq = 0; cq < 8; ++cq)
                  sts128(stg + lane * 128 + ((cq ^ (lane & 7)) * 16),
                         with_bias(g * 32 + cq * 4, make_float4(acc[g * 32 + cq * 4], acc[g * 32 + cq * 4 + 1],
                                                                acc[g * 32 + cq * 4 + 2], acc[g * 32 + cq * 4 + 3])));
              }
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0) {
                if (first) tma_store_3d(cmap, stg, c0, r0, w.zc);
                else tma_reduce_add_3d(cmap, stg, c0, r0, w.zc);
                if constexpr (Cfg::REP) if (!p.rep_lazy) {
                  for (int i = 0; i < p.n_rep; ++i) {   // the same piece to every further copy of the output
                    if (first) tma_store_3d(&p.tmRep[i], stg, c0, r0, w.zc);
                    else tma_reduce_add_3d(&p.tmRep[i], stg, c0, r0, w.zc);
                  }
                }
                tma_store_commit();
              }
              ++pc;
            }
          }
          if constexpr (Cfg::REP) if (last && p.rep_lazy) {   // this block becomes the pending one (the previous one has gone out by now)
            forward_until(FW_STEPS, true);
            fw_step = 0; fw_r0 = w.row0 + q * 32; fw_c0 = w.col0 + h * CW; fw_fresh = true;
          }
        } else if (p.os_on) {
          // Rows are strided pixels (one phase of a strided data gradient), which no tiled tensor map can
          // describe.  Same staging tile as above, but the warp itself carries each 32x32 piece out: a
          // lane stages its own row, then eight lanes together write one row's 128 bytes, four rows per
          // instruction - whole 128-byte segments instead of 32 scattered 16-byte stores.
          const uint32_t stg = stg0;
          const int row = w.row0 + q * 32 + lane;
          const PhaseView pv = phase_view(w.phase);
          long long row_off = -1;   // rows >= M have no pixel
          if (row < pv.M) {
            const int img = row / pv.os_uv, r = row - img * pv.os_uv;
            const int u = r / pv.os_v, v = r - u * pv.os_v;
            row_off = img * p.os_sn + u * p.os_su + v * p.os_sv;
          }
          const int sub = lane >> 3, chunk = lane & 7;
#pragma unroll
          for (int g = 0; g < CW / 32; ++g) {
            const int c0 = w.col0 + h * CW + g * 32;
            if (c0 < p.N && w.row0 + q * 32 < pv.M) {   // warp-uniform
#pragma unroll
              for (int cq = 0; cq < 8; ++cq)
                sts128(stg + lane * 128 + ((cq ^ (lane & 7)) * 16),
                       make_float4(acc[g * 32 + cq * 4], acc[g * 32 + cq * 4 + 1], acc[g * 32 + cq * 4 + 2],
                                   acc[g * 32 + cq * 4 + 3]));
              __syncwarp();
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const int r = i * 4 + sub;
                const long long off = __shfl_sync(0xffffffffu, row_off, r);
                const float4 v = lds128(stg + r * 128 + ((chunk ^ (r & 7)) * 16));
                if (off >= 0 && c0 + chunk * 4 < p.N) {   // p.N is a multiple of 4 here: a vector is whole or absent
                  float* dst = w.out + off + c0 + chunk * 4;
                  if (plain && first) *reinterpret_cast<float4*>(dst) = v;
                  else *reinterpret_cast<float4*>(dst) = with_bias(g * 32 + chunk * 4, plus_old(v, dst));
                }
              }
              __syncwarp();   // the piece has been read before the next one overwrites it
            }
          }
        } else {
          const int row = w.row0 + q * 32 + lane;
          if (row < p.M) {
            const long long row_off = static_cast<long long>(row) * p.ldc;
            float* dst = w.out + row_off + w.col0 + h * CW;
            const int ncols = p.N - (w.col0 + h * CW);  // columns left in this row segment
            if (p.vec4_ok) {
#pragma unroll
              for (int j = 0; j < CW; j += 4) {
                if (j + 3 < ncols) {
                  if (plain && first)
                    *reinterpret_cast<float4*>(dst + j) = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
                  else
                    *reinterpret_cast<float4*>(dst + j) =
                        with_bias(j, plus_old(make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]), dst + j));
                } else {
#pragma unroll
                  for (int e = 0; e < 4; ++e)
                    if (j + e < ncols) dst[j + e] = first ? acc[j + e] : dst[j + e] + acc[j + e];
                }
              }
            } else {
#pragma unroll
              for (int j = 0; j < CW; ++j)
                if (j < ncols) dst[j] = first ? acc[j] : dst[j] + acc[j];
            }
          }
        }
        if (last) break;
        first = false;
        since = 0;
#pragma unroll
        for (int j = 0; j < CW; ++j) acc[j] = 0.0f;
      }
      if (!alive) break;
    }
    if constexpr (Cfg::REP)
      if (alive) forward_until(FW_STEPS, true);   // the last block's copies
    // stores still in flight read this CTA's shared memory: let them finish before exit
    if (lane == 0) tma_store_wait_all();
  }

  // ---- common exit: everyone arrives here, also after a give-up
  tc_fence_before();
  __syncthreads();
  if (p.clock_acc != nullptr && blockIdx.x == 0 && threadIdx.x == 0) {
    atomicAdd(p.clock_acc + 0, static_cast<unsigned long long>(clock64() - clk_t0));
    atomicAdd(p.clock_acc + 1, globaltimer_ns() - clk_g0);
    atomicAdd(p.clock_acc + 2, 1ull);
  }
  if (CTAS == 2) cluster_sync();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc<CTAS>(tmem_base, Cfg::TMEM_COLS);
  }
}

template <class Cfg>
__global__ void __launch_bounds__(Cfg::THREADS, 1) gemm_tf32_kernel(const __grid_constant__ GemmParams p) {
  if constexpr (Cfg::SOFTMAX) {     // launched with the below-ridge geometry unless a tuning key says otherwise
    if (p.ring_fixed == 2) gemm_tf32_body<Cfg, 2>(p);
    else gemm_tf32_body<Cfg, 0>(p);
  } else if constexpr (Cfg::ALT_RAW > 0) {
    if (p.ring_fixed == 1) gemm_tf32_body<Cfg, 1>(p);
    else if (p.ring_fixed == 2) gemm_tf32_body<Cfg, 2>(p);
    else gemm_tf32_body<Cfg, 0>(p);
  } else {
    if (p.ring_fixed == 1) gemm_tf32_body<Cfg, 1>(p);
    else gemm_tf32_body<Cfg, 0>(p);
  }
}

}  // namespace dragon
