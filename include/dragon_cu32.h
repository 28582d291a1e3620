/* C ABI of libdragon_cu32.so: the dense-contraction entry points of Dragon-Alpha's
 * Cu32 GPU library (Cuda_matMul, Cuda_batchMatMul, and the GEMM / GEMMR forward
 * convolution of Cuda_conv3D), implemented for NVIDIA B200 (sm_100a).
 *
 * One function per JNI native of the reference, same argument order and meaning;
 * the JNI-only leading arguments (JNIEnv*, jclass) are dropped and the jlongArray
 * of stream handles becomes `const int64_t* streams` (each element a cudaStream_t
 * cast to a 64-bit integer, exactly what the Java side stores in its long[]).
 * The library also exports the Java_z_dragon_engine_cuda_impl_math_* symbols
 * themselves (thin wrappers over these functions), so a JVM can bind it directly.
 *
 * Conventions shared by all functions (identical to the reference natives):
 *  - every pointer is a device pointer owned by the caller; nothing is allocated or
 *    retained by the library; outputs are fully overwritten, inputs untouched;
 *  - calls are asynchronous: work is enqueued on streams[0] and the function returns
 *    without synchronising the device; `length` is the number of valid stream handles
 *    (1..10);
 *  - matrices are dense row-major FP32; letters follow the reference:
 *    C[N,M] has N rows and M columns;
 *  - every row pitch must be a multiple of 4 floats and every base pointer 16-byte
 *    aligned (the Java engine pads all tensors this way);
 *  - arithmetic: FP32 in, FP32 out.  The plain entry points are FP32-accurate (each
 *    product is formed from a hi/lo TF32 split of both inputs, three tensor-core
 *    products per term); the `_mma` entry points are the single-pass TF32 fast mode
 *    the Java engine selects with its tf32 flag.
 *
 * Return value: 0 on success; a positive value is a cudaError_t reported by the CUDA
 * runtime for this call; negative values are argument errors (CU32_E_*).  The JNI
 * wrappers translate any non-zero value into z.dragon.engine.cuda.impl.CudaException.
 */
#ifndef DRAGON_CU32_H
#define DRAGON_CU32_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define CU32_API __attribute__((visibility("default")))
#else
#define CU32_API
#endif

#define CU32_OK 0
#define CU32_E_NULL (-1)        /* a required pointer is null */
#define CU32_E_DIM (-2)         /* a dimension is <= 0 or too large */
#define CU32_E_STREAMS (-3)     /* length outside 1..10 or streams == NULL */
#define CU32_E_ALIGN (-4)       /* pointer not 16-byte aligned or pitch % 4 != 0 */
#define CU32_E_GEOMETRY (-5)    /* convolution geometry the tensor-map path cannot express */
#define CU32_E_DRIVER (-6)      /* tensor-map encoder entry point not available in the driver */
#define CU32_E_TENSORMAP (-7)   /* the driver rejected a tensor map */
#define CU32_E_ARG (-8)         /* other invalid argument (e.g. GridZ < 1, unknown tuning key) */
#define CU32_E_SCRATCH (-9)     /* cu32_matMulT1SK_noalloc: (GridZ-1)*N*M exceeds the built-in scratch */

/* ------------------------------------------------------------------ Cuda_matMul
 * Reference: source/engine-cuda-base/Cuda_matMul/Cuda_matMul/A.cu,
 * Java natives: z/dragon/engine/cuda/impl/math/Cuda_matMul.java. */

/* C[N,M] = A[N,K] * B[K,M].          replaces JNI matMul      (A.cu:41-56) */
CU32_API int cu32_matMul(const int64_t* streams, int length, const float* dA, const float* dB, float* dC,
                int N, int M, int K);
/* C[N,M] = A[K,N]^T * B[K,M].        replaces JNI matMulT1    (A.cu:90-105) */
CU32_API int cu32_matMulT1(const int64_t* streams, int length, const float* dA, const float* dB, float* dC,
                  int N, int M, int K);
/* C[N,M] = A[N,K] * B[M,K]^T.        replaces JNI matMulT2    (A.cu:139-154) */
CU32_API int cu32_matMulT2(const int64_t* streams, int length, const float* dA, const float* dB, float* dC,
                  int N, int M, int K);

/* Split-K forms: K is cut into GridZ slices; slice 0 is written to C and slice z >= 1 to
 * Cbuf[(z-1)*N*M ...]; the caller then sums them with cu32_SKbuf_summary.  Cbuf holds
 * (GridZ-1)*N*M floats.  Slice boundaries are multiples of 32 (the reference cuts at
 * multiples of 8, Cuda_matMul/micro.cuh:92); the sum over slices is the same product.
 * replaces JNI matMulSK (A.cu:59-79), matMulT1SK (A.cu:108-128), matMulT2SK (A.cu:157-178) */
CU32_API int cu32_matMulSK(const int64_t* streams, int length, int GridZ, const float* dA, const float* dB,
                  float* dC, float* dCbuf, int N, int M, int K);
CU32_API int cu32_matMulT1SK(const int64_t* streams, int length, int GridZ, const float* dA, const float* dB,
                    float* dC, float* dCbuf, int N, int M, int K);
CU32_API int cu32_matMulT2SK(const int64_t* streams, int length, int GridZ, const float* dA, const float* dB,
                    float* dC, float* dCbuf, int N, int M, int K);

/* C[i] += sum_{p < part} Cbuf[p*sizeC + i], compensated (Kahan) summation, in place.
 * replaces JNI SKbuf_summary (A.cu:20-30, SKbufsum.cuh:29-81) */
CU32_API int cu32_SKbuf_summary(int64_t stream, const float* dCbuf, float* dC, int part, int sizeC);

/* Single-pass TF32 fast mode; declared by the Java class (Cuda_matMul.java:163-166, :278-282,
 * :369-373) and called when the engine's tf32 flag is set; absent from the published C++. */
CU32_API int cu32_matMul_mma(const int64_t* streams, int length, const float* dA, const float* dB, float* dC,
                    int N, int M, int K);
CU32_API int cu32_matMulT1_mma(const int64_t* streams, int length, const float* dA, const float* dB,
                      float* dC, int N, int M, int K);
CU32_API int cu32_matMulT2_mma(const int64_t* streams, int length, const float* dA, const float* dB,
                      float* dC, int N, int M, int K);

/* Product stored to several buffers at once.  No counterpart in the reference (a single-GPU engine).
 * C = A*B (cu32_matMul_replicated) or A*B^T (cu32_matMulT2_replicated) exactly as the plain entry points, and every
 * store to dC is repeated, from the same shared-memory tile, to each of the n_replicas (0..7) buffers in
 * dC_replicas (same [N, M] layout, 16-byte aligned).  The use: the ranks of one NVLink domain each own a block of
 * rows of a larger product; a rank passes, for every peer, the address of its own block inside the peer's copy of
 * the full output (peer memory mapped into this process), and the reassembly that would otherwise be an all-gather
 * after the product rides on the epilogue's stores - nothing is ever loaded from a peer.  The caller orders the
 * end of the call before any peer reads (a barrier over the ranks after the stream has drained). */
CU32_API int cu32_matMul_replicated(const int64_t* streams, int length, const float* dA, const float* dB, float* dC,
                                    float* const* dC_replicas, int n_replicas, int N, int M, int K);
CU32_API int cu32_matMulT2_replicated(const int64_t* streams, int length, const float* dA, const float* dB, float* dC,
                                      float* const* dC_replicas, int n_replicas, int N, int M, int K);

/* Split-K A^T*B that allocates nothing and needs no partial buffer from the caller.
 * No counterpart in the reference (its split-K natives always take a caller-allocated Cbuf).
 *
 * C[N,M] = A[K,N]^T * B[K,M], K cut into GridZ slices, partials summed (Kahan) into C, all on
 * streams[0]; the result is the same as cu32_matMulT1SK followed by cu32_SKbuf_summary.
 *
 * Who needs it: hosts that cannot obtain device memory at the moment of the call - an engine
 * whose memory pool has already handed out everything it reserved (the Java engine takes the
 * partial buffer from such a pool, CudaFloat32EngineBase.java:1565-1568), or a thread that
 * must not trigger the device-wide synchronisation an allocation or a free implies.  For them
 * the partial products go to a scratch array compiled into the library:
 *  - capacity CU32_NOALLOC_SCRATCH_FLOATS floats (16 MiB), i.e. (GridZ-1)*N*M must not exceed
 *    it (e.g. 512x512 with GridZ <= 17); larger requests return CU32_E_SCRATCH and do nothing;
 *  - every GPU that loads the library carries the array for the life of the process;
 *  - the array is shared by all calls on a device: two calls whose GPU work can overlap
 *    (different streams, no ordering between them) race on it - serialise them.  Its contents
 *    after a call are the last call's partials; every call overwrites all the floats it reads
 *    back, so nothing has to be cleared beforehand;
 *  - the first call on each device looks up the array's device address (cudaGetSymbolAddress);
 *    make that first call outside any stream capture.
 * The function calls no allocation or free routine of the CUDA runtime or of any library. */
#define CU32_NOALLOC_SCRATCH_FLOATS (4 * 1024 * 1024)
CU32_API int cu32_matMulT1SK_noalloc(const int64_t* streams, int length, int GridZ, const float* dA,
                                     const float* dB, float* dC, int N, int M, int K);

/* ------------------------------------------------------------------ Cuda_batchMatMul
 * Reference: source/engine-cuda-base/Cuda_batchMatMul/Cuda_batchMatMul/A.cu. */

/* C[b][N,M] = A[b][N,AK] * B[b][BK,M]; the reduction runs over BK, AK >= BK is A's pitch.
 * replaces JNI batchMatMul (A.cu:20-39) and batchMatMul_texture (A.cu:42-62) */
CU32_API int cu32_batchMatMul(const int64_t* streams, int length, const float* dA, const float* dB, float* dC,
                     int Batch, int N, int M, int BK, int AK);
CU32_API int cu32_batchMatMul_texture(const int64_t* streams, int length, const float* dA, const float* dB,
                             float* dC, int Batch, int N, int M, int BK, int AK);
/* C[b][CN,M] = A[b][K,AN]^T * B[b][K,M]; AN >= CN is A's pitch.
 * replaces JNI batchMatMulT1 (A.cu:71-89) */
CU32_API int cu32_batchMatMulT1(const int64_t* streams, int length, const float* dA, const float* dB,
                       float* dC, int Batch, int CN, int AN, int M, int K);
/* C[b][N,CM] = A[b][N,K] * B[b][BM,K]^T; CM >= BM is C's pitch, columns BM..CM-1 are written 0.
 * replaces JNI batchMatMulT2 (A.cu:98-116) and batchMatMulT2_texture (A.cu:119-143) */
CU32_API int cu32_batchMatMulT2(const int64_t* streams, int length, const float* dA, const float* dB,
                       float* dC, int Batch, int N, int CM, int BM, int K);
CU32_API int cu32_batchMatMulT2_texture(const int64_t* streams, int length, const float* dA, const float* dB,
                               float* dC, int Batch, int N, int CM, int BM, int K);
/* TF32 fast mode (Cuda_batchMatMul.java:166-170, :236-239, :355-359). */
CU32_API int cu32_batchMatMul_mma(int useTexture, const int64_t* streams, int length, const float* dA,
                         const float* dB, float* dC, int Batch, int N, int M, int BK, int AK);
CU32_API int cu32_batchMatMulT1_mma(const int64_t* streams, int length, const float* dA, const float* dB,
                           float* dC, int Batch, int CN, int AN, int M, int K);
CU32_API int cu32_batchMatMulT2_mma(int useTexture, const int64_t* streams, int length, const float* dA,
                           const float* dB, float* dC, int Batch, int N, int CM, int BM, int K);

/* ------------------------------------------------------------------ Cuda_conv3D (GEMM / GEMMR)
 * Reference: source/engine-cuda-base/Cuda_conv3D/Cuda_conv3D/A.cu.
 * X[N,IH,IW,IC] (NHWC), W[OC,FH,FW,IC], CW[FH,FW,IC,OC], Y[N,OH,OW,OC];
 * Y[n,oh,ow,oc] = sum_{fh,fw,ic} X[n, oh*sh-ph+fh, ow*sw-pw+fw, ic] * W[oc,fh,fw,ic],
 * zero outside the image. */

/* CW[fh,fw,ic,oc] = W[oc,fh,fw,ic].   replaces JNI kernel_remode (A.cu:18-28) */
CU32_API int cu32_kernel_remode(int64_t stream, const float* dW, float* dCW, int FH, int FW, int OC, int IC);

/* replaces JNI conv3D_GemmR (A.cu:169-191), conv3D_GemmR_texture (A.cu:245-268) and their
 * _SGM forms (A.cu:194-236, :271-314; GM_slice only bounds the reference's grid size and does
 * not change the result) */
CU32_API int cu32_conv3D_GemmR(const int64_t* streams, int length, const float* dX, int IH, int IW,
                      const float* dW, const float* dCW, int FH, int FW, float* dY, int OH, int OW,
                      int N, int IC, int OC, int sh, int sw, int ph, int pw);
CU32_API int cu32_conv3D_GemmR_texture(const int64_t* streams, int length, const float* dX, int IH, int IW,
                              const float* dW, const float* dCW, int FH, int FW, float* dY, int OH,
                              int OW, int N, int IC, int OC, int sh, int sw, int ph, int pw);
CU32_API int cu32_conv3D_GemmR_SGM(const int64_t* streams, int length, const float* dX, int IH, int IW,
                          const float* dW, const float* dCW, int FH, int FW, float* dY, int OH,
                          int OW, int N, int IC, int OC, int sh, int sw, int ph, int pw,
                          int GM_slice);
CU32_API int cu32_conv3D_GemmR_texture_SGM(const int64_t* streams, int length, const float* dX, int IH,
                                  int IW, const float* dW, const float* dCW, int FH, int FW,
                                  float* dY, int OH, int OW, int N, int IC, int OC, int sh, int sw,
                                  int ph, int pw, int GM_slice);
/* 1x1, stride 1, no padding.  replaces JNI conv3D_GemmR_W1 (A.cu:323-341) and conv3D_GemmR_W1_SGM (A.cu:344-381) */
CU32_API int cu32_conv3D_GemmR_W1(const int64_t* streams, int length, const float* dX, int IH, int IW,
                         const float* dW, const float* dCW, float* dY, int N, int IC, int OC);
CU32_API int cu32_conv3D_GemmR_W1_SGM(const int64_t* streams, int length, const float* dX, int IH, int IW,
                             const float* dW, const float* dCW, float* dY, int N, int IC, int OC,
                             int GM_slice);
/* Filter not remoded (W only).  replaces JNI conv3D (A.cu:39-60), conv3D_texture (A.cu:63-87),
 * conv3D_np (A.cu:114-136, no padding) and conv3D_W1 (A.cu:138-155) */
CU32_API int cu32_conv3D(const int64_t* streams, int length, const float* dX, int IH, int IW,
                const float* dW, int FH, int FW, float* dY, int OH, int OW, int N, int IC, int OC,
                int sh, int sw, int ph, int pw);
CU32_API int cu32_conv3D_texture(const int64_t* streams, int length, const float* dX, int IH, int IW,
                        const float* dW, int FH, int FW, float* dY, int OH, int OW, int N, int IC,
                        int OC, int sh, int sw, int ph, int pw);
CU32_API int cu32_conv3D_np(const int64_t* streams, int length, const float* dX, int IH, int IW,
                   const float* dW, int FH, int FW, float* dY, int OH, int OW, int N, int IC, int OC,
                   int sh, int sw);
CU32_API int cu32_conv3D_W1(const int64_t* streams, int length, const float* dX, int IH, int IW,
                   const float* dW, float* dY, int N, int IC, int OC);

/* The reference's other forward-convolution natives, as further names for the same implicit GEMM.
 * With default flags the Java engine sends most stride-1 3x3..9x9 convolutions to these
 * (CudaFloat32EngineBase.java:2211-2255, :2300-2385) rather than to conv3D_GemmR; exporting them
 * makes the library a drop-in for default-configured models.  They compute exactly what
 * cu32_conv3D / cu32_conv3D_GemmR compute (the reference's V2 and Im2col-Winograd algorithms differ
 * only in rounding); useTexture and GM_slice are accepted and ignored.
 *   cu32_conv3DV2                              replaces JNI conv3DV2 (A.cu:89-111)
 *   cu32_conv3D_GemmV2R                        replaces JNI conv3D_GemmV2R (A.cu:390-412)
 *   cu32_conv3D_Im2col_Winograd_s8_R_texture   replaces JNI conv3D_Im2col_Winograd_s8_R_texture (A.cu:429-455)
 *   cu32_conv3D_Im2col_WinogradR_s8_texture_SGM   ... (A.cu:458-530)
 *   cu32_conv3D_Im2col_Winograd_s16_R_texture  ... (A.cu:539-565)
 *   cu32_conv3D_Im2col_WinogradR_s16_texture_SGM  ... (A.cu:568-637)
 * The Winograd natives are stride-1 only (no sh, sw) and return a jboolean "handled" to Java; here
 * every shape is handled, so the JNI shim returns true whenever the return code is 0. */
CU32_API int cu32_conv3DV2(int useTexture, const int64_t* streams, int length, const float* dX, int IH, int IW,
                  const float* dW, int FH, int FW, float* dY, int OH, int OW, int N, int IC, int OC,
                  int sh, int sw, int ph, int pw);
CU32_API int cu32_conv3D_GemmV2R(int useTexture, const int64_t* streams, int length, const float* dX, int IH,
                        int IW, const float* dW, const float* dCW, int FH, int FW, float* dY, int OH,
                        int OW, int N, int IC, int OC, int sh, int sw, int ph, int pw);
CU32_API int cu32_conv3D_Im2col_Winograd_s8_R_texture(int useTexture, const int64_t* streams, int length,
                        const float* dX, int IH, int IW, const float* dW, const float* dCW, int FH,
                        int FW, float* dY, int OH, int OW, int N, int IC, int OC, int ph, int pw);
CU32_API int cu32_conv3D_Im2col_WinogradR_s8_texture_SGM(int useTexture, const int64_t* streams, int length,
                        const float* dX, int IH, int IW, const float* dW, const float* dCW, int FH,
                        int FW, float* dY, int OH, int OW, int N, int IC, int OC, int ph, int pw,
                        int GM_slice);
CU32_API int cu32_conv3D_Im2col_Winograd_s16_R_texture(int useTexture, const int64_t* streams, int length,
                        const float* dX, int IH, int IW, const float* dW, const float* dCW, int FH,
                        int FW, float* dY, int OH, int OW, int N, int IC, int OC, int ph, int pw);
CU32_API int cu32_conv3D_Im2col_WinogradR_s16_texture_SGM(int useTexture, const int64_t* streams, int length,
                        const float* dX, int IH, int IW, const float* dW, const float* dCW, int FH,
                        int FW, float* dY, int OH, int OW, int N, int IC, int OC, int ph, int pw,
                        int GM_slice);

/* ------------------------------------------------------------------ Cuda_dconv3D_deltaX, stride 1
 * Data gradient of the forward convolution above for stride 1 (file:line below are in
 * engine-cuda-base/Cuda_dconv3D_deltaX/Cuda_dconv3D_deltaX/):
 *   deltaX[n,ih,iw,ic] = sum_{fh,fw,oc} deltaY[n, ih+ph-fh, iw+pw-fw, oc] * W[oc,fh,fw,ic], zero outside deltaY;
 *   deltaY[N,OH,OW,OC], W[OC,FH,FW,IC] (the forward filter, unchanged), deltaX[N,IH,IW,IC],
 *   IC % 4 == 0, OC % 4 == 0.  The forward convolution gives IH = OH - 1 + FH - 2*ph (likewise the width), but
 *   any pair of extents is served, as by the reference (its own test pairs IH = OH = 64 with an 8x8 filter,
 *   padding 4: test/cuda/conv3D/Cuda_conv3D_dX_test.java:178,216): the sum simply runs over the rows that exist.
 * It runs as a forward implicit GEMM over deltaY with padding (FH-1-ph, FW-1-pw) and the filter taps
 * reversed, W being read where it lies.  (Strides > 1: next section.)
 *   cu32_dconv3D_deltaX_s1[_texture][_SGM]   replace JNI dconv3D_deltaX_s1 (A.cu:21-42), _s1_SGM (:45-94),
 *                                            _s1_texture (:97-120), _s1_texture_SGM (:123-174)
 *   cu32_dconv3D_deltaX_W1[_SGM]             replace JNI dconv3D_deltaX_W1 (:177-196), _W1_SGM (:199-240): 1x1 filter
 *   cu32_dconv3D_deltaX_V2_s1                replaces JNI dconv3D_deltaX_V2_s1 (:243-277)
 *   cu32_dconv3D_deltaX_Im2col_Winograd_s8/s16_texture[_SGM]   replace JNI Im2col_Winograd_* (:837-1040); the
 *                                            JNI shim returns "handled" = true whenever the return code is 0
 * useTexture and GM_slice are accepted and ignored. */
CU32_API int cu32_dconv3D_deltaX_s1(const int64_t* streams, int length, const float* d_deltaY, int OH, int OW,
                           const float* dW, int FH, int FW, float* d_deltaX, int IH, int IW, int N, int IC,
                           int OC, int ph, int pw);
CU32_API int cu32_dconv3D_deltaX_s1_texture(const int64_t* streams, int length, const float* d_deltaY, int OH, int OW,
                           const float* dW, int FH, int FW, float* d_deltaX, int IH, int IW, int N, int IC,
                           int OC, int ph, int pw);
CU32_API int cu32_dconv3D_deltaX_s1_SGM(const int64_t* streams, int length, const float* d_deltaY, int OH, int OW,
                           const float* dW, int FH, int FW, float* d_deltaX, int IH, int IW, int N, int IC,
                           int OC, int ph, int pw, int GM_slice);
CU32_API int cu32_dconv3D_deltaX_s1_texture_SGM(const int64_t* streams, int length, const float* d_deltaY, int OH,
                           int OW, const float* dW, int FH, int FW, float* d_deltaX, int IH, int IW, int N,
                           int IC, int OC, int ph, int pw, int GM_slice);
CU32_API int cu32_dconv3D_deltaX_V2_s1(int useTexture, const int64_t* streams, int length, const float* d_deltaY,
                           int OH, int OW, const float* dW, int FH, int FW, float* d_deltaX, int IH, int IW,
                           int N, int IC, int OC, int ph, int pw);
CU32_API int cu32_dconv3D_deltaX_W1(const int64_t* streams, int length, const float* d_deltaY, const float* dW,
                           float* d_deltaX, int IH, int IW, int N, int IC, int OC);
CU32_API int cu32_dconv3D_deltaX_W1_SGM(const int64_t* streams, int length, const float* d_deltaY, const float* dW,
                           float* d_deltaX, int IH, int IW, int N, int IC, int OC, int GM_slice);
CU32_API int cu32_dconv3D_deltaX_Im2col_Winograd_s8_texture(int useTexture, const int64_t* streams, int length,
                           const float* d_deltaY, int OH, int OW, const float* dW, int FH, int FW,
                           float* d_deltaX, int IH, int IW, int N, int IC, int OC, int ph, int pw);
CU32_API int cu32_dconv3D_deltaX_Im2col_Winograd_s8_texture_SGM(int useTexture, const int64_t* streams, int length,
                           const float* d_deltaY, int OH, int OW, const float* dW, int FH, int FW,
                           float* d_deltaX, int IH, int IW, int N, int IC, int OC, int ph, int pw, int GM_slice);
CU32_API int cu32_dconv3D_deltaX_Im2col_Winograd_s16_texture(int useTexture, const int64_t* streams, int length,
                           const float* d_deltaY, int OH, int OW, const float* dW, int FH, int FW,
                           float* d_deltaX, int IH, int IW, int N, int IC, int OC, int ph, int pw);
CU32_API int cu32_dconv3D_deltaX_Im2col_Winograd_s16_texture_SGM(int useTexture, const int64_t* streams, int length,
                           const float* d_deltaY, int OH, int OW, const float* dW, int FH, int FW,
                           float* d_deltaX, int IH, int IW, int N, int IC, int OC, int ph, int pw, int GM_slice);

/* ------------------------------------------------------------------ data gradient + bias row (optional)
 * The Java engine's transposed convolution (deconv3D_biased, CudaFloat32EngineBase.java:2590-2740) runs a deltaX native
 * and then Cuda_function.linear_dual2D_row(Y, Bias, 1, 1, 0, Y, lengthv, width, stride) as a second kernel; these two
 * add the bias row (IC floats; columns >= width come out 0) in the epilogue with the bits of that sequence.  _s1: the
 * forward filter as it lies; _ksImsR: the ks_remodev2 workspace, any stride (FH >= sh and FW >= sw required here).
 * No counterpart among the reference's natives. */
CU32_API int cu32_dconv3D_deltaX_s1_biased(const int64_t* streams, int length, const float* d_deltaY, int OH, int OW,
                           const float* dW, int FH, int FW, float* d_deltaX, int IH, int IW, int N, int IC, int OC,
                           int ph, int pw, const float* dBias, int width);
CU32_API int cu32_dconv3D_deltaX_ksImsR_biased(const int64_t* streams, int length, const float* d_deltaY, int OH, int OW,
                           const float* dCW, int FH, int FW, float* d_deltaX, int IH, int IW, int N, int IC, int OC,
                           int sh, int sw, int ph, int pw, const float* dBias, int width);

/* ------------------------------------------------------------------ batched contraction + scale (optional)
 * C = alpha * (A x B) with the product rounded to FP32 first and the scale applied as one fused multiply-add with a
 * zero addend - the bits of the reference's two-kernel sequence batchMatMul* followed by sdiv(sqrt(d), C) =
 * linear2D(1/sqrt(d), C, 0) (nn/unit/complex/block/ImageMHA.java:67-68, Engine.java:4002,
 * Cuda_function/type1_linear2D.cuh:40-58, micro.cuh:54-58) - without the second pass over C.  No counterpart among the
 * reference's natives; arguments as the unscaled entry points plus alpha.  C must be 16-byte aligned with a pitch that
 * is a multiple of 4 floats (CU32_E_ALIGN otherwise). */
CU32_API int cu32_batchMatMul_scaled(const int64_t* streams, int length, const float* dA, const float* dB, float* dC,
                           int Batch, int N, int M, int BK, int AK, float alpha);
CU32_API int cu32_batchMatMulT1_scaled(const int64_t* streams, int length, const float* dA, const float* dB, float* dC,
                           int Batch, int CN, int AN, int M, int K, float alpha);
CU32_API int cu32_batchMatMulT2_scaled(const int64_t* streams, int length, const float* dA, const float* dB, float* dC,
                           int Batch, int N, int CM, int BM, int K, float alpha);

/* ------------------------------------------------------------------ Cuda_dconv3D_deltaW
 * deltaW[oc,fh,fw,ic] = sum over (n,oh,ow) of deltaY[n,oh,ow,oc] * X[n, oh*sh-ph+fh, ow*sw-pw+fw, ic] (zero outside
 * the image); X [N,IH,IW,IC], deltaY [N,OH,OW,OC], deltaW [OC,FH,FW,IC], IC and OC multiples of 4.  These replace the
 * natives of the Java class z/dragon/engine/cuda/impl/math/Cuda_dconv3D_deltaW.java (:288 dconv3D_deltaW, :342 _W1,
 * :352 buf_summary, :404 _GemmSK, :473 _GemmV2SK, :518 _GemmSK_W1, :557/:595/:634 Im2col_WinogradV2_SHW_s4/s8/s16);
 * the reference's CUDA source for them is not published, so argument order and the split-K protocol follow the Java
 * declarations and their caller (CudaFloat32EngineBase.java:3520-3640): slice 0 of the reduction over pixels goes to
 * deltaW, slice s = 1..GridZ-1 to d_deltaW_buf + (s-1)*OC*FH*FW*IC, and buf_summary adds the partials into deltaW.
 * The Winograd natives return through the JNI layer as "handled"; OH_slice, OW_slice, c64 and n are ignored. */
CU32_API int cu32_dconv3D_deltaW(const int64_t* streams, int length, const float* dX, int IH, int IW,
                           const float* d_deltaY, int OH, int OW, float* d_deltaW, int FH, int FW, int N, int IC,
                           int OC, int sh, int sw, int ph, int pw);
CU32_API int cu32_dconv3D_deltaW_W1(const int64_t* streams, int length, const float* dX, int IH, int IW,
                           const float* d_deltaY, float* d_deltaW, int N, int IC, int OC);
CU32_API int cu32_dconv3D_deltaW_buf_summary(int64_t stream, const float* d_deltaW_buf, float* d_deltaW, int part,
                           int sizeW);
CU32_API int cu32_dconv3D_deltaW_GemmSK(const int64_t* streams, int length, int GridZ, const float* dX, int IH, int IW,
                           const float* d_deltaY, int OH, int OW, float* d_deltaW, float* d_deltaW_buf, int FH, int FW,
                           int N, int IC, int OC, int sh, int sw, int ph, int pw);
CU32_API int cu32_dconv3D_deltaW_GemmV2SK(const int64_t* streams, int length, int GridZ, const float* dX, int IH,
                           int IW, const float* d_deltaY, int OH, int OW, float* d_deltaW, float* d_deltaW_buf, int FH,
                           int FW, int N, int IC, int OC, int sh, int sw, int ph, int pw);
CU32_API int cu32_dconv3D_deltaW_GemmSK_W1(const int64_t* streams, int length, int GridZ, const float* dX, int IH,
                           int IW, const float* d_deltaY, float* d_deltaW, float* d_deltaW_buf, int N, int IC, int OC);
CU32_API int cu32_dconv3D_deltaW_Im2col_WinogradV2_SHW_s4_texture(const int64_t* streams, int length, int GridZ,
                           int OH_slice, int OW_slice, const float* dX, int IH, int IW, const float* d_deltaY, int OH,
                           int OW, float* d_deltaW, float* d_deltaW_buf, int FH, int FW, int N, int IC, int OC, int ph,
                           int pw, int n);
CU32_API int cu32_dconv3D_deltaW_Im2col_WinogradV2_SHW_s8_texture(const int64_t* streams, int length, int GridZ,
                           int OH_slice, int OW_slice, const float* dX, int IH, int IW, const float* d_deltaY, int OH,
                           int OW, float* d_deltaW, float* d_deltaW_buf, int FH, int FW, int N, int IC, int OC, int ph,
                           int pw, int n);
CU32_API int cu32_dconv3D_deltaW_Im2col_WinogradV2_SHW_s16_texture(const int64_t* streams, int length, int GridZ,
                           int OH_slice, int OW_slice, int c64, const float* dX, int IH, int IW, const float* d_deltaY,
                           int OH, int OW, float* d_deltaW, float* d_deltaW_buf, int FH, int FW, int N, int IC, int OC,
                           int ph, int pw, int n);

/* ------------------------------------------------------------------ Cuda_dconv3D_deltaX, any stride
 * deltaX[n,ih,iw,ic] = sum over (oh,ow,fh,fw,oc) with oh*sh - ph + fh == ih and ow*sw - pw + fw == iw of
 * deltaY[n,oh,ow,oc] * W[oc,fh,fw,ic];  the forward convolution gives OH = (IH + 2*ph - FH) / sh + 1 (likewise OW),
 * any other pair of extents is served as well (the sum runs over the rows that exist).  Computed as sh*sw stride-1
 * sub-problems, one per residue of (ih + ph, iw + pw) modulo the stride, each a launch of the contraction kernel
 * whose output rows are the strided pixels of that residue class.
 *   cu32_ks_remode / cu32_ks_remodev2   replace JNI ks_remode (A.cu:280-291) and ks_remodev2 (:294-306): the filter
 *       workspace CW[sh*sw][...] of OC*CFH*CFW*IC floats per phase, CFH = ceil(FH/sh), CFW = ceil(FW/sw), bit for
 *       bit the reference's layouts (v1: [oc][fhr][fwr][ic], v2: [fhr][fwr][oc][ic], taps reversed)
 *   cu32_dconv3D_deltaX_kernelSplit[_SGM], _ksImsR[_SGM|_texture|_texture_SGM]   replace JNI (:314-386, :389-540);
 *       dCW is the ks_remodev2 workspace, which is what the Java engine passes (CudaFloat32EngineBase.java:3824-3900)
 *   cu32_dconv3D_deltaX_ksIms2R[_SGM|_texture|_texture_SGM], _ksV2_Ims2R   replace JNI (:543-728): stride 2 x 2
 *   cu32_dconv3D_deltaX_crossAdd[_SGM]   replace JNI (:731-834): takes the forward filter W itself (read in place)
 * The reference's Ims natives require IH % sh == 0 and IW % sw == 0; these do not. */
CU32_API int cu32_ks_remode(int64_t stream, const float* dW, int FH, int FW, float* dCW, int CFH, int CFW, int OC,
                   int IC, int sh, int sw);
CU32_API int cu32_ks_remodev2(int64_t stream, const float* dW, int FH, int FW, float* dCW, int CFH, int CFW, int OC,
                     int IC, int sh, int sw);
#define CU32_DX_KS_ARGS const int64_t* streams, int length, const float* d_deltaY, int OH, int OW, const float* dCW, \
                        int FH, int FW, float* d_deltaX, int IH, int IW, int N, int IC, int OC
CU32_API int cu32_dconv3D_deltaX_kernelSplit(CU32_DX_KS_ARGS, int sh, int sw, int ph, int pw);
CU32_API int cu32_dconv3D_deltaX_kernelSplit_SGM(CU32_DX_KS_ARGS, int sh, int sw, int ph, int pw, int GM_slice);
CU32_API int cu32_dconv3D_deltaX_ksImsR(CU32_DX_KS_ARGS, int sh, int sw, int ph, int pw);
CU32_API int cu32_dconv3D_deltaX_ksImsR_SGM(CU32_DX_KS_ARGS, int sh, int sw, int ph, int pw, int GM_slice);
CU32_API int cu32_dconv3D_deltaX_ksImsR_texture(CU32_DX_KS_ARGS, int sh, int sw, int ph, int pw);
CU32_API int cu32_dconv3D_deltaX_ksImsR_texture_SGM(CU32_DX_KS_ARGS, int sh, int sw, int ph, int pw, int GM_slice);
CU32_API int cu32_dconv3D_deltaX_ksIms2R(CU32_DX_KS_ARGS, int ph, int pw);
CU32_API int cu32_dconv3D_deltaX_ksIms2R_SGM(CU32_DX_KS_ARGS, int ph, int pw, int GM_slice);
CU32_API int cu32_dconv3D_deltaX_ksIms2R_texture(CU32_DX_KS_ARGS, int ph, int pw);
CU32_API int cu32_dconv3D_deltaX_ksIms2R_texture_SGM(CU32_DX_KS_ARGS, int ph, int pw, int GM_slice);
CU32_API int cu32_dconv3D_deltaX_ksV2_Ims2R(int useTexture, CU32_DX_KS_ARGS, int ph, int pw);
CU32_API int cu32_dconv3D_deltaX_crossAdd(const int64_t* streams, int length, const float* d_deltaY, int OH, int OW,
                           const float* dW, int FH, int FW, float* d_deltaX, int IH, int IW, int N, int IC,
                           int OC, int sh, int sw, int ph, int pw);
CU32_API int cu32_dconv3D_deltaX_crossAdd_SGM(const int64_t* streams, int length, const float* d_deltaY, int OH,
                           int OW, const float* dW, int FH, int FW, float* d_deltaX, int IH, int IW, int N,
                           int IC, int OC, int sh, int sw, int ph, int pw, int GM_slice);

/* ------------------------------------------------------------------ contraction + bias row
 * No counterpart among the reference's natives.  The Java engine's matMul_biased / conv3D_biased
 * (CudaFloat32EngineBase.java:1594-1688, :2389-2542) run the contraction and then, as a second
 * kernel on the same stream, Cuda_function.linear_dual2D_row(C, Bias, row_lengthv, 1, 1, 0, C,
 * lengthv, width, stride) (Cuda_function/type1_linear_dual2D_row.cuh:41-70): every row gets the
 * bias vector added and the padding columns (width <= col < stride) are zeroed.  These entry points
 * do both in one pass: the add happens on the FP32 value the contraction would have stored, so the
 * result has the same bits as the two-kernel sequence, and one read and one write of C are saved.
 *   Bias: M (resp. OC) floats, 16-byte aligned; width: true row width, 0 < width <= M (resp. OC).
 * Split-K: run cu32_matMulSK as before and replace SKbuf_summary + linear_dual2D_row by
 * cu32_SKbuf_summary_biased (part may be 0: then it is the bias add alone). */
CU32_API int cu32_matMul_biased(const int64_t* streams, int length, const float* dA, const float* dB, float* dC,
                       const float* dBias, int N, int M, int K, int width);
CU32_API int cu32_matMul_mma_biased(const int64_t* streams, int length, const float* dA, const float* dB,
                           float* dC, const float* dBias, int N, int M, int K, int width);
CU32_API int cu32_SKbuf_summary_biased(int64_t stream, const float* dCbuf, float* dC, const float* dBias,
                              int part, int sizeC, int M, int width);
CU32_API int cu32_conv3D_GemmR_biased(const int64_t* streams, int length, const float* dX, int IH, int IW,
                             const float* dW, const float* dCW, int FH, int FW, float* dY, int OH,
                             int OW, int N, int IC, int OC, int sh, int sw, int ph, int pw,
                             const float* dBias, int width);

/* Attention scores in one pass (no counterpart among the reference's natives).
 * P[b][N, CM] = softmax over each row of alpha * A[b][N,K] * B[b][BM,K]^T: columns 0..BM-1 hold the softmax,
 * the pitch padding BM..CM-1 holds zeros.  Arguments as cu32_batchMatMulT2 plus the scale.
 * What it replaces in the reference's attention block (nn/unit/complex/block/ImageMHA.java:67-68): batchMatMulT2,
 * then linear2D (sdiv by sqrt(d), Engine.java:4002), then softmax2D = row_max + row_softmax + div2D_field
 * (CudaFloat32EngineBase.java:5738-5775) - five kernels that write the score tensor three times and read it four.
 * For rows of at most 512 columns and K <= 64 the product stays in tensor memory until the row is normalised, so
 * the scores are written once and never read; longer rows or reductions run the scaled product followed by one
 * in-place row softmax.  Values: x' = fma(x, alpha, 0), e = expf(x' - max x'), p = e * (1 / sum e); they differ
 * from the five-kernel sequence only in the order of the row sum and in multiplying by the reciprocal instead of
 * dividing (a few units in the last place). */
CU32_API int cu32_batchMatMulT2_softmax(const int64_t* streams, int length, const float* dA, const float* dB,
                                        float* dP, int Batch, int N, int CM, int BM, int K, float alpha);

/* ------------------------------------------------------------------ library control
 * No counterpart in the reference (its only native-side switch is a compile-time macro). */

/* Tuning / diagnostics knobs, process-wide.  Keys:
 *   "kc"       k-blocks (of 32) accumulated inside the tensor core before each FP32
 *              register add, FP32-accurate mode (default 2)
 *   "kc_fast"  same for the TF32 fast mode (default 4)
 *   "tile"     force a tile configuration: 0..5 = 128x64, 128x128, 128x256, 256x128 pair,
 *              256x256 pair, 256x64 pair; -1 = choose from the shape (default)
 *   "l2hint"   L2 eviction priority of the operand loads: 0 = none (default; measured best),
 *              1 = A evict-last and B evict-first, 2 = A evict-last only
 *   "ring_raw", "ring_lo", "store_bufs"
 *              shared-memory pipeline of the contraction kernel: slots for raw operand tiles (2..8), slots
 *              for their low-order parts (1..ring_raw) and store-staging tiles per drain warp (1, 2);
 *              0 = choose from the shape (default).  A combination that does not fit in shared memory
 *              makes the call return cudaErrorInvalidValue.
 *   "clock"    1 = CTA 0 of every contraction launch adds its run time in SM cycles and in nanoseconds to a
 *              device-side accumulator (cu32_read_clock); 0 = off (default)
 *   "gather"   1 = the convolution family builds its im2col tiles with plain loads even where a tensor map could
 *              (diagnostics: same bits); 0 = only for geometries no tensor map can express (default)
 *   "phase_overlap" 1 = the launches of a strided data gradient's phases may overlap one another (default); 0 = serial
 *   "ring_fixed"    1 = launches whose rings are the tile's default use the kernel path with compile-time ring geometry
 *                   (default); 0 = always the launch-parameter path (diagnostics: same bits)
 *   "ring_paired"   1 = with equally long rings each lo tile sits right behind its raw tile (default); 0 = two separate rings
 *   "phase_fused"   1 = a strided data gradient with 2 to 4 phases runs them in one launch, a CTA taking tile j of every
 *                   phase in turn (default); 0 = one launch per phase (same bits)
 *   "rep_lazy"      1 = the replicated entry points store a finished block to C and carry it to the copies while the
 *                   next tile is multiplied (default); 0 = every store is repeated to every copy at once
 *   "sm_reserve" SMs the contraction kernel's persistent grid leaves free, for kernels a host runs beside it on
 *              another stream (a collective that reassembles output shards); 0 = none (default)
 *   "last_tile" (read only) tile configuration of the most recent contraction call of this process
 *   "arrive_release"  1 = barrier arrivals between the two CTAs of a pair carry a cluster-scope release
 *              (diagnostics: results must not depend on it); 0 = default
 * Returns 0, or CU32_E_ARG for an unknown key / out-of-range value. */
CU32_API int cu32_tune(const char* key, int value);
CU32_API int cu32_get_tune(const char* key, int* value);

/* Device-side give-up word of the current device: 0 if no kernel of this library ever ran
 * out of its bounded waits, else (role<<24 | stage<<16 | iteration) of the first one.
 * Synchronises the device; resets the word.  For tests and diagnostics only. */
CU32_API int cu32_read_status(int* status);

/* Reads and clears the clock accumulator the "clock" tuning key switches on: out3 = {SM cycles, nanoseconds,
 * launches} summed over the contraction launches since the last read.  cycles / nanoseconds is the SM clock in
 * GHz the kernels actually ran at.  Synchronises the device.  No counterpart in the reference. */
CU32_API int cu32_read_clock(unsigned long long* out3);

/* Self-test of the bounded waits (no counterpart in the reference): launches one warp that waits, for at most
 * limit_cycles SM clock cycles (1 .. 100 000 000), on a barrier nobody arrives at.  The wait runs out, the kernel
 * stores the give-up record (7<<24 | 1<<16 | 42) in the status word like the contraction kernel's roles do and
 * returns normally; cu32_read_status then reports it.  Lets a host check the time-out path without any fault. */
CU32_API int cu32_selftest_wait_giveup(int64_t stream, long long limit_cycles);

/* "dragon_cu32 <version> sm_100a" */
CU32_API const char* cu32_version(void);

#ifdef __cplusplus
}
#endif
#endif /* DRAGON_CU32_H */
