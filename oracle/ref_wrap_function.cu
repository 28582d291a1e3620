// Builds the two routines of the reference's Cuda_function project that follow the contractions
// on the hot path - linear_dual2D_row, the bias-row add of matMul_biased / conv3D_biased
// (CudaFloat32EngineBase.java:1630, :2472), and linear2D, the attention block's scale - into
// oracle/_ref/ for sm_100a.  This file contains
// no reference code, only #includes of the reference tree (given with -I) and an extern "C"
// forward so ctypes can call the C++ function.  Test infrastructure only.
#include "frame.cuh"  // the reference's own include list (A.cu:1-4), in order
#include "Cuda_function.cuh"
#include "JNITool.cuh"
#include "micro.cuh"
#include "type1_linear_dual2D_row.cuh"
#include "type1_linear2D.cuh"
#include "type1_div2D_field.cuh"

extern "C" {
// Called exactly as the reference's JNI function calls it (Cuda_function/A.cu:288-302).
int ref_gpu_linear_dual2D_row(long long stream, float* X1, float* X2, int row_lengthv, float alpha, float beta,
                              float gamma, float* Y, int lengthv, int width, int stride) {
  __linear_dual2D_row((cudaStream_t)(intptr_t)stream, X1, X2, row_lengthv, alpha, beta, gamma, Y, lengthv, width,
                      stride);
  return (int)cudaGetLastError();
}
// Y = alpha * X + beta (the engine's sdiv / linear; Cuda_function/A.cu calls __linear2D the same way).
int ref_gpu_linear2D(long long stream, float alpha, float* X, float beta, float* Y, int lengthv, int width, int stride) {
  __linear2D((cudaStream_t)(intptr_t)stream, alpha, X, beta, Y, lengthv, width, stride);
  return (int)cudaGetLastError();
}
// Y = (alpha1 * X1 + beta1) / (alpha2 * X2[row] + beta2) + gamma: the last kernel of the engine's softmax2D
// (CudaFloat32EngineBase.java:5768-5773 calls it with 1, 0, 1, 0, 0).
int ref_gpu_div2D_field(long long stream, float alpha1, float* X1, float beta1, float alpha2, float* X2, float beta2,
                        float gamma, int row_lengthv, float* Y, int lengthv, int width, int stride) {
  __div2D_field((cudaStream_t)(intptr_t)stream, alpha1, X1, beta1, alpha2, X2, beta2, gamma, row_lengthv, Y, lengthv,
                width, stride);
  return (int)cudaGetLastError();
}
}
