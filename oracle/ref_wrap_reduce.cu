// Builds the reference's row softmax (Cuda_reduce: row_max and row_softmax with the field stages they fall back
// on for long rows) into oracle/_ref/ for sm_100a: the kernels the Java engine's softmax2D runs before
// div2D_field (CudaFloat32EngineBase.java:5738-5775).  This file contains no reference code, only #includes of
// the reference tree (given with -I) and extern "C" forwards so ctypes can call the C++ functions.
// Test infrastructure only.
#include "frame.cuh"  // the reference's own include list (A.cu:1-4), in order
#include "Cuda_reduce.cuh"
#include "JNITool.cuh"
#include "micro.cuh"
#include "field_linear.cuh"
#include "field_max.cuh"
#include "row_max.cuh"
#include "row_softmax.cuh"

extern "C" {
// Called as the reference's JNI functions call them (Cuda_reduce/A.cu:818-927), partNum = 1 as the Java side passes.
// V needs row_nextM(M) * ((N + 3) & ~3) floats, maxX and the returned sums N floats.
int ref_gpu_row_max(long long stream, float* X, int N, int M, float* V, float* Y, int width, int stride) {
  __row_max((cudaStream_t)(intptr_t)stream, X, N, M, V, Y, width, stride, 1);
  return (int)cudaGetLastError();
}
int ref_gpu_row_softmax(long long stream, float* X, float* maxX, float* expX, int N, int M, float* V, int width,
                        int stride) {
  __row_softmax((cudaStream_t)(intptr_t)stream, X, maxX, expX, N, M, V, width, stride, 1);
  return (int)cudaGetLastError();
}
}
