// Builds the reference's Cuda_matMul project into oracle/_ref/: its C++ dispatchers and
// SIMT kernels (compiled for sm_100a) and the CPU check loops of its test.cuh.  This file
// contains no reference code, only #includes of the reference tree (given with -I) and
// extern "C" forwards so ctypes can call the C++ functions.  Test infrastructure only.
#include "frame.cuh"  // the reference's own include list (A.cu:1-11), in order
#include "Cuda_matMul.cuh"
#include "JNITool.cuh"
#include "micro.cuh"
#include "SKbufsum.cuh"
#include "matMul.cuh"
#include "matMulT1.cuh"
#include "matMulT2.cuh"
using namespace std;
// test.cuh holds the CPU loops behind `#ifndef COMPILE`; its main() is renamed away.
#undef COMPILE
#define main int cu32_ref_matmul_test_main
#include "test.cuh"
#undef main

extern "C" {
// CPU check loops (C must be zeroed by the caller).
void ref_cpu_multiply(float* A, float* B, float* C, int N, int M, int K) { multiply(A, B, C, N, M, K); }
void ref_cpu_multiplyT1(float* A, float* B, float* C, int N, int M, int K) { multiplyT1(A, B, C, N, M, K); }
void ref_cpu_multiplyT2(float* A, float* B, float* C, int N, int M, int K) { multiplyT2(A, B, C, N, M, K); }
float ref_cpu_samePercent(float* a, float* b, int length) { return samePercent(a, b, length); }
// GPU dispatchers, called exactly as the reference's JNI functions call them (A.cu:41-178).
int ref_gpu_matMul(long long* streams, int length, float* A, float* B, float* C, int N, int M, int K) {
  int index = 0; matMul4x((jlong*)streams, index, length, A, B, C, N, M, K, M); return (int)cudaGetLastError();
}
int ref_gpu_matMulT1(long long* streams, int length, float* A, float* B, float* C, int N, int M, int K) {
  int index = 0; matMul4x_T1((jlong*)streams, index, length, A, B, C, N, M, K, N, M); return (int)cudaGetLastError();
}
int ref_gpu_matMulT2(long long* streams, int length, float* A, float* B, float* C, int N, int M, int K) {
  int index = 0; matMul4x_T2((jlong*)streams, index, length, A, B, C, N, M, K, M); return (int)cudaGetLastError();
}
int ref_gpu_matMulT1SK(long long* streams, int length, int GridZ, float* A, float* B, float* C, float* Cbuf,
                       int N, int M, int K) {
  int K_slice = SK_K_slice(K, GridZ); int index = 0;
  matMul4x_T1_SK((jlong*)streams, index, length, GridZ, A, B, C, Cbuf, N, M, K, K_slice, N, M);
  return (int)cudaGetLastError();
}
int ref_gpu_SKbuf_summary(long long stream, float* Cbuf, float* C, int part, int sizeC) {
  SKbuf_summary((cudaStream_t)(intptr_t)stream, Cbuf, C, part, sizeC); return (int)cudaGetLastError();
}
}
