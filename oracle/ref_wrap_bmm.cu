// Builds the reference's Cuda_batchMatMul project into oracle/_ref/ (dispatchers, SIMT
// kernels for sm_100a, and the CPU loops of its test.cuh).  No reference code here, only
// #includes of the reference tree and extern "C" forwards.  Test infrastructure only.
#include "frame.cuh"  // the reference's own include list (A.cu:1-12), in order
#include "Cuda_batchMatMul.cuh"
#include "JNITool.cuh"
#include "micro.cuh"
#include "texture.cuh"
#include "batchMatMul.cuh"
#include "batchMatMulT1.cuh"
#include "batchMatMulT2.cuh"
using namespace std;
#undef COMPILE
#define main int cu32_ref_bmm_test_main
#include "test.cuh"
#undef main

extern "C" {
void ref_cpu_bmm(float* A, float* B, float* C, int Batch, int N, int CM, int BK, int AK) { bmm(A, B, C, Batch, N, CM, BK, AK); }
void ref_cpu_bmmT1(float* A, float* B, float* C, int Batch, int CN, int AN, int CM, int K) { bmmT1(A, B, C, Batch, CN, AN, CM, K); }
void ref_cpu_bmmT2(float* A, float* B, float* C, int Batch, int N, int CM, int BM, int K) { bmmT2(A, B, C, Batch, N, CM, BM, K); }
int ref_gpu_batchMatMul(long long* streams, int length, float* A, float* B, float* C, int Batch, int N, int M, int BK, int AK) {
  int index = 0; __batch_matMul(1, 1, (jlong*)streams, index, length, A, B, C, Batch, N, M, BK, AK); return (int)cudaGetLastError();
}
int ref_gpu_batchMatMulT1(long long* streams, int length, float* A, float* B, float* C, int Batch, int CN, int AN, int M, int K) {
  int index = 0; __batch_matMulT1(1, 1, (jlong*)streams, index, length, A, B, C, Batch, CN, AN, M, K); return (int)cudaGetLastError();
}
int ref_gpu_batchMatMulT2(long long* streams, int length, float* A, float* B, float* C, int Batch, int N, int CM, int BM, int K) {
  int index = 0; __batch_matMulT2(1, 1, (jlong*)streams, index, length, A, B, C, Batch, N, CM, BM, K); return (int)cudaGetLastError();
}
}
