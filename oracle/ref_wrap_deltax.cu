// Builds the reference's Cuda_dconv3D_deltaX project into oracle/_ref/: the CPU check loop of its
// test.cuh for the stride-1 data gradient and its zero-padding stride-1 dispatcher (SIMT kernels
// for sm_100a) as a witness on the GPU.  This file contains no reference code, only #includes of
// the reference tree (given with -I) and extern "C" forwards so ctypes can call the C++ functions.
// Test infrastructure only.
#include "frame.cuh"  // the reference's own include list (A.cu:1-6), in order
#include "JNITool.cuh"
#include "Cuda_dconv3D_deltaX.cuh"
#include "micro.cuh"
#include "texture.cuh"
#include "dconv3D_dX.cuh"
using namespace std;
// test.cuh holds the CPU loops behind `#ifndef COMPILE`; its main() is renamed away.
#undef COMPILE
#define main int cu32_ref_deltax_test_main
#include "test.cuh"
#undef main

extern "C" {
// CPU check loop (Cuda_dconv3D_deltaX/test.cuh:154-196); sh, sw are accepted by the reference and unused.
void ref_cpu_deconv3D_deltaX_img2col_s1(float* deltaY, int OH, int OW, float* W, int FH, int FW, float* deltaX,
                                        int IH, int IW, int N, int IC, int OC, int ph, int pw) {
  deconv3D_deltaX_img2col_s1(deltaY, OH, OW, W, FH, FW, deltaX, IH, IW, N, IC, OC, 1, 1, ph, pw);
}
// Any-stride CPU check loop (test.cuh:109-152).
void ref_cpu_deconv3D_deltaX_img2col(float* deltaY, int OH, int OW, float* W, int FH, int FW, float* deltaX, int IH,
                                     int IW, int N, int IC, int OC, int sh, int sw, int ph, int pw) {
  deconv3D_deltaX_img2col(deltaY, OH, OW, W, FH, FW, deltaX, IH, IW, N, IC, OC, sh, sw, ph, pw);
}
// Filter workspace kernels (A.cu:280-306).
int ref_gpu_ks_remode(long long stream, float* W, int FH, int FW, float* CW, int CFH, int CFW, int OC, int IC, int sh,
                      int sw) {
  __ks_remode((cudaStream_t)(intptr_t)stream, W, FH, FW, CW, CFH, CFW, OC, IC, sh, sw);
  return (int)cudaGetLastError();
}
int ref_gpu_ks_remodev2(long long stream, float* W, int FH, int FW, float* CW, int CFH, int CFW, int OC, int IC, int sh,
                        int sw) {
  __ks_remodev2((cudaStream_t)(intptr_t)stream, W, FH, FW, CW, CFH, CFW, OC, IC, sh, sw);
  return (int)cudaGetLastError();
}
// The scatter-add form for any stride, as its JNI function runs it (A.cu:731-764): zero deltaX, then accumulate.
int ref_gpu_dconv3D_deltaX_crossAdd(long long* streams, int length, float* deltaY, int OH, int OW, float* W, int FH,
                                    int FW, float* deltaX, int IH, int IW, int N, int IC, int OC, int sh, int sw,
                                    int ph, int pw) {
  cudaStream_t s0 = (cudaStream_t)(intptr_t)streams[0];
  cudaMemsetAsync(deltaX, 0, sizeof(float) * (size_t)N * IH * IW * IC, s0);
  cudaStreamSynchronize(s0);
  int index = 0;
  __dconv3D_deltaX_CrossAdd((jlong*)streams, index, length, deltaY, OH, OW, W, FH, FW, deltaX, IH, IW, N, IC, OC, sh,
                            sw, ph, pw);
  return (int)cudaGetLastError();
}
// GPU dispatcher, called exactly as the reference's JNI function calls it (A.cu:21-42).
int ref_gpu_dconv3D_deltaX_s1(long long* streams, int length, float* deltaY, int OH, int OW, float* W, int FH,
                              int FW, float* deltaX, int IH, int IW, int N, int IC, int OC, int ph, int pw) {
  int index = 0;
  __dconv3D_deltaX_ZeroPadding_s1((jlong*)streams, index, length, deltaY, OH, OW, W, FH, FW, deltaX, IH, IW, N, IC, OC,
                                  ph, pw);
  return (int)cudaGetLastError();
}
}
