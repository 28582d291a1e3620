// Builds the reference's Cuda_conv3D project into oracle/_ref/ (dispatchers, SIMT kernels
// for sm_100a, and the CPU loops of its test.cuh).  No reference code here, only #includes
// of the reference tree and extern "C" forwards.  Test infrastructure only.  The build takes
// about 25 minutes (the project is one 126k-line translation unit).
#include "frame.cuh"  // the reference's own include list (A.cu:1-8), in order
#include "Cuda_conv3D.cuh"
#include "JNITool.cuh"
#include "micro.cuh"
#include "texture.cuh"
#include "conv3D.cuh"
using namespace std;
#undef COMPILE
#define main int cu32_ref_conv_test_main
#include "test.cuh"
#undef main

extern "C" {
void ref_cpu_conv3D_naive(float* X, int IH, int IW, float* W, int FH, int FW, float* Y, int OH, int OW,
                          int N, int IC, int OC, int sh, int sw, int ph, int pw) {
  CONV_3D_NAIVE(X, IH, IW, W, FH, FW, Y, OH, OW, N, IC, OC, sh, sw, ph, pw);
}
void ref_cpu_conv3D_img2col(float* X, int IH, int IW, float* W, int FH, int FW, float* Y, int OH, int OW,
                            int N, int IC, int OC, int sh, int sw, int ph, int pw) {
  CONV_3D_img2col(X, IH, IW, W, FH, FW, Y, OH, OW, N, IC, OC, sh, sw, ph, pw);
}
int ref_gpu_kernel_remode(long long stream, float* W, float* CW, int FH, int FW, int OC, int IC) {
  __kernel_remode((cudaStream_t)(intptr_t)stream, W, CW, FH, FW, OC, IC); return (int)cudaGetLastError();
}
int ref_gpu_conv3D_GemmR(long long* streams, int length, float* X, int IH, int IW, float* W, float* CW,
                         int FH, int FW, float* Y, int OH, int OW, int N, int IC, int OC, int sh, int sw,
                         int ph, int pw) {
  int index = 0;
  __conv3D_GemmR((jlong*)streams, index, length, X, IH, IW, W, CW, FH, FW, Y, OH, OW, N, IC, OC, sh, sw, ph, pw);
  return (int)cudaGetLastError();
}
}
