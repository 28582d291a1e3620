// JNI exports: the Java_z_dragon_engine_cuda_impl_math_Cuda_1* symbols that the
// Java classes Cuda_matMul, Cuda_batchMatMul and Cuda_conv3D bind to, as thin
// wrappers over the C ABI in include/dragon_cu32.h.
//
// Behaviour mirrors the reference wrappers (engine-cuda-base/Cuda_matMul/Cuda_matMul/A.cu,
// Cuda_batchMatMul/.../A.cu, Cuda_conv3D/.../A.cu and JNITool.cuh): copy up to 10 stream
// handles out of the long[] with GetLongArrayRegion, cast the jlong addresses to device
// pointers, run the operation, and on a non-zero result construct
// z.dragon.engine.cuda.impl.CudaException(int) and Throw it, returning normally.
#ifdef DRAGON_USE_SYSTEM_JNI
#include <jni.h>
static inline jclass jni_FindClass(JNIEnv* env, const char* n) { return env->FindClass(n); }
static inline jint jni_Throw(JNIEnv* env, jthrowable o) { return env->Throw(o); }
static inline jobject jni_NewObjectA(JNIEnv* env, jclass c, jmethodID m, const jvalue* a) { return env->NewObjectA(c, m, a); }
static inline jmethodID jni_GetMethodID(JNIEnv* env, jclass c, const char* n, const char* s) { return env->GetMethodID(c, n, s); }
static inline void jni_GetLongArrayRegion(JNIEnv* env, jlongArray a, jint s, jint l, jlong* b) { env->GetLongArrayRegion(a, s, l, b); }
#else
#include "jni_min.h"
#endif
#include "../../include/dragon_cu32.h"

namespace {

void throw_cuda_exception(JNIEnv* env, int code) {
  jclass cls = jni_FindClass(env, "z/dragon/engine/cuda/impl/CudaException");
  if (!cls) return;  // FindClass has already raised NoClassDefFoundError
  jmethodID ctor = jni_GetMethodID(env, cls, "<init>", "(I)V");
  if (!ctor) return;
  jvalue arg;
  arg.i = code;
  jobject ex = jni_NewObjectA(env, cls, ctor, &arg);
  if (ex) jni_Throw(env, static_cast<jthrowable>(ex));
}

struct Streams {
  int64_t h[10];
  int n;
  Streams(JNIEnv* env, jlongArray arr, jint length) : n(length) {
    for (int i = 0; i < 10; ++i) h[i] = 0;
    if (length >= 1 && length <= 10) {
      jlong tmp[10];
      jni_GetLongArrayRegion(env, arr, 0, length, tmp);
      for (int i = 0; i < length; ++i) h[i] = tmp[i];
    }
  }
};

inline const float* cptr(jlong a) { return reinterpret_cast<const float*>(static_cast<intptr_t>(a)); }
inline float* mptr(jlong a) { return reinterpret_cast<float*>(static_cast<intptr_t>(a)); }
inline void done(JNIEnv* env, int rc) { if (rc != 0) throw_cuda_exception(env, rc); }
// The boolean natives tell Java whether they handled the shape: the engine tries them in an else-if chain
// (`algo == X && native(...)`) and falls through to the general native on false.  A refused shape or argument
// (negative code) is therefore a plain false with no exception pending, as in the reference; only a CUDA
// runtime error (positive code) is thrown.
inline jboolean handled(JNIEnv* env, int rc) {
  if (rc > 0) throw_cuda_exception(env, rc);
  return rc == 0 ? 1 : 0;
}

}  // namespace

#define JNAME(cls, method) Java_z_dragon_engine_cuda_impl_math_Cuda_1##cls##_##method

extern "C" {

// ---------------------------------------------------------------- Cuda_matMul
JNIEXPORT void JNICALL JNAME(matMul, SKbuf_1summary)(JNIEnv* env, jclass, jlong stream, jlong dCbuf, jlong dC,
                                                     jint part, jint sizeC) {
  done(env, cu32_SKbuf_summary(stream, cptr(dCbuf), mptr(dC), part, sizeC));
}
#define MATMUL_PLAIN(jname, cname)                                                                  \
  JNIEXPORT void JNICALL JNAME(matMul, jname)(JNIEnv* env, jclass, jlongArray streams, jint length, \
                                              jlong dA, jlong dB, jlong dC, jint N, jint M, jint K) { \
    Streams s(env, streams, length);                                                                \
    done(env, cname(s.h, s.n, cptr(dA), cptr(dB), mptr(dC), N, M, K));                              \
  }
#define MATMUL_SK(jname, cname)                                                                     \
  JNIEXPORT void JNICALL JNAME(matMul, jname)(JNIEnv* env, jclass, jlongArray streams, jint length, \
                                              jint GridZ, jlong dA, jlong dB, jlong dC, jlong dCbuf, \
                                              jint N, jint M, jint K) {                             \
    Streams s(env, streams, length);                                                                \
    done(env, cname(s.h, s.n, GridZ, cptr(dA), cptr(dB), mptr(dC), mptr(dCbuf), N, M, K));          \
  }
MATMUL_PLAIN(matMul, cu32_matMul)
MATMUL_PLAIN(matMulT1, cu32_matMulT1)
MATMUL_PLAIN(matMulT2, cu32_matMulT2)
MATMUL_PLAIN(matMul_1mma, cu32_matMul_mma)
MATMUL_PLAIN(matMulT1_1mma, cu32_matMulT1_mma)
MATMUL_PLAIN(matMulT2_1mma, cu32_matMulT2_mma)
MATMUL_SK(matMulSK, cu32_matMulSK)
MATMUL_SK(matMulT1SK, cu32_matMulT1SK)
MATMUL_SK(matMulT2SK, cu32_matMulT2SK)

// Reads and clears the device status word (0 = every bounded wait of the kernels completed; otherwise the
// first give-up record, see cu32_read_status).  Not in the reference's Java class: a maintainer declares
// `public static native int kernelStatus();` in Cuda_matMul and calls it where the engine already
// synchronises (its Syncer), so that a protocol time-out surfaces as an error instead of a wrong tensor.
JNIEXPORT jint JNICALL JNAME(matMul, kernelStatus)(JNIEnv* env, jclass) {
  int status = 0;
  const int rc = cu32_read_status(&status);
  if (rc != 0) { throw_cuda_exception(env, rc); return -1; }
  return status;
}

// ---------------------------------------------------------------- Cuda_batchMatMul
#define BMM_PLAIN(jname, cname)                                                                          \
  JNIEXPORT void JNICALL JNAME(batchMatMul, jname)(JNIEnv* env, jclass, jlongArray streams, jint length, \
                                                   jlong dA, jlong dB, jlong dC, jint Batch, jint d0,    \
                                                   jint d1, jint d2, jint d3) {                          \
    Streams s(env, streams, length);                                                                     \
    done(env, cname(s.h, s.n, cptr(dA), cptr(dB), mptr(dC), Batch, d0, d1, d2, d3));                     \
  }
#define BMM_TEX_FLAG(jname, cname)                                                                       \
  JNIEXPORT void JNICALL JNAME(batchMatMul, jname)(JNIEnv* env, jclass, jboolean useTexture,             \
                                                   jlongArray streams, jint length, jlong dA, jlong dB,  \
                                                   jlong dC, jint Batch, jint d0, jint d1, jint d2,      \
                                                   jint d3) {                                            \
    Streams s(env, streams, length);                                                                     \
    done(env, cname(useTexture ? 1 : 0, s.h, s.n, cptr(dA), cptr(dB), mptr(dC), Batch, d0, d1, d2, d3)); \
  }
BMM_PLAIN(batchMatMul, cu32_batchMatMul)
BMM_PLAIN(batchMatMul_1texture, cu32_batchMatMul_texture)
BMM_PLAIN(batchMatMulT1, cu32_batchMatMulT1)
BMM_PLAIN(batchMatMulT2, cu32_batchMatMulT2)
BMM_PLAIN(batchMatMulT2_1texture, cu32_batchMatMulT2_texture)
BMM_PLAIN(batchMatMulT1_1mma, cu32_batchMatMulT1_mma)
BMM_TEX_FLAG(batchMatMul_1mma, cu32_batchMatMul_mma)
BMM_TEX_FLAG(batchMatMulT2_1mma, cu32_batchMatMulT2_mma)

// ---------------------------------------------------------------- Cuda_conv3D
JNIEXPORT void JNICALL JNAME(conv3D, kernel_1remode)(JNIEnv* env, jclass, jlong stream, jlong dW, jlong dCW,
                                                     jint FH, jint FW, jint OC, jint IC) {
  done(env, cu32_kernel_remode(stream, cptr(dW), mptr(dCW), FH, FW, OC, IC));
}
JNIEXPORT void JNICALL JNAME(conv3D, conv3D)(JNIEnv* env, jclass, jlongArray streams, jint length, jlong dX,
                                             jint IH, jint IW, jlong dW, jint FH, jint FW, jlong dY, jint OH,
                                             jint OW, jint N, jint IC, jint OC, jint sh, jint sw, jint ph,
                                             jint pw) {
  Streams s(env, streams, length);
  done(env, cu32_conv3D(s.h, s.n, cptr(dX), IH, IW, cptr(dW), FH, FW, mptr(dY), OH, OW, N, IC, OC, sh, sw, ph, pw));
}
JNIEXPORT void JNICALL JNAME(conv3D, conv3D_1texture)(JNIEnv* env, jclass, jlongArray streams, jint length,
                                                      jlong dX, jint IH, jint IW, jlong dW, jint FH, jint FW,
                                                      jlong dY, jint OH, jint OW, jint N, jint IC, jint OC,
                                                      jint sh, jint sw, jint ph, jint pw) {
  Streams s(env, streams, length);
  done(env, cu32_conv3D_texture(s.h, s.n, cptr(dX), IH, IW, cptr(dW), FH, FW, mptr(dY), OH, OW, N, IC, OC, sh, sw, ph, pw));
}
JNIEXPORT void JNICALL JNAME(conv3D, conv3D_1np)(JNIEnv* env, jclass, jlongArray streams, jint length,
                                                 jlong dX, jint IH, jint IW, jlong dW, jint FH, jint FW,
                                                 jlong dY, jint OH, jint OW, jint N, jint IC, jint OC,
                                                 jint sh, jint sw) {
  Streams s(env, streams, length);
  done(env, cu32_conv3D_np(s.h, s.n, cptr(dX), IH, IW, cptr(dW), FH, FW, mptr(dY), OH, OW, N, IC, OC, sh, sw));
}
JNIEXPORT void JNICALL JNAME(conv3D, conv3D_1W1)(JNIEnv* env, jclass, jlongArray streams, jint length,
                                                 jlong dX, jint IH, jint IW, jlong dW, jlong dY, jint N,
                                                 jint IC, jint OC) {
  Streams s(env, streams, length);
  done(env, cu32_conv3D_W1(s.h, s.n, cptr(dX), IH, IW, cptr(dW), mptr(dY), N, IC, OC));
}
#define CONV_GEMMR(jname, cname)                                                                          \
  JNIEXPORT void JNICALL JNAME(conv3D, jname)(JNIEnv* env, jclass, jlongArray streams, jint length,       \
                                              jlong dX, jint IH, jint IW, jlong dW, jlong dCW, jint FH,   \
                                              jint FW, jlong dY, jint OH, jint OW, jint N, jint IC,       \
                                              jint OC, jint sh, jint sw, jint ph, jint pw) {              \
    Streams s(env, streams, length);                                                                      \
    done(env, cname(s.h, s.n, cptr(dX), IH, IW, cptr(dW), cptr(dCW), FH, FW, mptr(dY), OH, OW, N, IC, OC, \
                    sh, sw, ph, pw));                                                                     \
  }
#define CONV_GEMMR_SGM(jname, cname)                                                                      \
  JNIEXPORT void JNICALL JNAME(conv3D, jname)(JNIEnv* env, jclass, jlongArray streams, jint length,       \
                                              jlong dX, jint IH, jint IW, jlong dW, jlong dCW, jint FH,   \
                                              jint FW, jlong dY, jint OH, jint OW, jint N, jint IC,       \
                                              jint OC, jint sh, jint sw, jint ph, jint pw,                \
                                              jint GM_slice) {                                            \
    Streams s(env, streams, length);                                                                      \
    done(env, cname(s.h, s.n, cptr(dX), IH, IW, cptr(dW), cptr(dCW), FH, FW, mptr(dY), OH, OW, N, IC, OC, \
                    sh, sw, ph, pw, GM_slice));                                                           \
  }
CONV_GEMMR(conv3D_1GemmR, cu32_conv3D_GemmR)
CONV_GEMMR(conv3D_1GemmR_1texture, cu32_conv3D_GemmR_texture)
CONV_GEMMR_SGM(conv3D_1GemmR_1SGM, cu32_conv3D_GemmR_SGM)
CONV_GEMMR_SGM(conv3D_1GemmR_1texture_1SGM, cu32_conv3D_GemmR_texture_SGM)
// ---- Cuda_dconv3D_deltaX, the stride-1 natives (reference: Cuda_dconv3D_deltaX/A.cu:21-277, :837-1040)
#define JNAME_DX(method) Java_z_dragon_engine_cuda_impl_math_Cuda_1dconv3D_1deltaX_##method
#define DX_S1(jname, cname)                                                                               \
  JNIEXPORT void JNICALL JNAME_DX(jname)(JNIEnv* env, jclass, jlongArray streams, jint length, jlong dDY,  \
                                         jint OH, jint OW, jlong dW, jint FH, jint FW, jlong dDX, jint IH, \
                                         jint IW, jint N, jint IC, jint OC, jint ph, jint pw) {            \
    Streams s(env, streams, length);                                                                       \
    done(env, cname(s.h, s.n, cptr(dDY), OH, OW, cptr(dW), FH, FW, mptr(dDX), IH, IW, N, IC, OC, ph, pw)); \
  }
#define DX_S1_SGM(jname, cname)                                                                            \
  JNIEXPORT void JNICALL JNAME_DX(jname)(JNIEnv* env, jclass, jlongArray streams, jint length, jlong dDY,  \
                                         jint OH, jint OW, jlong dW, jint FH, jint FW, jlong dDX, jint IH, \
                                         jint IW, jint N, jint IC, jint OC, jint ph, jint pw,              \
                                         jint GM_slice) {                                                  \
    Streams s(env, streams, length);                                                                       \
    done(env, cname(s.h, s.n, cptr(dDY), OH, OW, cptr(dW), FH, FW, mptr(dDX), IH, IW, N, IC, OC, ph, pw,   \
                    GM_slice));                                                                            \
  }
DX_S1(dconv3D_1deltaX_1s1, cu32_dconv3D_deltaX_s1)
DX_S1(dconv3D_1deltaX_1s1_1texture, cu32_dconv3D_deltaX_s1_texture)
DX_S1_SGM(dconv3D_1deltaX_1s1_1SGM, cu32_dconv3D_deltaX_s1_SGM)
DX_S1_SGM(dconv3D_1deltaX_1s1_1texture_1SGM, cu32_dconv3D_deltaX_s1_texture_SGM)
JNIEXPORT void JNICALL JNAME_DX(dconv3D_1deltaX_1V2_1s1)(JNIEnv* env, jclass, jboolean useTexture,
                                                         jlongArray streams, jint length, jlong dDY, jint OH,
                                                         jint OW, jlong dW, jint FH, jint FW, jlong dDX, jint IH,
                                                         jint IW, jint N, jint IC, jint OC, jint ph, jint pw) {
  Streams s(env, streams, length);
  done(env, cu32_dconv3D_deltaX_V2_s1(useTexture ? 1 : 0, s.h, s.n, cptr(dDY), OH, OW, cptr(dW), FH, FW, mptr(dDX), IH,
                                      IW, N, IC, OC, ph, pw));
}
JNIEXPORT void JNICALL JNAME_DX(dconv3D_1deltaX_1W1)(JNIEnv* env, jclass, jlongArray streams, jint length,
                                                     jlong dDY, jlong dW, jlong dDX, jint IH, jint IW, jint N,
                                                     jint IC, jint OC) {
  Streams s(env, streams, length);
  done(env, cu32_dconv3D_deltaX_W1(s.h, s.n, cptr(dDY), cptr(dW), mptr(dDX), IH, IW, N, IC, OC));
}
JNIEXPORT void JNICALL JNAME_DX(dconv3D_1deltaX_1W1_1SGM)(JNIEnv* env, jclass, jlongArray streams, jint length,
                                                          jlong dDY, jlong dW, jlong dDX, jint IH, jint IW,
                                                          jint N, jint IC, jint OC, jint GM_slice) {
  Streams s(env, streams, length);
  done(env, cu32_dconv3D_deltaX_W1_SGM(s.h, s.n, cptr(dDY), cptr(dW), mptr(dDX), IH, IW, N, IC, OC, GM_slice));
}
#define DX_WINOGRAD(jname, cname)                                                                          \
  JNIEXPORT jboolean JNICALL JNAME_DX(jname)(JNIEnv* env, jclass, jboolean useTexture, jlongArray streams, \
                                             jint length, jlong dDY, jint OH, jint OW, jlong dW, jint FH,  \
                                             jint FW, jlong dDX, jint IH, jint IW, jint N, jint IC,        \
                                             jint OC, jint ph, jint pw) {                                  \
    Streams s(env, streams, length);                                                                       \
    const int rc = cname(useTexture ? 1 : 0, s.h, s.n, cptr(dDY), OH, OW, cptr(dW), FH, FW, mptr(dDX), IH, \
                         IW, N, IC, OC, ph, pw);                                                           \
    return handled(env, rc);                                                                                         \
                                                                                    \
  }
#define DX_WINOGRAD_SGM(jname, cname)                                                                      \
  JNIEXPORT jboolean JNICALL JNAME_DX(jname)(JNIEnv* env, jclass, jboolean useTexture, jlongArray streams, \
                                             jint length, jlong dDY, jint OH, jint OW, jlong dW, jint FH,  \
                                             jint FW, jlong dDX, jint IH, jint IW, jint N, jint IC,        \
                                             jint OC, jint ph, jint pw, jint GM_slice) {                   \
    Streams s(env, streams, length);                                                                       \
    const int rc = cname(useTexture ? 1 : 0, s.h, s.n, cptr(dDY), OH, OW, cptr(dW), FH, FW, mptr(dDX), IH, \
                         IW, N, IC, OC, ph, pw, GM_slice);                                                 \
    return handled(env, rc);                                                                                         \
                                                                                    \
  }
DX_WINOGRAD(Im2col_1Winograd_1s8_1texture, cu32_dconv3D_deltaX_Im2col_Winograd_s8_texture)
DX_WINOGRAD_SGM(Im2col_1Winograd_1s8_1texture_1SGM, cu32_dconv3D_deltaX_Im2col_Winograd_s8_texture_SGM)
DX_WINOGRAD(Im2col_1Winograd_1s16_1texture, cu32_dconv3D_deltaX_Im2col_Winograd_s16_texture)
DX_WINOGRAD_SGM(Im2col_1Winograd_1s16_1texture_1SGM, cu32_dconv3D_deltaX_Im2col_Winograd_s16_texture_SGM)

// ---- Cuda_dconv3D_deltaX for strides > 1 (reference: Cuda_dconv3D_deltaX/A.cu:280-834)
JNIEXPORT void JNICALL JNAME_DX(ks_1remode)(JNIEnv* env, jclass, jlong stream, jlong dW, jint FH, jint FW, jlong dCW,
                                            jint CFH, jint CFW, jint OC, jint IC, jint sh, jint sw) {
  done(env, cu32_ks_remode(stream, cptr(dW), FH, FW, mptr(dCW), CFH, CFW, OC, IC, sh, sw));
}
JNIEXPORT void JNICALL JNAME_DX(ks_1remodev2)(JNIEnv* env, jclass, jlong stream, jlong dW, jint FH, jint FW,
                                              jlong dCW, jint CFH, jint CFW, jint OC, jint IC, jint sh, jint sw) {
  done(env, cu32_ks_remodev2(stream, cptr(dW), FH, FW, mptr(dCW), CFH, CFW, OC, IC, sh, sw));
}
#define DX_HEAD jlongArray streams, jint length, jlong dDY, jint OH, jint OW, jlong dF, jint FH, jint FW, jlong dDX, \
                jint IH, jint IW, jint N, jint IC, jint OC
#define DX_PASS s.h, s.n, cptr(dDY), OH, OW, cptr(dF), FH, FW, mptr(dDX), IH, IW, N, IC, OC
#define DX_KS(jname, cname)                                                                                      \
  JNIEXPORT void JNICALL JNAME_DX(jname)(JNIEnv* env, jclass, DX_HEAD, jint sh, jint sw, jint ph, jint pw) {     \
    Streams s(env, streams, length);                                                                             \
    done(env, cname(DX_PASS, sh, sw, ph, pw));                                                                   \
  }
#define DX_KS_SGM(jname, cname)                                                                                  \
  JNIEXPORT void JNICALL JNAME_DX(jname)(JNIEnv* env, jclass, DX_HEAD, jint sh, jint sw, jint ph, jint pw,       \
                                         jint GM_slice) {                                                        \
    Streams s(env, streams, length);                                                                             \
    done(env, cname(DX_PASS, sh, sw, ph, pw, GM_slice));                                                         \
  }
#define DX_KS2(jname, cname)                                                                                     \
  JNIEXPORT void JNICALL JNAME_DX(jname)(JNIEnv* env, jclass, DX_HEAD, jint ph, jint pw) {                       \
    Streams s(env, streams, length);                                                                             \
    done(env, cname(DX_PASS, ph, pw));                                                                           \
  }
#define DX_KS2_SGM(jname, cname)                                                                                 \
  JNIEXPORT void JNICALL JNAME_DX(jname)(JNIEnv* env, jclass, DX_HEAD, jint ph, jint pw, jint GM_slice) {        \
    Streams s(env, streams, length);                                                                             \
    done(env, cname(DX_PASS, ph, pw, GM_slice));                                                                 \
  }
DX_KS(dconv3D_1deltaX_1kernelSplit, cu32_dconv3D_deltaX_kernelSplit)
DX_KS_SGM(dconv3D_1deltaX_1kernelSplit_1SGM, cu32_dconv3D_deltaX_kernelSplit_SGM)
DX_KS(dconv3D_1deltaX_1ksImsR, cu32_dconv3D_deltaX_ksImsR)
DX_KS_SGM(dconv3D_1deltaX_1ksImsR_1SGM, cu32_dconv3D_deltaX_ksImsR_SGM)
DX_KS(dconv3D_1deltaX_1ksImsR_1texture, cu32_dconv3D_deltaX_ksImsR_texture)
DX_KS_SGM(dconv3D_1deltaX_1ksImsR_1texture_1SGM, cu32_dconv3D_deltaX_ksImsR_texture_SGM)
DX_KS2(dconv3D_1deltaX_1ksIms2R, cu32_dconv3D_deltaX_ksIms2R)
DX_KS2_SGM(dconv3D_1deltaX_1ksIms2R_1SGM, cu32_dconv3D_deltaX_ksIms2R_SGM)
DX_KS2(dconv3D_1deltaX_1ksIms2R_1texture, cu32_dconv3D_deltaX_ksIms2R_texture)
DX_KS2_SGM(dconv3D_1deltaX_1ksIms2R_1texture_1SGM, cu32_dconv3D_deltaX_ksIms2R_texture_SGM)
DX_KS(dconv3D_1deltaX_1crossAdd, cu32_dconv3D_deltaX_crossAdd)
DX_KS_SGM(dconv3D_1deltaX_1crossAdd_1SGM, cu32_dconv3D_deltaX_crossAdd_SGM)
JNIEXPORT void JNICALL JNAME_DX(dconv3D_1deltaX_1ksV2_1Ims2R)(JNIEnv* env, jclass, jboolean useTexture, DX_HEAD,
                                                              jint ph, jint pw) {
  Streams s(env, streams, length);
  done(env, cu32_dconv3D_deltaX_ksV2_Ims2R(useTexture ? 1 : 0, DX_PASS, ph, pw));
}

// Data gradient / transposed convolution + bias row in one pass (arguments of the unbiased native, then the bias
// address and the true row width).
JNIEXPORT void JNICALL JNAME_DX(dconv3D_1deltaX_1s1_1biased)(JNIEnv* env, jclass, DX_HEAD, jint ph, jint pw,
                                                             jlong dBias, jint width) {
  Streams s(env, streams, length);
  done(env, cu32_dconv3D_deltaX_s1_biased(DX_PASS, ph, pw, cptr(dBias), width));
}
JNIEXPORT void JNICALL JNAME_DX(dconv3D_1deltaX_1ksImsR_1biased)(JNIEnv* env, jclass, DX_HEAD, jint sh, jint sw, jint ph,
                                                                 jint pw, jlong dBias, jint width) {
  Streams s(env, streams, length);
  done(env, cu32_dconv3D_deltaX_ksImsR_biased(DX_PASS, sh, sw, ph, pw, cptr(dBias), width));
}

// Batched contraction + scale in one pass; a Java class would declare them as
//   public static native void batchMatMul[T1|T2]_scaled(long[] streamArray, int length, long dA, long dB, long dC,
//                                                       int Batch, int d0, int d1, int d2, int d3, float alpha);
#define BMM_SCALED(jname, cname)                                                                                   \
  JNIEXPORT void JNICALL JNAME(batchMatMul, jname)(JNIEnv* env, jclass, jlongArray streams, jint length, jlong dA,  \
                                                   jlong dB, jlong dC, jint Batch, jint d0, jint d1, jint d2,       \
                                                   jint d3, jfloat alpha) {                                        \
    Streams s(env, streams, length);                                                                               \
    done(env, cname(s.h, s.n, cptr(dA), cptr(dB), mptr(dC), Batch, d0, d1, d2, d3, alpha));                        \
  }
BMM_SCALED(batchMatMul_1scaled, cu32_batchMatMul_scaled)
BMM_SCALED(batchMatMulT1_1scaled, cu32_batchMatMulT1_scaled)
BMM_SCALED(batchMatMulT2_1scaled, cu32_batchMatMulT2_scaled)
BMM_SCALED(batchMatMulT2_1softmax, cu32_batchMatMulT2_softmax)

// ---- Cuda_dconv3D_deltaW (Java declarations: Cuda_dconv3D_deltaW.java:288-640)
#define JNAME_DW(method) Java_z_dragon_engine_cuda_impl_math_Cuda_1dconv3D_1deltaW_##method
JNIEXPORT void JNICALL JNAME_DW(dconv3D_1deltaW)(JNIEnv* env, jclass, jlongArray streams, jint length, jlong dX, jint IH,
                                                 jint IW, jlong dDY, jint OH, jint OW, jlong dDW, jint FH, jint FW,
                                                 jint N, jint IC, jint OC, jint sh, jint sw, jint ph, jint pw) {
  Streams s(env, streams, length);
  done(env, cu32_dconv3D_deltaW(s.h, s.n, cptr(dX), IH, IW, cptr(dDY), OH, OW, mptr(dDW), FH, FW, N, IC, OC, sh, sw, ph, pw));
}
JNIEXPORT void JNICALL JNAME_DW(dconv3D_1deltaW_1W1)(JNIEnv* env, jclass, jlongArray streams, jint length, jlong dX,
                                                     jint IH, jint IW, jlong dDY, jlong dDW, jint N, jint IC, jint OC) {
  Streams s(env, streams, length);
  done(env, cu32_dconv3D_deltaW_W1(s.h, s.n, cptr(dX), IH, IW, cptr(dDY), mptr(dDW), N, IC, OC));
}
JNIEXPORT void JNICALL JNAME_DW(buf_1summary)(JNIEnv* env, jclass, jlong stream, jlong dBuf, jlong dDW, jint part,
                                              jint sizeW) {
  done(env, cu32_dconv3D_deltaW_buf_summary(stream, cptr(dBuf), mptr(dDW), part, sizeW));
}
#define DW_SK(jname, cname)                                                                                       \
  JNIEXPORT void JNICALL JNAME_DW(jname)(JNIEnv* env, jclass, jlongArray streams, jint length, jint GridZ, jlong dX, \
                                         jint IH, jint IW, jlong dDY, jint OH, jint OW, jlong dDW, jlong dBuf,      \
                                         jint FH, jint FW, jint N, jint IC, jint OC, jint sh, jint sw, jint ph,     \
                                         jint pw) {                                                                 \
    Streams s(env, streams, length);                                                                                \
    done(env, cname(s.h, s.n, GridZ, cptr(dX), IH, IW, cptr(dDY), OH, OW, mptr(dDW), mptr(dBuf), FH, FW, N, IC, OC, \
                    sh, sw, ph, pw));                                                                               \
  }
DW_SK(dconv3D_1deltaW_1GemmSK, cu32_dconv3D_deltaW_GemmSK)
DW_SK(dconv3D_1deltaW_1GemmV2SK, cu32_dconv3D_deltaW_GemmV2SK)
JNIEXPORT void JNICALL JNAME_DW(dconv3D_1deltaW_1GemmSK_1W1)(JNIEnv* env, jclass, jlongArray streams, jint length,
                                                             jint GridZ, jlong dX, jint IH, jint IW, jlong dDY,
                                                             jlong dDW, jlong dBuf, jint N, jint IC, jint OC) {
  Streams s(env, streams, length);
  done(env, cu32_dconv3D_deltaW_GemmSK_W1(s.h, s.n, GridZ, cptr(dX), IH, IW, cptr(dDY), mptr(dDW), mptr(dBuf), N, IC, OC));
}
#define DW_TAIL jlong dX, jint IH, jint IW, jlong dDY, jint OH, jint OW, jlong dDW, jlong dBuf, jint FH, jint FW, jint N, \
                jint IC, jint OC, jint ph, jint pw, jint n
#define DW_TAIL_PASS cptr(dX), IH, IW, cptr(dDY), OH, OW, mptr(dDW), mptr(dBuf), FH, FW, N, IC, OC, ph, pw, n
JNIEXPORT jboolean JNICALL JNAME_DW(Im2col_1WinogradV2_1SHW_1s4_1texture)(JNIEnv* env, jclass, jlongArray streams,
                                                                          jint length, jint GridZ, jint OH_slice,
                                                                          jint OW_slice, DW_TAIL) {
  Streams s(env, streams, length);
  const int rc = cu32_dconv3D_deltaW_Im2col_WinogradV2_SHW_s4_texture(s.h, s.n, GridZ, OH_slice, OW_slice, DW_TAIL_PASS);
  return handled(env, rc);
  
}
JNIEXPORT jboolean JNICALL JNAME_DW(Im2col_1WinogradV2_1SHW_1s8_1texture)(JNIEnv* env, jclass, jlongArray streams,
                                                                          jint length, jint GridZ, jint OH_slice,
                                                                          jint OW_slice, DW_TAIL) {
  Streams s(env, streams, length);
  const int rc = cu32_dconv3D_deltaW_Im2col_WinogradV2_SHW_s8_texture(s.h, s.n, GridZ, OH_slice, OW_slice, DW_TAIL_PASS);
  return handled(env, rc);
  
}
JNIEXPORT jboolean JNICALL JNAME_DW(Im2col_1WinogradV2_1SHW_1s16_1texture)(JNIEnv* env, jclass, jlongArray streams,
                                                                           jint length, jint GridZ, jint OH_slice,
                                                                           jint OW_slice, jint c64, DW_TAIL) {
  Streams s(env, streams, length);
  const int rc =
      cu32_dconv3D_deltaW_Im2col_WinogradV2_SHW_s16_texture(s.h, s.n, GridZ, OH_slice, OW_slice, c64, DW_TAIL_PASS);
  return handled(env, rc);
  
}

// Contraction + bias row in one pass.  These natives do not exist in the reference's Java classes; a
// maintainer who wants the fusion declares them in the Java class and calls them from
// CudaFloat32EngineBase.matMul_biased / conv3D_biased instead of the two-kernel sequence.
JNIEXPORT void JNICALL JNAME(matMul, matMul_1biased)(JNIEnv* env, jclass, jlongArray streams, jint length,
                                                     jlong dA, jlong dB, jlong dC, jlong dBias, jint N, jint M,
                                                     jint K, jint width) {
  Streams s(env, streams, length);
  done(env, cu32_matMul_biased(s.h, s.n, cptr(dA), cptr(dB), mptr(dC), cptr(dBias), N, M, K, width));
}
JNIEXPORT void JNICALL JNAME(matMul, matMul_1mma_1biased)(JNIEnv* env, jclass, jlongArray streams, jint length,
                                                          jlong dA, jlong dB, jlong dC, jlong dBias, jint N,
                                                          jint M, jint K, jint width) {
  Streams s(env, streams, length);
  done(env, cu32_matMul_mma_biased(s.h, s.n, cptr(dA), cptr(dB), mptr(dC), cptr(dBias), N, M, K, width));
}
JNIEXPORT void JNICALL JNAME(matMul, SKbuf_1summary_1biased)(JNIEnv* env, jclass, jlong stream, jlong dCbuf,
                                                             jlong dC, jlong dBias, jint part, jint sizeC,
                                                             jint M, jint width) {
  done(env, cu32_SKbuf_summary_biased(stream, cptr(dCbuf), mptr(dC), cptr(dBias), part, sizeC, M, width));
}
JNIEXPORT void JNICALL JNAME(conv3D, conv3D_1GemmR_1biased)(JNIEnv* env, jclass, jlongArray streams, jint length,
                                                            jlong dX, jint IH, jint IW, jlong dW, jlong dCW,
                                                            jint FH, jint FW, jlong dY, jint OH, jint OW, jint N,
                                                            jint IC, jint OC, jint sh, jint sw, jint ph, jint pw,
                                                            jlong dBias, jint width) {
  Streams s(env, streams, length);
  done(env, cu32_conv3D_GemmR_biased(s.h, s.n, cptr(dX), IH, IW, cptr(dW), cptr(dCW), FH, FW, mptr(dY), OH, OW, N,
                                     IC, OC, sh, sw, ph, pw, cptr(dBias), width));
}
// The V2 and Im2col-Winograd natives (reference: Cuda_conv3D/A.cu:89-111, :390-412, :429-637): same
// arguments, same result; the Winograd ones tell Java whether they handled the shape - always.
JNIEXPORT void JNICALL JNAME(conv3D, conv3DV2)(JNIEnv* env, jclass, jboolean useTexture, jlongArray streams,
                                               jint length, jlong dX, jint IH, jint IW, jlong dW, jint FH,
                                               jint FW, jlong dY, jint OH, jint OW, jint N, jint IC, jint OC,
                                               jint sh, jint sw, jint ph, jint pw) {
  Streams s(env, streams, length);
  done(env, cu32_conv3DV2(useTexture ? 1 : 0, s.h, s.n, cptr(dX), IH, IW, cptr(dW), FH, FW, mptr(dY), OH, OW, N, IC,
                          OC, sh, sw, ph, pw));
}
JNIEXPORT void JNICALL JNAME(conv3D, conv3D_1GemmV2R)(JNIEnv* env, jclass, jboolean useTexture,
                                                      jlongArray streams, jint length, jlong dX, jint IH,
                                                      jint IW, jlong dW, jlong dCW, jint FH, jint FW, jlong dY,
                                                      jint OH, jint OW, jint N, jint IC, jint OC, jint sh,
                                                      jint sw, jint ph, jint pw) {
  Streams s(env, streams, length);
  done(env, cu32_conv3D_GemmV2R(useTexture ? 1 : 0, s.h, s.n, cptr(dX), IH, IW, cptr(dW), cptr(dCW), FH, FW,
                                mptr(dY), OH, OW, N, IC, OC, sh, sw, ph, pw));
}
#define CONV_WINOGRAD(jname, cname)                                                                        \
  JNIEXPORT jboolean JNICALL JNAME(conv3D, jname)(JNIEnv* env, jclass, jboolean useTexture,                \
                                                  jlongArray streams, jint length, jlong dX, jint IH,      \
                                                  jint IW, jlong dW, jlong dCW, jint FH, jint FW,          \
                                                  jlong dY, jint OH, jint OW, jint N, jint IC, jint OC,    \
                                                  jint ph, jint pw) {                                      \
    Streams s(env, streams, length);                                                                       \
    const int rc = cname(useTexture ? 1 : 0, s.h, s.n, cptr(dX), IH, IW, cptr(dW), cptr(dCW), FH, FW,      \
                         mptr(dY), OH, OW, N, IC, OC, ph, pw);                                             \
    return handled(env, rc);                                                                                         \
                                                                                    \
  }
#define CONV_WINOGRAD_SGM(jname, cname)                                                                    \
  JNIEXPORT jboolean JNICALL JNAME(conv3D, jname)(JNIEnv* env, jclass, jboolean useTexture,                \
                                                  jlongArray streams, jint length, jlong dX, jint IH,      \
                                                  jint IW, jlong dW, jlong dCW, jint FH, jint FW,          \
                                                  jlong dY, jint OH, jint OW, jint N, jint IC, jint OC,    \
                                                  jint ph, jint pw, jint GM_slice) {                       \
    Streams s(env, streams, length);                                                                       \
    const int rc = cname(useTexture ? 1 : 0, s.h, s.n, cptr(dX), IH, IW, cptr(dW), cptr(dCW), FH, FW,      \
                         mptr(dY), OH, OW, N, IC, OC, ph, pw, GM_slice);                                   \
    return handled(env, rc);                                                                                         \
                                                                                    \
  }
CONV_WINOGRAD(conv3D_1Im2col_1Winograd_1s8_1R_1texture, cu32_conv3D_Im2col_Winograd_s8_R_texture)
CONV_WINOGRAD_SGM(conv3D_1Im2col_1WinogradR_1s8_1texture_1SGM, cu32_conv3D_Im2col_WinogradR_s8_texture_SGM)
CONV_WINOGRAD(conv3D_1Im2col_1Winograd_1s16_1R_1texture, cu32_conv3D_Im2col_Winograd_s16_R_texture)
CONV_WINOGRAD_SGM(conv3D_1Im2col_1WinogradR_1s16_1texture_1SGM, cu32_conv3D_Im2col_WinogradR_s16_texture_SGM)
JNIEXPORT void JNICALL JNAME(conv3D, conv3D_1GemmR_1W1)(JNIEnv* env, jclass, jlongArray streams, jint length,
                                                        jlong dX, jint IH, jint IW, jlong dW, jlong dCW,
                                                        jlong dY, jint N, jint IC, jint OC) {
  Streams s(env, streams, length);
  done(env, cu32_conv3D_GemmR_W1(s.h, s.n, cptr(dX), IH, IW, cptr(dW), cptr(dCW), mptr(dY), N, IC, OC));
}
JNIEXPORT void JNICALL JNAME(conv3D, conv3D_1GemmR_1W1_1SGM)(JNIEnv* env, jclass, jlongArray streams,
                                                             jint length, jlong dX, jint IH, jint IW,
                                                             jlong dW, jlong dCW, jlong dY, jint N, jint IC,
                                                             jint OC, jint GM_slice) {
  Streams s(env, streams, length);
  done(env, cu32_conv3D_GemmR_W1_SGM(s.h, s.n, cptr(dX), IH, IW, cptr(dW), cptr(dCW), mptr(dY), N, IC, OC, GM_slice));
}

}  // extern "C"
