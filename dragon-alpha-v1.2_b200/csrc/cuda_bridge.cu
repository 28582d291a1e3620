// libdragon_cuda.so: the reference's `Cuda` runtime bridge for Linux - the natives of
// z.dragon.engine.cuda.impl.Cuda that a matMul / batchMatMul / conv3D program of the Java engine calls around the
// contraction natives: device memory, asynchronous copies, streams, events, fills, error strings.
// The C ABI is declared in include/dragon_cuda.h; the JNI symbols below wrap it one to one, with the reference's
// error behaviour (a failing CUDA call raises z.dragon.engine.cuda.impl.CudaException(int) and returns normally,
// engine-cuda-base/Cuda/Cuda/JNITool.cuh:9-26).
#include <cuda_runtime.h>
#include <cstdint>
#include <cstring>
#include <vector>

#ifdef DRAGON_USE_SYSTEM_JNI
#include <jni.h>
static inline jclass jni_FindClass(JNIEnv* env, const char* n) { return env->FindClass(n); }
static inline jint jni_Throw(JNIEnv* env, jthrowable o) { return env->Throw(o); }
static inline jobject jni_NewObjectA(JNIEnv* env, jclass c, jmethodID m, const jvalue* a) { return env->NewObjectA(c, m, a); }
static inline jmethodID jni_GetMethodID(JNIEnv* env, jclass c, const char* n, const char* s) { return env->GetMethodID(c, n, s); }
static inline void jni_GetLongArrayRegion(JNIEnv* env, jlongArray a, jint s, jint l, jlong* b) { env->GetLongArrayRegion(a, s, l, b); }
static inline jstring jni_NewStringUTF(JNIEnv* env, const char* u) { return env->NewStringUTF(u); }
static inline jintArray jni_NewIntArray(JNIEnv* env, jint n) { return env->NewIntArray(n); }
static inline void jni_GetFloatArrayRegion(JNIEnv* env, jfloatArray a, jint s, jint l, jfloat* b) { env->GetFloatArrayRegion(a, s, l, b); }
static inline void jni_SetIntArrayRegion(JNIEnv* env, jintArray a, jint s, jint l, const jint* b) { env->SetIntArrayRegion(a, s, l, b); }
static inline void jni_SetFloatArrayRegion(JNIEnv* env, jfloatArray a, jint s, jint l, const jfloat* b) { env->SetFloatArrayRegion(a, s, l, b); }
#else
#include "jni_min.h"
#endif
#include "../../include/dragon_cuda.h"

namespace {

inline cudaStream_t as_stream(int64_t h) { return reinterpret_cast<cudaStream_t>(static_cast<intptr_t>(h)); }
inline cudaEvent_t as_event(int64_t h) { return reinterpret_cast<cudaEvent_t>(static_cast<intptr_t>(h)); }
inline void* as_ptr(int64_t a) { return reinterpret_cast<void*>(static_cast<intptr_t>(a)); }

// X[i] = value, four floats per thread per step.
__global__ void fill1d_kernel(float* __restrict__ X, float value, int length) {
  const int step = gridDim.x * blockDim.x * 4;
  for (int i = (blockIdx.x * blockDim.x + threadIdx.x) * 4; i < length; i += step) {
    if (i + 3 < length) {
      *reinterpret_cast<float4*>(X + i) = make_float4(value, value, value, value);
    } else {
      for (int j = i; j < length; ++j) X[j] = value;
    }
  }
}
// X[row][col] = col < width ? value : 0 over [height][stride] floats (stride % 4 == 0).
__global__ void fill2d_kernel(float* __restrict__ X, float value, long long lengthv, int width, int stride) {
  const long long step = static_cast<long long>(gridDim.x) * blockDim.x * 4;
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4; i < lengthv; i += step) {
    const int col = static_cast<int>(i % stride);
    float4 v;
    v.x = col + 0 < width ? value : 0.f;
    v.y = col + 1 < width ? value : 0.f;
    v.z = col + 2 < width ? value : 0.f;
    v.w = col + 3 < width ? value : 0.f;
    *reinterpret_cast<float4*>(X + i) = v;
  }
}

int fill_blocks(long long elems) {
  int dev = 0, sms = 1;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  long long b = (elems / 4 + 255) / 256;
  if (b > sms * 16LL) b = sms * 16LL;
  return b < 1 ? 1 : static_cast<int>(b);
}

}  // namespace

extern "C" {

// ------------------------------------------------------------------ memory
int dcuda_malloc(int64_t size, int64_t* address) {
  void* p = nullptr;
  const cudaError_t e = cudaMalloc(&p, static_cast<size_t>(size));
  *address = static_cast<int64_t>(reinterpret_cast<intptr_t>(p));
  return static_cast<int>(e);
}
int dcuda_free(int64_t address) { return static_cast<int>(cudaFree(as_ptr(address))); }
int dcuda_mallocHost(int64_t size, int64_t* address) {
  void* p = nullptr;
  const cudaError_t e = cudaMallocHost(&p, static_cast<size_t>(size));
  *address = static_cast<int64_t>(reinterpret_cast<intptr_t>(p));
  return static_cast<int>(e);
}
int dcuda_freeHost(int64_t address) { return static_cast<int>(cudaFreeHost(as_ptr(address))); }
int dcuda_memsetAsync(int64_t stream, int64_t address, int value, int64_t size) {
  return static_cast<int>(cudaMemsetAsync(as_ptr(address), value, static_cast<size_t>(size), as_stream(stream)));
}
int dcuda_memcpyAsync(int64_t stream, int64_t dst, int64_t src, int64_t size, int kind) {
  static const cudaMemcpyKind kinds[5] = {cudaMemcpyHostToDevice, cudaMemcpyHostToHost, cudaMemcpyDeviceToHost,
                                          cudaMemcpyDeviceToDevice, cudaMemcpyDefault};
  if (kind < 0 || kind > 4) return static_cast<int>(cudaErrorInvalidMemcpyDirection);
  return static_cast<int>(cudaMemcpyAsync(as_ptr(dst), as_ptr(src), static_cast<size_t>(size), kinds[kind], as_stream(stream)));
}

// ------------------------------------------------------------------ device
int dcuda_getDeviceId(int* id) { return static_cast<int>(cudaGetDevice(id)); }
int dcuda_getDeviceCount(int* count) { return static_cast<int>(cudaGetDeviceCount(count)); }
int dcuda_setDevice(int id) { return static_cast<int>(cudaSetDevice(id)); }
int dcuda_deviceSynchronize(void) { return static_cast<int>(cudaDeviceSynchronize()); }
int dcuda_resetDevice(void) { return static_cast<int>(cudaDeviceReset()); }
int dcuda_isDeviceP2PAccessEnabled(int dev1, int dev2, int* enabled) {
  return static_cast<int>(cudaDeviceCanAccessPeer(enabled, dev1, dev2));
}
int dcuda_enableDeviceP2PAccess(int dev2) { return static_cast<int>(cudaDeviceEnablePeerAccess(dev2, 0)); }
int dcuda_disableDeviceP2PAccess(int dev2) { return static_cast<int>(cudaDeviceDisablePeerAccess(dev2)); }

// ------------------------------------------------------------------ streams
int dcuda_getStreamPriorityRange(int* low, int* high) { return static_cast<int>(cudaDeviceGetStreamPriorityRange(low, high)); }
int dcuda_newStream(int nonblocking, int use_priority, int priority, int64_t* stream) {
  cudaStream_t s = nullptr;
  const unsigned flags = nonblocking ? cudaStreamNonBlocking : cudaStreamDefault;
  const cudaError_t e = use_priority ? cudaStreamCreateWithPriority(&s, flags, priority)
                                     : (nonblocking ? cudaStreamCreateWithFlags(&s, flags) : cudaStreamCreate(&s));
  *stream = static_cast<int64_t>(reinterpret_cast<intptr_t>(s));
  return static_cast<int>(e);
}
int dcuda_deleteStream(int64_t stream) { return static_cast<int>(cudaStreamDestroy(as_stream(stream))); }
int dcuda_streamQuery(int64_t stream, int* completed) {
  const cudaError_t e = cudaStreamQuery(as_stream(stream));
  *completed = e == cudaSuccess ? 1 : 0;
  return (e == cudaSuccess || e == cudaErrorNotReady) ? 0 : static_cast<int>(e);
}
int dcuda_streamSynchronize(int64_t stream) { return static_cast<int>(cudaStreamSynchronize(as_stream(stream))); }

// ------------------------------------------------------------------ events
int dcuda_newEvent(int flavour, int64_t* event) {
  static const unsigned flags[4] = {cudaEventDefault, cudaEventBlockingSync, cudaEventDisableTiming, cudaEventInterprocess};
  if (flavour < 0 || flavour > 3) return static_cast<int>(cudaErrorInvalidValue);
  cudaEvent_t ev = nullptr;
  // an interprocess event must also have timing disabled
  const cudaError_t e = cudaEventCreateWithFlags(&ev, flavour == 3 ? (cudaEventInterprocess | cudaEventDisableTiming) : flags[flavour]);
  *event = static_cast<int64_t>(reinterpret_cast<intptr_t>(ev));
  return static_cast<int>(e);
}
int dcuda_deleteEvent(int64_t event) { return static_cast<int>(cudaEventDestroy(as_event(event))); }
int dcuda_eventRecord(int64_t event, int64_t stream) { return static_cast<int>(cudaEventRecord(as_event(event), as_stream(stream))); }
int dcuda_eventRecordStreams(int64_t event, const int64_t* streams, int length) {
  (void)event;
  for (int i = 0; i < length; ++i) {
    const cudaError_t e = cudaStreamSynchronize(as_stream(streams[i]));
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  return 0;
}
int dcuda_eventSynchronize(int64_t event) { return static_cast<int>(cudaEventSynchronize(as_event(event))); }
int dcuda_eventElapsedTime(int64_t start, int64_t stop, float* ms) {
  return static_cast<int>(cudaEventElapsedTime(ms, as_event(start), as_event(stop)));
}
int dcuda_streamWaitEvent(int64_t stream, int64_t event, int external) {
  return static_cast<int>(cudaStreamWaitEvent(as_stream(stream), as_event(event), external ? cudaEventWaitExternal : cudaEventWaitDefault));
}

// ------------------------------------------------------------------ errors
const char* dcuda_getExceptionName(int type) { return cudaGetErrorName(static_cast<cudaError_t>(type)); }
const char* dcuda_getExceptionInfo(int type) { return cudaGetErrorString(static_cast<cudaError_t>(type)); }
int dcuda_getLastExceptionType(void) { return static_cast<int>(cudaGetLastError()); }

// ------------------------------------------------------------------ FP32 fills and transfers
int dcuda_set1D(int64_t stream, int64_t address, float value, int length) {
  if (length <= 0) return static_cast<int>(cudaErrorInvalidValue);
  fill1d_kernel<<<fill_blocks(length), 256, 0, as_stream(stream)>>>(static_cast<float*>(as_ptr(address)), value, length);
  return static_cast<int>(cudaPeekAtLastError());
}
int dcuda_set2D(int64_t stream, int64_t address, float value, int height, int width, int stride) {
  if (height <= 0 || width <= 0 || stride < width || (stride & 3)) return static_cast<int>(cudaErrorInvalidValue);
  const long long lengthv = static_cast<long long>(height) * stride;
  fill2d_kernel<<<fill_blocks(lengthv), 256, 0, as_stream(stream)>>>(static_cast<float*>(as_ptr(address)), value, lengthv, width, stride);
  return static_cast<int>(cudaPeekAtLastError());
}
int dcuda_get1D(int64_t stream, int64_t address, float* host, int length) {
  cudaError_t e = cudaMemcpyAsync(host, as_ptr(address), static_cast<size_t>(length) * 4, cudaMemcpyDeviceToHost, as_stream(stream));
  if (e != cudaSuccess) return static_cast<int>(e);
  return static_cast<int>(cudaStreamSynchronize(as_stream(stream)));
}
int dcuda_put1D(int64_t stream, int64_t address, const float* host, int length) {
  cudaError_t e = cudaMemcpyAsync(as_ptr(address), host, static_cast<size_t>(length) * 4, cudaMemcpyHostToDevice, as_stream(stream));
  if (e != cudaSuccess) return static_cast<int>(e);
  return static_cast<int>(cudaStreamSynchronize(as_stream(stream)));
}
int dcuda_get2D(int64_t stream, int64_t address, float* host, int height, int width, int stride) {
  cudaError_t e = cudaMemcpy2DAsync(host, static_cast<size_t>(width) * 4, as_ptr(address), static_cast<size_t>(stride) * 4,
                                    static_cast<size_t>(width) * 4, static_cast<size_t>(height), cudaMemcpyDeviceToHost, as_stream(stream));
  if (e != cudaSuccess) return static_cast<int>(e);
  return static_cast<int>(cudaStreamSynchronize(as_stream(stream)));
}
int dcuda_put2D(int64_t stream, int64_t address, const float* host, int height, int width, int stride) {
  // padded image built on the host, as the reference does (Cuda_float.cuh:311-335): padding columns are zeros
  std::vector<float> padded(static_cast<size_t>(height) * stride, 0.0f);
  for (int r = 0; r < height; ++r)
    std::memcpy(padded.data() + static_cast<size_t>(r) * stride, host + static_cast<size_t>(r) * width, static_cast<size_t>(width) * 4);
  cudaError_t e = cudaMemcpyAsync(as_ptr(address), padded.data(), padded.size() * 4, cudaMemcpyHostToDevice, as_stream(stream));
  if (e != cudaSuccess) return static_cast<int>(e);
  return static_cast<int>(cudaStreamSynchronize(as_stream(stream)));   // `padded` must outlive the copy
}

}  // extern "C"

// ==================================================================== JNI exports
namespace {

void throw_cuda_exception(JNIEnv* env, int code) {
  jclass cls = jni_FindClass(env, "z/dragon/engine/cuda/impl/CudaException");
  if (!cls) return;
  jmethodID ctor = jni_GetMethodID(env, cls, "<init>", "(I)V");
  if (!ctor) return;
  jvalue arg;
  arg.i = code;
  jobject ex = jni_NewObjectA(env, cls, ctor, &arg);
  if (ex) jni_Throw(env, static_cast<jthrowable>(ex));
}
inline void done(JNIEnv* env, int rc) { if (rc != 0) throw_cuda_exception(env, rc); }

// Up to `length` stream handles out of a Java long[] (the reference uses GetLongArrayElements; a region copy
// needs no release call).
std::vector<int64_t> handles(JNIEnv* env, jlongArray arr, jint length) {
  std::vector<int64_t> out(length > 0 ? length : 0);
  if (length > 0) {
    std::vector<jlong> tmp(length);
    jni_GetLongArrayRegion(env, arr, 0, length, tmp.data());
    for (jint i = 0; i < length; ++i) out[i] = tmp[i];
  }
  return out;
}

}  // namespace

#define CUDA_NATIVE(name) Java_z_dragon_engine_cuda_impl_Cuda_##name

extern "C" {

JNIEXPORT jlong JNICALL CUDA_NATIVE(malloc)(JNIEnv* env, jclass, jlong size) {
  int64_t a = 0; done(env, dcuda_malloc(size, &a)); return a;
}
JNIEXPORT void JNICALL CUDA_NATIVE(free)(JNIEnv* env, jclass, jlong address) { done(env, dcuda_free(address)); }
JNIEXPORT jlong JNICALL CUDA_NATIVE(mallocHost)(JNIEnv* env, jclass, jlong size) {
  int64_t a = 0; done(env, dcuda_mallocHost(size, &a)); return a;
}
JNIEXPORT void JNICALL CUDA_NATIVE(freeHost)(JNIEnv* env, jclass, jlong address) { done(env, dcuda_freeHost(address)); }
JNIEXPORT void JNICALL CUDA_NATIVE(memsetAsync)(JNIEnv* env, jclass, jlong stream, jlong address, jint value, jlong size) {
  done(env, dcuda_memsetAsync(stream, address, value, size));
}
#define MEMCPY_NATIVE(name, kind)                                                                                 \
  JNIEXPORT void JNICALL CUDA_NATIVE(name)(JNIEnv* env, jclass, jlong stream, jlong dst, jlong src, jlong size) { \
    done(env, dcuda_memcpyAsync(stream, dst, src, size, kind));                                                    \
  }
MEMCPY_NATIVE(memcpyAsyncHostToDevice, 0)
MEMCPY_NATIVE(memcpyAsyncHostToHost, 1)
MEMCPY_NATIVE(memcpyAsyncDeviceToHost, 2)
MEMCPY_NATIVE(memcpyAsyncDeviceToDevice, 3)
MEMCPY_NATIVE(memcpyAsyncDefault, 4)

JNIEXPORT jint JNICALL CUDA_NATIVE(getDeviceId)(JNIEnv* env, jclass) { int v = 0; done(env, dcuda_getDeviceId(&v)); return v; }
JNIEXPORT jint JNICALL CUDA_NATIVE(getDeviceCount)(JNIEnv* env, jclass) { int v = 0; done(env, dcuda_getDeviceCount(&v)); return v; }
JNIEXPORT void JNICALL CUDA_NATIVE(setDevice)(JNIEnv* env, jclass, jint id) { done(env, dcuda_setDevice(id)); }
JNIEXPORT void JNICALL CUDA_NATIVE(resetDevice)(JNIEnv* env, jclass) { done(env, dcuda_resetDevice()); }
JNIEXPORT void JNICALL CUDA_NATIVE(deviceSynchronize)(JNIEnv* env, jclass) { done(env, dcuda_deviceSynchronize()); }
JNIEXPORT jboolean JNICALL CUDA_NATIVE(isDeviceP2PAccessEnabled)(JNIEnv* env, jclass, jint d1, jint d2) {
  int v = 0; done(env, dcuda_isDeviceP2PAccessEnabled(d1, d2, &v)); return v ? 1 : 0;
}
JNIEXPORT void JNICALL CUDA_NATIVE(enableDeviceP2PAccess)(JNIEnv* env, jclass, jint d2) { done(env, dcuda_enableDeviceP2PAccess(d2)); }
JNIEXPORT void JNICALL CUDA_NATIVE(disableDeviceP2PAccess)(JNIEnv* env, jclass, jint d2) { done(env, dcuda_disableDeviceP2PAccess(d2)); }

JNIEXPORT jintArray JNICALL CUDA_NATIVE(getStreamPriorityRange)(JNIEnv* env, jclass) {
  jint range[2] = {0, 0};
  int lo = 0, hi = 0;
  done(env, dcuda_getStreamPriorityRange(&lo, &hi));
  range[0] = lo; range[1] = hi;
  jintArray arr = jni_NewIntArray(env, 2);
  if (arr) jni_SetIntArrayRegion(env, arr, 0, 2, range);
  return arr;
}
JNIEXPORT jlong JNICALL CUDA_NATIVE(newStream_1Blocking__)(JNIEnv* env, jclass) {
  int64_t s = 0; done(env, dcuda_newStream(0, 0, 0, &s)); return s;
}
JNIEXPORT jlong JNICALL CUDA_NATIVE(newStream_1Blocking__I)(JNIEnv* env, jclass, jint priority) {
  int64_t s = 0; done(env, dcuda_newStream(0, 1, priority, &s)); return s;
}
JNIEXPORT jlong JNICALL CUDA_NATIVE(newStream_1NonBlocking__)(JNIEnv* env, jclass) {
  int64_t s = 0; done(env, dcuda_newStream(1, 0, 0, &s)); return s;
}
JNIEXPORT jlong JNICALL CUDA_NATIVE(newStream_1NonBlocking__I)(JNIEnv* env, jclass, jint priority) {
  int64_t s = 0; done(env, dcuda_newStream(1, 1, priority, &s)); return s;
}
JNIEXPORT void JNICALL CUDA_NATIVE(deleteStream__J)(JNIEnv* env, jclass, jlong stream) { done(env, dcuda_deleteStream(stream)); }
JNIEXPORT void JNICALL CUDA_NATIVE(deleteStream___3JI)(JNIEnv* env, jclass, jlongArray streams, jint length) {
  for (int64_t s : handles(env, streams, length)) done(env, dcuda_deleteStream(s));
}
JNIEXPORT jboolean JNICALL CUDA_NATIVE(streamQuery)(JNIEnv* env, jclass, jlong stream) {
  int v = 0; done(env, dcuda_streamQuery(stream, &v)); return v ? 1 : 0;
}
JNIEXPORT void JNICALL CUDA_NATIVE(streamSynchronize__J)(JNIEnv* env, jclass, jlong stream) { done(env, dcuda_streamSynchronize(stream)); }
JNIEXPORT void JNICALL CUDA_NATIVE(streamSynchronize___3JI)(JNIEnv* env, jclass, jlongArray streams, jint length) {
  for (int64_t s : handles(env, streams, length)) done(env, dcuda_streamSynchronize(s));
}

#define EVENT_NEW(name, flavour)                                                                   \
  JNIEXPORT jlong JNICALL CUDA_NATIVE(name)(JNIEnv* env, jclass) {                                 \
    int64_t e = 0; done(env, dcuda_newEvent(flavour, &e)); return e;                               \
  }
EVENT_NEW(newEvent_1Default, 0)
EVENT_NEW(newEvent_1BlockingSync, 1)
EVENT_NEW(newEvent_1DisableTiming, 2)
EVENT_NEW(newEvent_1Interprocess, 3)
JNIEXPORT void JNICALL CUDA_NATIVE(deleteEvent)(JNIEnv* env, jclass, jlong event) { done(env, dcuda_deleteEvent(event)); }
JNIEXPORT void JNICALL CUDA_NATIVE(eventRecord__JJ)(JNIEnv* env, jclass, jlong event, jlong stream) {
  done(env, dcuda_eventRecord(event, stream));
}
JNIEXPORT void JNICALL CUDA_NATIVE(eventRecord__J_3JI)(JNIEnv* env, jclass, jlong event, jlongArray streams, jint length) {
  const std::vector<int64_t> h = handles(env, streams, length);
  done(env, dcuda_eventRecordStreams(event, h.data(), static_cast<int>(h.size())));
}
JNIEXPORT void JNICALL CUDA_NATIVE(eventSynchronize)(JNIEnv* env, jclass, jlong event) { done(env, dcuda_eventSynchronize(event)); }
JNIEXPORT void JNICALL CUDA_NATIVE(eventSync_1Del)(JNIEnv* env, jclass, jlong event) {
  done(env, dcuda_eventSynchronize(event));
  done(env, dcuda_deleteEvent(event));
}
JNIEXPORT jfloat JNICALL CUDA_NATIVE(eventElapsedTime)(JNIEnv* env, jclass, jlong start, jlong stop) {
  float ms = 0.f; done(env, dcuda_eventElapsedTime(start, stop, &ms)); return ms;
}
JNIEXPORT void JNICALL CUDA_NATIVE(streamWaitEvent_1default)(JNIEnv* env, jclass, jlong stream, jlong event) {
  done(env, dcuda_streamWaitEvent(stream, event, 0));
}
JNIEXPORT void JNICALL CUDA_NATIVE(streamWaitEvent_1external)(JNIEnv* env, jclass, jlong stream, jlong event) {
  done(env, dcuda_streamWaitEvent(stream, event, 1));
}
JNIEXPORT void JNICALL CUDA_NATIVE(streamsWaitEvent_1default)(JNIEnv* env, jclass, jlongArray streams, jint length, jlong event) {
  for (int64_t s : handles(env, streams, length)) done(env, dcuda_streamWaitEvent(s, event, 0));
}
JNIEXPORT void JNICALL CUDA_NATIVE(streamsWaitEvent_1external)(JNIEnv* env, jclass, jlongArray streams, jint length, jlong event) {
  for (int64_t s : handles(env, streams, length)) done(env, dcuda_streamWaitEvent(s, event, 1));
}

JNIEXPORT jstring JNICALL CUDA_NATIVE(getExceptionName)(JNIEnv* env, jclass, jint type) {
  return jni_NewStringUTF(env, dcuda_getExceptionName(type));
}
JNIEXPORT jstring JNICALL CUDA_NATIVE(getExceptionInfo)(JNIEnv* env, jclass, jint type) {
  return jni_NewStringUTF(env, dcuda_getExceptionInfo(type));
}
JNIEXPORT jint JNICALL CUDA_NATIVE(getLastExceptionType)(JNIEnv*, jclass) { return dcuda_getLastExceptionType(); }

JNIEXPORT void JNICALL CUDA_NATIVE(set1D__JJFI)(JNIEnv* env, jclass, jlong stream, jlong address, jfloat value, jint length) {
  done(env, dcuda_set1D(stream, address, value, length));
}
JNIEXPORT void JNICALL CUDA_NATIVE(set2D__JJFIII)(JNIEnv* env, jclass, jlong stream, jlong address, jfloat value, jint height,
                                                   jint width, jint stride) {
  done(env, dcuda_set2D(stream, address, value, height, width, stride));
}
JNIEXPORT void JNICALL CUDA_NATIVE(get1D)(JNIEnv* env, jclass, jlong stream, jlong address, jfloatArray value, jint length) {
  std::vector<float> host(length > 0 ? length : 0);
  const int rc = dcuda_get1D(stream, address, host.data(), length);
  done(env, rc);
  if (rc == 0) jni_SetFloatArrayRegion(env, value, 0, length, host.data());
}
JNIEXPORT void JNICALL CUDA_NATIVE(get2D)(JNIEnv* env, jclass, jlong stream, jlong address, jfloatArray value, jint height,
                                           jint width, jint stride) {
  std::vector<float> host(static_cast<size_t>(height > 0 ? height : 0) * (width > 0 ? width : 0));
  const int rc = dcuda_get2D(stream, address, host.data(), height, width, stride);
  done(env, rc);
  if (rc == 0) jni_SetFloatArrayRegion(env, value, 0, height * width, host.data());
}
JNIEXPORT void JNICALL CUDA_NATIVE(set1D__JJ_3FI)(JNIEnv* env, jclass, jlong stream, jlong address, jfloatArray value, jint length) {
  std::vector<float> host(length > 0 ? length : 0);
  jni_GetFloatArrayRegion(env, value, 0, length, host.data());
  done(env, dcuda_put1D(stream, address, host.data(), length));
}
JNIEXPORT void JNICALL CUDA_NATIVE(set2D__JJ_3FIII)(JNIEnv* env, jclass, jlong stream, jlong address, jfloatArray value, jint height,
                                                     jint width, jint stride) {
  std::vector<float> host(static_cast<size_t>(height > 0 ? height : 0) * (width > 0 ? width : 0));
  jni_GetFloatArrayRegion(env, value, 0, height * width, host.data());
  done(env, dcuda_put2D(stream, address, host.data(), height, width, stride));
}

}  // extern "C"
