/* C ABI of libdragon_cuda.so: the part of the reference's `Cuda` runtime-bridge library (its Windows DLL Cuda.dll,
 * Java class z.dragon.engine.cuda.impl.Cuda) that the callers of the contraction natives use - device memory,
 * asynchronous copies, streams, events, fills and error strings - so that a matMul / batchMatMul / conv3D program of
 * the Java engine finds every native it needs on Linux.  The JNI symbols of the same library
 * (Java_z_dragon_engine_cuda_impl_Cuda_*) are thin wrappers over these functions.
 *
 * Every function returns 0 or a cudaError_t value (the JNI wrapper turns a non-zero value into
 * z.dragon.engine.cuda.impl.CudaException(int), as the reference's handleError does, Cuda/JNITool.cuh:9-26).
 * Reference: source/engine-cuda-base/Cuda/Cuda/ (file and lines given per function). */
#ifndef DRAGON_CUDA_H
#define DRAGON_CUDA_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#define DCUDA_API __attribute__((visibility("default")))
#else
#define DCUDA_API
#endif

/* ---- memory (Cuda_memory.cuh:6-110) */
DCUDA_API int dcuda_malloc(int64_t size, int64_t* address);
DCUDA_API int dcuda_free(int64_t address);
DCUDA_API int dcuda_mallocHost(int64_t size, int64_t* address);
DCUDA_API int dcuda_freeHost(int64_t address);
DCUDA_API int dcuda_memsetAsync(int64_t stream, int64_t address, int value, int64_t size);
/* kind: 0 host to device, 1 host to host, 2 device to host, 3 device to device, 4 default (Cuda.java:74-78) */
DCUDA_API int dcuda_memcpyAsync(int64_t stream, int64_t dst, int64_t src, int64_t size, int kind);

/* ---- device (Cuda_Device.cuh) */
DCUDA_API int dcuda_getDeviceId(int* id);
DCUDA_API int dcuda_getDeviceCount(int* count);
DCUDA_API int dcuda_setDevice(int id);
DCUDA_API int dcuda_deviceSynchronize(void);
/* The next four change state that outlasts the call (device reset, peer access); the Java engine calls them at
 * start-up and shut-down only. */
DCUDA_API int dcuda_resetDevice(void);
DCUDA_API int dcuda_isDeviceP2PAccessEnabled(int dev1, int dev2, int* enabled);
DCUDA_API int dcuda_enableDeviceP2PAccess(int dev2);
DCUDA_API int dcuda_disableDeviceP2PAccess(int dev2);

/* ---- streams (Cuda_Stream.cuh:6-110) */
DCUDA_API int dcuda_getStreamPriorityRange(int* low, int* high);
/* nonblocking: 0 = cudaStreamDefault, 1 = cudaStreamNonBlocking; use_priority 0 ignores `priority` */
DCUDA_API int dcuda_newStream(int nonblocking, int use_priority, int priority, int64_t* stream);
DCUDA_API int dcuda_deleteStream(int64_t stream);
DCUDA_API int dcuda_streamQuery(int64_t stream, int* completed);
DCUDA_API int dcuda_streamSynchronize(int64_t stream);

/* ---- events (Cuda_Event.cuh:6-150) */
/* flavour: 0 default, 1 blocking sync, 2 timing disabled, 3 interprocess */
DCUDA_API int dcuda_newEvent(int flavour, int64_t* event);
DCUDA_API int dcuda_deleteEvent(int64_t event);
DCUDA_API int dcuda_eventRecord(int64_t event, int64_t stream);
/* The reference's eventRecord(event, long[] streams, n) does not record anything: it synchronises each stream in turn
 * (Cuda_Event.cuh:56-65).  Same here. */
DCUDA_API int dcuda_eventRecordStreams(int64_t event, const int64_t* streams, int length);
DCUDA_API int dcuda_eventSynchronize(int64_t event);
DCUDA_API int dcuda_eventElapsedTime(int64_t start, int64_t stop, float* ms);
DCUDA_API int dcuda_streamWaitEvent(int64_t stream, int64_t event, int external);

/* ---- errors (Cuda_Exception.cuh) */
DCUDA_API const char* dcuda_getExceptionName(int type);
DCUDA_API const char* dcuda_getExceptionInfo(int type);
DCUDA_API int dcuda_getLastExceptionType(void);

/* ---- FP32 fills and transfers (Cuda_float.cuh, Cuda_float_set1D.cuh:20-60, Cuda_float_set2D.cuh:29-75)
 * set1D: X[0..length) = value.  set2D: X is [height][stride]; columns < width get value, the padding columns 0.
 * length and stride are multiples of 4 (the engine's padding rule), X 16-byte aligned. */
DCUDA_API int dcuda_set1D(int64_t stream, int64_t address, float value, int length);
DCUDA_API int dcuda_set2D(int64_t stream, int64_t address, float value, int height, int width, int stride);
/* host <-> device with the stream synchronised before returning, as the reference's get1D / set1D(float[]) do;
 * the 2-D forms convert between the packed host layout [height][width] and the padded device layout
 * [height][stride] (padding written as 0). */
DCUDA_API int dcuda_get1D(int64_t stream, int64_t address, float* host, int length);
DCUDA_API int dcuda_put1D(int64_t stream, int64_t address, const float* host, int length);
DCUDA_API int dcuda_get2D(int64_t stream, int64_t address, float* host, int height, int width, int stride);
DCUDA_API int dcuda_put2D(int64_t stream, int64_t address, const float* host, int height, int width, int stride);

#ifdef __cplusplus
}
#endif
#endif /* DRAGON_CUDA_H */
