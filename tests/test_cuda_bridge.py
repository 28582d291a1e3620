"""libdragon_cuda.so: the Linux port of the reference's `Cuda` runtime-bridge natives (device memory, copies, streams,
events, fills, error strings), driven through the C ABI and through the Java_* symbols with a fake JNIEnv.

Without a GPU every CUDA call fails cleanly, which is what the error path needs: the shim must construct
z.dragon.engine.cuda.impl.CudaException(int) and Throw it (engine-cuda-base/Cuda/Cuda/JNITool.cuh:9-26).  The natives
that change state outlasting the call - resetDevice and the peer-access switches - are exercised on that path only,
never on a GPU."""
import ctypes
import re
from ctypes import CFUNCTYPE, POINTER, c_char_p, c_float, c_int32, c_int64, c_void_p
from pathlib import Path

import numpy as np
import pytest

from test_jni import FakeJNI, ARRAY_HANDLE

ROOT = Path(__file__).resolve().parent.parent


class FakeJNI2(FakeJNI):
    """Adds the slots the bridge uses: NewStringUTF 167, NewIntArray 179, GetFloatArrayRegion 205,
    SetIntArrayRegion 211, SetFloatArrayRegion 213."""

    def __init__(self, streams, floats=None):
        super().__init__(streams)
        self.strings, self.int_arrays, self.floats = [], {}, floats

        def put(idx, proto, fn):
            cb = proto(fn)
            self._keep.append(cb)
            self.table[idx] = ctypes.cast(cb, c_void_p).value

        def new_string_utf(env, utf):
            self.strings.append(utf.decode())
            return 0x5000 + len(self.strings)

        def new_int_array(env, n):
            h = 0x6000 + len(self.int_arrays)
            self.int_arrays[h] = [None] * n
            return h

        def set_int_array_region(env, arr, start, n, buf):
            for i in range(n):
                self.int_arrays[arr][start + i] = buf[i]

        def get_float_array_region(env, arr, start, n, buf):
            for i in range(n):
                buf[i] = self.floats[start + i]

        def set_float_array_region(env, arr, start, n, buf):
            for i in range(n):
                self.floats[start + i] = buf[i]

        put(167, CFUNCTYPE(c_void_p, c_void_p, c_char_p), new_string_utf)
        put(179, CFUNCTYPE(c_void_p, c_void_p, c_int32), new_int_array)
        put(205, CFUNCTYPE(None, c_void_p, c_void_p, c_int32, c_int32, POINTER(c_float)), get_float_array_region)
        put(211, CFUNCTYPE(None, c_void_p, c_void_p, c_int32, c_int32, POINTER(c_int32)), set_int_array_region)
        put(213, CFUNCTYPE(None, c_void_p, c_void_p, c_int32, c_int32, POINTER(c_float)), set_float_array_region)


@pytest.fixture(scope="module")
def bridge(pkg):
    path = pkg.cu32.LIB_PATH.parent / "libdragon_cuda.so"
    if not path.exists():
        pkg.build.build()
    return ctypes.CDLL(str(path))


def _native(lib, name, argtypes, restype=None):
    f = getattr(lib, "Java_z_dragon_engine_cuda_impl_Cuda_" + name)
    f.argtypes = [c_void_p, c_void_p] + argtypes
    f.restype = restype
    return f


def test_bridge_exports_every_declared_symbol(bridge):
    header = (ROOT / "include" / "dragon_cuda.h").read_text()
    names = re.findall(r"DCUDA_API\s+[\w\s\*]+?\b(dcuda_\w+)\s*\(", header)
    assert len(names) >= 34
    for n in names:
        assert hasattr(bridge, n), n
    for n in ("malloc", "free", "mallocHost", "freeHost", "memsetAsync", "memcpyAsyncHostToDevice", "memcpyAsyncHostToHost",
              "memcpyAsyncDeviceToHost", "memcpyAsyncDeviceToDevice", "memcpyAsyncDefault", "getDeviceId", "getDeviceCount",
              "setDevice", "resetDevice", "deviceSynchronize", "isDeviceP2PAccessEnabled", "enableDeviceP2PAccess",
              "disableDeviceP2PAccess", "getStreamPriorityRange", "newStream_1Blocking__", "newStream_1Blocking__I",
              "newStream_1NonBlocking__", "newStream_1NonBlocking__I", "deleteStream__J", "deleteStream___3JI", "streamQuery",
              "streamSynchronize__J", "streamSynchronize___3JI", "newEvent_1Default", "newEvent_1BlockingSync",
              "newEvent_1DisableTiming", "newEvent_1Interprocess", "deleteEvent", "eventRecord__JJ", "eventRecord__J_3JI",
              "eventSynchronize", "eventSync_1Del", "eventElapsedTime", "streamWaitEvent_1default", "streamWaitEvent_1external",
              "streamsWaitEvent_1default", "streamsWaitEvent_1external", "getExceptionName", "getExceptionInfo",
              "getLastExceptionType", "set1D__JJFI", "set2D__JJFIII", "get1D", "get2D", "set1D__JJ_3FI", "set2D__JJ_3FIII"):
        assert hasattr(bridge, "Java_z_dragon_engine_cuda_impl_Cuda_" + n), n


def test_error_strings_need_no_device(bridge):
    bridge.dcuda_getExceptionName.restype = c_char_p
    bridge.dcuda_getExceptionInfo.restype = c_char_p
    assert bridge.dcuda_getExceptionName(2) == b"cudaErrorMemoryAllocation"
    assert bridge.dcuda_getExceptionName(0) == b"cudaSuccess"
    assert b"memory" in bridge.dcuda_getExceptionInfo(2)
    jni = FakeJNI2([0])
    h = _native(bridge, "getExceptionName", [c_int32], c_void_p)(jni.env, None, 700)
    assert jni.strings == ["cudaErrorIllegalAddress"] and h == 0x5001


def test_failures_become_cuda_exceptions_without_a_device(bridge):
    import torch
    if torch.cuda.is_available():
        pytest.skip("this is the no-device error path; on a GPU the same calls succeed (see the gpu test)")
    for name, args, argtypes in (("malloc", (1024,), [c_int64]), ("getDeviceCount", (), []), ("deviceSynchronize", (), []),
                                 ("resetDevice", (), []), ("enableDeviceP2PAccess", (1,), [c_int32]),
                                 ("disableDeviceP2PAccess", (1,), [c_int32]), ("newEvent_1Default", (), []),
                                 ("set1D__JJFI", (0, 0x10000, 1.0, 64), [c_int64, c_int64, c_float, c_int32])):
        jni = FakeJNI2([0])
        _native(bridge, name, argtypes, c_int64 if name in ("malloc", "newEvent_1Default") else None)(jni.env, None, *args)
        assert jni.thrown == 0x3333, name
        assert ("FindClass", "z/dragon/engine/cuda/impl/CudaException") in jni.log, name
        codes = [e[3] for e in jni.log if e[0] == "NewObjectA"]
        assert codes and codes[0] > 0, name          # a cudaError_t value
    # a rejected argument is reported the same way, before any CUDA call
    jni = FakeJNI2([0])
    _native(bridge, "set2D__JJFIII", [c_int64, c_int64, c_float, c_int32, c_int32, c_int32])(jni.env, None, 0, 0x10000, 1.0, 4, 8, 6)
    assert ("NewObjectA", 0x1111, 0x2222, 1) in jni.log     # cudaErrorInvalidValue: stride < width


@pytest.mark.gpu
def test_bridge_round_trip_on_gpu(bridge, pkg, cuda):
    """The sequence a matMul program of the engine performs around the contraction: allocate, upload, multiply
    through the Cu32 native on a bridge-created stream, record / wait events, download - all through JNI symbols."""
    torch = cuda
    jni = FakeJNI2([0])
    J = lambda name, argtypes, restype=None: _native(bridge, name, argtypes, restype)
    assert J("getDeviceCount", [], c_int32)(jni.env, None) >= 1
    assert J("getDeviceId", [], c_int32)(jni.env, None) == torch.cuda.current_device()
    rng_arr = J("getStreamPriorityRange", [], c_void_p)(jni.env, None)
    lo, hi = jni.int_arrays[rng_arr]
    assert hi <= lo                                       # CUDA: numerically lower = higher priority
    stream = J("newStream_1NonBlocking__", [], c_int64)(jni.env, None)
    stream2 = J("newStream_1Blocking__I", [c_int32], c_int64)(jni.env, None, hi)
    assert stream and stream2 and jni.thrown is None
    N, M, K = 64, 128, 96
    rng = np.random.default_rng(1)
    A, B = rng.standard_normal((N, K)).astype(np.float32), rng.standard_normal((K, M)).astype(np.float32)
    malloc = J("malloc", [c_int64], c_int64)
    dA, dB, dC = (malloc(jni.env, None, n * 4) for n in (N * K, K * M, N * M))
    put = J("set1D__JJ_3FI", [c_int64, c_int64, c_void_p, c_int32])
    for dev_ptr, host in ((dA, A), (dB, B)):
        jni.floats = host.ravel().tolist()
        put(jni.env, None, stream, dev_ptr, 0x7777, host.size)
    J("set1D__JJFI", [c_int64, c_int64, c_float, c_int32])(jni.env, None, stream, dC, -1.0, N * M)
    ev0, ev1 = (J("newEvent_1Default", [], c_int64)(jni.env, None) for _ in range(2))
    rec = J("eventRecord__JJ", [c_int64, c_int64])
    rec(jni.env, None, ev0, stream)
    pkg.cu32.Cuda_matMul.matMul([stream], 1, dA, dB, dC, N, M, K)
    rec(jni.env, None, ev1, stream)
    J("streamWaitEvent_1default", [c_int64, c_int64])(jni.env, None, stream2, ev1)
    jni.streams = [stream, stream2]
    J("eventRecord__J_3JI", [c_int64, c_void_p, c_int32])(jni.env, None, ev1, ARRAY_HANDLE, 2)     # joins both streams
    assert J("streamQuery", [c_int64], ctypes.c_uint8)(jni.env, None, stream) == 1
    assert J("eventElapsedTime", [c_int64, c_int64], c_float)(jni.env, None, ev0, ev1) >= 0.0
    jni.floats = [0.0] * (N * M)
    J("get1D", [c_int64, c_int64, c_void_p, c_int32])(jni.env, None, stream, dC, 0x7777, N * M)
    C = np.array(jni.floats, np.float32).reshape(N, M)
    ref = A.astype(np.float64) @ B.astype(np.float64)
    assert np.linalg.norm(C - ref) / np.linalg.norm(ref) <= 1e-6
    # 2-D fill and packed <-> padded transfers
    H, W, S = 5, 6, 8
    d2 = malloc(jni.env, None, H * S * 4)
    J("set2D__JJFIII", [c_int64, c_int64, c_float, c_int32, c_int32, c_int32])(jni.env, None, stream, d2, 2.5, H, W, S)
    jni.floats = [0.0] * (H * S)
    J("get1D", [c_int64, c_int64, c_void_p, c_int32])(jni.env, None, stream, d2, 0x7777, H * S)
    img = np.array(jni.floats, np.float32).reshape(H, S)
    assert np.all(img[:, :W] == 2.5) and np.all(img[:, W:] == 0)
    packed = rng.standard_normal((H, W)).astype(np.float32)
    jni.floats = packed.ravel().tolist()
    J("set2D__JJ_3FIII", [c_int64, c_int64, c_void_p, c_int32, c_int32, c_int32])(jni.env, None, stream, d2, 0x7777, H, W, S)
    jni.floats = [0.0] * (H * W)
    J("get2D", [c_int64, c_int64, c_void_p, c_int32, c_int32, c_int32])(jni.env, None, stream, d2, 0x7777, H, W, S)
    assert np.array_equal(np.array(jni.floats, np.float32).reshape(H, W), packed)
    # device-to-device copy, memset, then clean-up
    J("memsetAsync", [c_int64, c_int64, c_int32, c_int64])(jni.env, None, stream, dC, 0, N * M * 4)
    J("memcpyAsyncDeviceToDevice", [c_int64, c_int64, c_int64, c_int64])(jni.env, None, stream, dC, dA, N * K * 4)
    J("streamSynchronize__J", [c_int64])(jni.env, None, stream)
    J("eventSync_1Del", [c_int64])(jni.env, None, ev1)
    J("deleteEvent", [c_int64])(jni.env, None, ev0)
    free = J("free", [c_int64])
    for ptr in (dA, dB, dC, d2):
        free(jni.env, None, ptr)
    J("deleteStream___3JI", [c_void_p, c_int32])(jni.env, None, ARRAY_HANDLE, 2)
    assert jni.thrown is None, jni.log[-3:]
    assert J("getLastExceptionType", [], c_int32)(jni.env, None) == 0
    pkg.cu32.read_status()
