"""The Java_* exports, driven through a fake JNIEnv built with ctypes.

A JNIEnv is a pointer to a pointer to a table of function pointers.  The shim uses five
entries (FindClass 6, Throw 13, NewObjectA 30, GetMethodID 33, GetLongArrayRegion 204 - the
indices of the JNI specification's function table); the fake fills exactly those, so a call
through any other slot would crash the test rather than pass silently."""
import ctypes
from ctypes import CFUNCTYPE, POINTER, c_char_p, c_int32, c_int64, c_void_p

import numpy as np
import pytest


class FakeJNI:
    def __init__(self, streams):
        self.streams = list(streams)
        self.log = []
        self.thrown = None
        table = (c_void_p * 230)()
        self._keep = []

        def put(idx, proto, fn):
            cb = proto(fn)
            self._keep.append(cb)
            table[idx] = ctypes.cast(cb, c_void_p).value

        def find_class(env, name):
            self.log.append(("FindClass", name.decode()))
            return 0x1111

        def get_method_id(env, cls, name, sig):
            self.log.append(("GetMethodID", cls, name.decode(), sig.decode()))
            return 0x2222

        def new_object_a(env, cls, mid, args):
            code = ctypes.cast(args, POINTER(c_int32))[0]   # jvalue.i of the first argument
            self.log.append(("NewObjectA", cls, mid, code))
            return 0x3333

        def throw(env, obj):
            self.thrown = obj
            self.log.append(("Throw", obj))
            return 0

        def get_long_array_region(env, arr, start, length, buf):
            self.log.append(("GetLongArrayRegion", arr, start, length))
            for i in range(length):
                buf[i] = self.streams[start + i]

        put(6, CFUNCTYPE(c_void_p, c_void_p, c_char_p), find_class)
        put(13, CFUNCTYPE(c_int32, c_void_p, c_void_p), throw)
        put(30, CFUNCTYPE(c_void_p, c_void_p, c_void_p, c_void_p, c_void_p), new_object_a)
        put(33, CFUNCTYPE(c_void_p, c_void_p, c_void_p, c_char_p, c_char_p), get_method_id)
        put(204, CFUNCTYPE(None, c_void_p, c_void_p, c_int32, c_int32, POINTER(c_int64)), get_long_array_region)
        self.table = table
        self.table_ptr = c_void_p(ctypes.addressof(table))
        self.env = ctypes.pointer(self.table_ptr)      # JNIEnv* : pointer to pointer to table


ARRAY_HANDLE = 0xABCD


def _fn(lib, name, argtypes):
    f = getattr(lib, "Java_z_dragon_engine_cuda_impl_math_Cuda_1" + name)
    f.argtypes = [c_void_p, c_void_p] + argtypes
    f.restype = None
    return f


MATMUL_ARGS = [c_void_p, c_int32, c_int64, c_int64, c_int64, c_int32, c_int32, c_int32]


def test_error_becomes_cuda_exception(pkg):
    """Argument errors are detected before any CUDA call, so this runs without a GPU: the shim
    must construct z.dragon.engine.cuda.impl.CudaException(int) and Throw it
    (reference: Cuda_matMul/JNITool.cuh:9-26)."""
    lib = pkg.cu32.load()
    jni = FakeJNI([0])
    f = _fn(lib, "matMul_matMul", MATMUL_ARGS)
    f(jni.env, None, ARRAY_HANDLE, 1, 0x10000, 0x10000, 0x10000, 0, 4, 4)   # N = 0
    assert ("GetLongArrayRegion", ARRAY_HANDLE, 0, 1) in jni.log
    assert ("FindClass", "z/dragon/engine/cuda/impl/CudaException") in jni.log
    assert ("GetMethodID", 0x1111, "<init>", "(I)V") in jni.log
    assert ("NewObjectA", 0x1111, 0x2222, -2) in jni.log
    assert jni.thrown == 0x3333
    # a stream-array length outside 1..10 is rejected without touching the array
    jni = FakeJNI([0])
    f(jni.env, None, ARRAY_HANDLE, 11, 0x10000, 0x10000, 0x10000, 4, 4, 4)
    assert not any(e[0] == "GetLongArrayRegion" for e in jni.log)
    assert ("NewObjectA", 0x1111, 0x2222, -3) in jni.log
    # SKbuf_summary takes a single stream handle, no array
    g = _fn(lib, "matMul_SKbuf_1summary", [c_int64, c_int64, c_int64, c_int32, c_int32])
    jni = FakeJNI([0])
    g(jni.env, None, 0, 0x10000, 0, 3, 8)
    assert ("NewObjectA", 0x1111, 0x2222, -1) in jni.log


@pytest.mark.gpu
def test_jni_matmul_and_conv_on_gpu(pkg, O, cuda):
    import gpu_util as G
    torch = cuda
    lib = pkg.cu32.load()
    jni = FakeJNI([G.stream()])
    N, M, K = 132, 260, 96
    A, B = G.rand_pm1((N, K), 1), G.rand_pm1((K, M), 2)
    dA, dB = G.dev(A), G.dev(B)
    out = G.Out(N * M)
    _fn(lib, "matMul_matMul", MATMUL_ARGS)(jni.env, None, ARRAY_HANDLE, 1, dA.data_ptr(), dB.data_ptr(), out.ptr, N, M, K)
    C = out.host((N, M))
    assert jni.thrown is None
    rep = O.report(C, O.f64.matMul(A, B))
    assert rep["frob"] <= 1e-6 and rep["elem"] <= 1e-4, rep
    # batched, through the JNI symbol
    Batch, L, D = 3, 64, 32
    Q = np.random.default_rng(1).standard_normal((Batch, L, D)).astype(np.float32)
    Kt = np.random.default_rng(2).standard_normal((Batch, L, D)).astype(np.float32)
    dQ, dK = G.dev(Q), G.dev(Kt)
    out = G.Out(Batch * L * L)
    _fn(lib, "batchMatMul_batchMatMulT2", [c_void_p, c_int32, c_int64, c_int64, c_int64] + [c_int32] * 5)(
        jni.env, None, ARRAY_HANDLE, 1, dQ.data_ptr(), dK.data_ptr(), out.ptr, Batch, L, L, L, D)
    rep = O.report(out.host((Batch, L, L)), O.f64.batchMatMulT2(Q, Kt))
    assert rep["frob"] <= 1e-6, rep
    # convolution: kernel_remode + conv3D_GemmR
    X = np.random.default_rng(3).standard_normal((4, 8, 8, 16)).astype(np.float32)
    W = np.random.default_rng(4).standard_normal((8, 3, 3, 16)).astype(np.float32) * 0.1
    dX, dW = G.dev(X), G.dev(W)
    dCW = torch.empty(W.size, device="cuda")
    _fn(lib, "conv3D_kernel_1remode", [c_int64, c_int64, c_int64] + [c_int32] * 4)(
        jni.env, None, G.stream(), dW.data_ptr(), dCW.data_ptr(), 3, 3, 8, 16)
    out = G.Out(4 * 8 * 8 * 8)
    _fn(lib, "conv3D_conv3D_1GemmR", [c_void_p, c_int32, c_int64, c_int32, c_int32, c_int64, c_int64, c_int32, c_int32,
                                     c_int64] + [c_int32] * 9)(
        jni.env, None, ARRAY_HANDLE, 1, dX.data_ptr(), 8, 8, dW.data_ptr(), dCW.data_ptr(), 3, 3, out.ptr, 8, 8, 4, 16, 8,
        1, 1, 1, 1)
    rep = O.report(out.host((4, 8, 8, 8)), O.f64.conv3D(X, W, 8, 8, 1, 1, 1, 1))
    assert jni.thrown is None and rep["frob"] <= 1e-6, rep
    # an Im2col-Winograd native: jboolean "handled" comes back true, same bits as conv3D_GemmR
    base = out.host((4, 8, 8, 8)).copy()
    out2 = G.Out(4 * 8 * 8 * 8)
    wino = _fn(lib, "conv3D_conv3D_1Im2col_1Winograd_1s8_1R_1texture",
               [ctypes.c_uint8, c_void_p, c_int32, c_int64, c_int32, c_int32, c_int64, c_int64, c_int32, c_int32, c_int64]
               + [c_int32] * 7)
    wino.restype = ctypes.c_uint8
    handled = wino(jni.env, None, 1, ARRAY_HANDLE, 1, dX.data_ptr(), 8, 8, dW.data_ptr(), dCW.data_ptr(), 3, 3, out2.ptr,
                   8, 8, 4, 16, 8, 1, 1)
    assert handled == 1 and jni.thrown is None
    assert np.array_equal(out2.host((4, 8, 8, 8)), base)
    torch.cuda.synchronize()
    assert np.array_equal(dCW.cpu().numpy().reshape(3, 3, 16, 8), O.ref_loops.kernel_remode(W))
    G.check_status(pkg)


@pytest.mark.gpu
def test_jni_deltax_on_gpu(pkg, O, cuda):
    """The stride-1 data-gradient natives under their JNI names (class Cuda_dconv3D_deltaX)."""
    import gpu_util as G
    lib = pkg.cu32.load()
    jni = FakeJNI([G.stream()])
    rng = np.random.default_rng(9)
    N, IH, IW, IC, OC, F, p = 2, 10, 9, 8, 12, 3, 1
    dY = rng.standard_normal((N, IH, IW, OC)).astype(np.float32)
    W = rng.standard_normal((OC, F, F, IC)).astype(np.float32) * 0.1
    ddY, dW = G.dev(dY), G.dev(W)
    want = O.f64.deconv3D_deltaX_s1(dY, W, IH, IW, p, p)
    sig = [c_void_p, c_int32, c_int64, c_int32, c_int32, c_int64, c_int32, c_int32, c_int64] + [c_int32] * 7
    out = G.Out(N * IH * IW * IC)
    f = getattr(lib, "Java_z_dragon_engine_cuda_impl_math_Cuda_1dconv3D_1deltaX_dconv3D_1deltaX_1s1")
    f.argtypes = [c_void_p, c_void_p] + sig
    f.restype = None
    f(jni.env, None, ARRAY_HANDLE, 1, ddY.data_ptr(), IH, IW, dW.data_ptr(), F, F, out.ptr, IH, IW, N, IC, OC, p, p)
    base = out.host((N, IH, IW, IC)).copy()
    rep = O.report(base, want)
    assert jni.thrown is None and rep["frob"] <= 1e-6, rep
    out2 = G.Out(N * IH * IW * IC)
    w = getattr(lib, "Java_z_dragon_engine_cuda_impl_math_Cuda_1dconv3D_1deltaX_Im2col_1Winograd_1s8_1texture")
    w.argtypes = [c_void_p, c_void_p, ctypes.c_uint8] + sig
    w.restype = ctypes.c_uint8
    assert w(jni.env, None, 1, ARRAY_HANDLE, 1, ddY.data_ptr(), IH, IW, dW.data_ptr(), F, F, out2.ptr, IH, IW, N, IC, OC,
             p, p) == 1
    assert np.array_equal(out2.host((N, IH, IW, IC)), base)
    # an impossible geometry becomes a CudaException(-2), nothing is launched
    f(jni.env, None, ARRAY_HANDLE, 1, ddY.data_ptr(), IH, IW, dW.data_ptr(), F, F, out.ptr, 0, IW, N, IC, OC, p, p)
    assert ("NewObjectA", 0x1111, 0x2222, -2) in jni.log and jni.thrown == 0x3333
    G.check_status(pkg)


@pytest.mark.gpu
def test_jni_strided_deltax_on_gpu(pkg, O, cuda):
    """The engine's sequence for strides > 1 under the JNI names: ks_remodev2, then a kernel-split native."""
    import gpu_util as G
    import torch
    lib = pkg.cu32.load()
    jni = FakeJNI([G.stream()])
    rng = np.random.default_rng(10)
    N, IH, IW, IC, OC, F, p, st = 2, 13, 12, 8, 12, 3, 1, 2
    OH, OW = (IH + 2 * p - F) // st + 1, (IW + 2 * p - F) // st + 1
    dY = rng.standard_normal((N, OH, OW, OC)).astype(np.float32)
    W = rng.standard_normal((OC, F, F, IC)).astype(np.float32) * 0.1
    ddY, dW = G.dev(dY), G.dev(W)
    want = O.f64.deconv3D_deltaX(dY, W, IH, IW, st, st, p, p)
    CF = (F + st - 1) // st
    dCW = torch.zeros(st * st * OC * CF * CF * IC, device="cuda")
    pre = "Java_z_dragon_engine_cuda_impl_math_Cuda_1dconv3D_1deltaX_"
    r = getattr(lib, pre + "ks_1remodev2")
    r.argtypes = [c_void_p, c_void_p, c_int64, c_int64, c_int32, c_int32, c_int64] + [c_int32] * 6
    r.restype = None
    r(jni.env, None, G.stream(), dW.data_ptr(), F, F, dCW.data_ptr(), CF, CF, OC, IC, st, st)
    assert jni.thrown is None
    head = [c_void_p, c_void_p, c_void_p, c_int32, c_int64, c_int32, c_int32, c_int64, c_int32, c_int32, c_int64]
    results = []
    for name, lead, tail in (("dconv3D_1deltaX_1kernelSplit", [], [st, st, p, p]),
                             ("dconv3D_1deltaX_1ksIms2R_1texture", [], [p, p]),
                             ("dconv3D_1deltaX_1ksImsR_1SGM", [], [st, st, p, p, 64]),
                             ("dconv3D_1deltaX_1ksV2_1Ims2R", [1], [p, p])):
        f = getattr(lib, pre + name)
        f.argtypes = head[:2] + [ctypes.c_uint8] * len(lead) + head[2:] + [c_int32] * (5 + len(tail))
        f.restype = None
        out = G.Out(N * IH * IW * IC)
        f(jni.env, None, *lead, ARRAY_HANDLE, 1, ddY.data_ptr(), OH, OW, dCW.data_ptr(), F, F, out.ptr, IH, IW, N, IC,
          OC, *tail)
        assert jni.thrown is None, name
        results.append(out.host((N, IH, IW, IC)).copy())
        assert O.report(results[-1], want)["frob"] <= 1e-6, name
        assert np.array_equal(results[-1], results[0]), name
    # scatter-add name, forward filter as it lies
    c = getattr(lib, pre + "dconv3D_1deltaX_1crossAdd")
    c.argtypes = head + [c_int32] * 9
    c.restype = None
    out = G.Out(N * IH * IW * IC)
    c(jni.env, None, ARRAY_HANDLE, 1, ddY.data_ptr(), OH, OW, dW.data_ptr(), F, F, out.ptr, IH, IW, N, IC, OC, st, st, p, p)
    assert jni.thrown is None and np.array_equal(out.host((N, IH, IW, IC)), results[0])
    G.check_status(pkg)


@pytest.mark.gpu
def test_jni_deltaw_on_gpu(pkg, O, cuda):
    """The engine's split-K sequence for the weight gradient under the JNI names of class Cuda_dconv3D_deltaW."""
    import gpu_util as G
    import torch
    lib = pkg.cu32.load()
    jni = FakeJNI([G.stream()])
    rng = np.random.default_rng(11)
    N, IH, IW, IC, OC, F, p, GZ = 3, 9, 8, 8, 12, 3, 1, 3
    X = rng.standard_normal((N, IH, IW, IC)).astype(np.float32)
    dY = rng.standard_normal((N, IH, IW, OC)).astype(np.float32)
    dX_, ddY = G.dev(X), G.dev(dY)
    want = O.f64.deconv3D_deltaW(X, dY, F, F, 1, 1, p, p)
    size = OC * F * F * IC
    buf = torch.full(((GZ - 1) * size,), float("nan"), device="cuda")
    pre = "Java_z_dragon_engine_cuda_impl_math_Cuda_1dconv3D_1deltaW_"
    f = getattr(lib, pre + "dconv3D_1deltaW_1GemmSK")
    f.argtypes = [c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int64, c_int32, c_int32, c_int64, c_int32, c_int32,
                  c_int64, c_int64] + [c_int32] * 9
    f.restype = None
    sm = getattr(lib, pre + "buf_1summary")
    sm.argtypes = [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int32, c_int32]
    sm.restype = None
    out = G.Out(size)
    f(jni.env, None, ARRAY_HANDLE, 1, GZ, dX_.data_ptr(), IH, IW, ddY.data_ptr(), IH, IW, out.ptr, buf.data_ptr(), F, F,
      N, IC, OC, 1, 1, p, p)
    sm(jni.env, None, G.stream(), buf.data_ptr(), out.ptr, GZ - 1, size)
    assert jni.thrown is None
    base = out.host((OC, F, F, IC)).copy()
    assert O.report(base, want)["frob"] <= 1e-6
    w = getattr(lib, pre + "Im2col_1WinogradV2_1SHW_1s8_1texture")
    w.argtypes = [c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32, c_int64, c_int32, c_int32, c_int64,
                  c_int32, c_int32, c_int64, c_int64] + [c_int32] * 8
    w.restype = ctypes.c_uint8
    out2 = G.Out(size)
    assert w(jni.env, None, ARRAY_HANDLE, 1, GZ, IH, IW, dX_.data_ptr(), IH, IW, ddY.data_ptr(), IH, IW, out2.ptr,
             buf.data_ptr(), F, F, N, IC, OC, p, p, 6) == 1
    sm(jni.env, None, G.stream(), buf.data_ptr(), out2.ptr, GZ - 1, size)
    assert np.array_equal(out2.host((OC, F, F, IC)), base)
    # an impossible geometry becomes a CudaException(-2)
    f(jni.env, None, ARRAY_HANDLE, 1, GZ, dX_.data_ptr(), IH, IW, ddY.data_ptr(), 0, IW, out.ptr, buf.data_ptr(), F, F,
      N, IC, OC, 1, 1, p, p)
    assert ("NewObjectA", 0x1111, 0x2222, -2) in jni.log and jni.thrown == 0x3333
    G.check_status(pkg)


def test_refused_boolean_native_returns_false_without_an_exception(pkg):
    """The Java engine tries the Winograd natives inside an else-if chain (`algo == X && native(...)`,
    CudaFloat32EngineBase.java:2603-2616) and falls through to the general native on false, so a shape
    this library refuses must come back as a plain false with no exception pending."""
    lib = pkg.cu32.load()
    jni = FakeJNI([0])
    f = getattr(lib, "Java_z_dragon_engine_cuda_impl_math_Cuda_1conv3D_conv3D_1Im2col_1Winograd_1s8_1R_1texture")
    f.argtypes = [c_void_p, c_void_p, ctypes.c_uint8, c_void_p, c_int32, c_int64, c_int32, c_int32, c_int64, c_int64,
                  c_int32, c_int32, c_int64] + [c_int32] * 7
    f.restype = ctypes.c_uint8
    # IC = 6 is not a multiple of 4: refused with CU32_E_ALIGN before any CUDA call
    handled = f(jni.env, None, 1, ARRAY_HANDLE, 1, 0x10000, 8, 8, 0x10000, 0x10000, 3, 3, 0x10000, 8, 8, 4, 6, 8, 1, 1)
    assert handled == 0
    assert jni.thrown is None and not any(e[0] in ("FindClass", "NewObjectA", "Throw") for e in jni.log)


def test_kernel_status_native_is_exported(pkg):
    lib = pkg.cu32.load()
    assert hasattr(lib, "Java_z_dragon_engine_cuda_impl_math_Cuda_1matMul_kernelStatus")
