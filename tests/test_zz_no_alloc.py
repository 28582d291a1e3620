"""The allocation-free split-K entry point, cu32_matMulT1SK_noalloc.

Some hosts cannot hand the library a partial buffer: their device-memory pool is exhausted or
they must not allocate (and thereby synchronise the device) at that point.  For them the library
keeps the split-K partial products in a fixed scratch array of its own.  This test calls the
entry point through the C ABI twice in a row - different shapes and inputs, so the second call
runs over the first call's leftovers - and checks each result against the existing pair
cu32_matMulT1SK + cu32_SKbuf_summary on a caller buffer (same kernels, same order of adds:
the results must be identical; the tolerance of the parity tests is asserted as well), and
against the FP64 oracle.  It also checks that a request beyond the scratch capacity is refused.

Collected last on purpose (file name): a failure here cannot hide the other GPU tests."""
import ctypes

import numpy as np
import pytest

SCRATCH_FLOATS = 4 * 1024 * 1024


def _call_noalloc(pkg, G, A, B, N, M, K, GZ):
    lib = pkg.cu32.load()
    fp = ctypes.POINTER(ctypes.c_float)
    dA, dB = G.dev(A), G.dev(B)
    out = G.Out(N * M)
    s = (ctypes.c_int64 * 10)(G.stream())
    cast = lambda p: ctypes.cast(ctypes.c_void_p(p), fp)
    rc = lib.cu32_matMulT1SK_noalloc(s, 1, GZ, cast(dA.data_ptr()), cast(dB.data_ptr()), cast(out.ptr), N, M, K)
    assert rc == 0, rc
    C = out.host((N, M))
    G.check_status(pkg)
    return C


@pytest.mark.gpu
def test_noalloc_matches_caller_buffer_path_twice(pkg, O, cuda):
    import gpu_util as G
    cases = [(132, 260, 4100, 8, 61), (256, 128, 2048, 16, 62)]   # N, M, K, GridZ, seed
    for N, M, K, GZ, seed in cases:
        A, B = G.rand_pm1((K, N), seed), G.rand_pm1((K, M), seed + 100)
        C = _call_noalloc(pkg, G, A, B, N, M, K, GZ)
        want, _, _ = G.matmul_sk(pkg, "T1", A, B, N, M, K, GZ)
        assert np.array_equal(C, want), f"{N}x{M}x{K} GridZ={GZ}"
        rep = O.report(C, O.f64.matMulT1(A, B))
        assert rep["frob"] <= 1e-6 and rep["elem"] <= 1e-4, rep
        assert O.frob_rel(C, want) <= 1e-6


def test_noalloc_refuses_oversized_request(pkg):
    # argument checks come before any CUDA call, so this part also runs without a GPU
    lib = pkg.cu32.load()
    fp = ctypes.POINTER(ctypes.c_float)
    fake = ctypes.cast(ctypes.c_void_p(0x10000), fp)
    s = (ctypes.c_int64 * 10)()
    N = M = 1024
    GZ = SCRATCH_FLOATS // (N * M) + 2          # (GZ-1)*N*M just over the capacity
    assert lib.cu32_matMulT1SK_noalloc(s, 1, GZ, fake, fake, fake, N, M, 8192) == -9
    assert lib.cu32_matMulT1SK_noalloc(s, 1, 0, fake, fake, fake, N, M, 8192) == -8
    assert lib.cu32_matMulT1SK_noalloc(s, 0, 2, fake, fake, fake, N, M, 8192) == -3
