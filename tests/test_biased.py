"""Contraction + bias row in one pass (the fusion of the engine's matMul_biased / conv3D_biased).

The oracle is the two-step sequence the Java engine runs: the contraction, then
Cuda_function.linear_dual2D_row(C, Bias, row_lengthv, 1, 1, 0, C, lengthv, width, stride)
(CudaFloat32EngineBase.java:1594-1688, :2389-2542; Cuda_function/type1_linear_dual2D_row.cuh:41-70).
The fused entry points must return the same bits as this library's contraction followed by the
restated bias kernel, and meet the FP64 tolerance of the contraction itself."""
import ctypes

import numpy as np
import pytest


# ------------------------------------------------------------------ CPU: the restated bias kernel
def test_linear_dual2D_row_oracle_known_answers(O):
    X1 = np.arange(24, dtype=np.float32).reshape(3, 8) * 0.5
    X2 = np.array([1, -2, 3, -4, 5, -6, 7, -8], np.float32)
    Y = O.ref_loops.linear_dual2D_row(X1, X2, 1.0, 1.0, 0.0, 6)
    want = X1 + X2
    want[:, 6:] = 0          # padding columns of the [height][stride] matrix are zeroed
    assert np.array_equal(Y, want)
    # general coefficients
    Y = O.ref_loops.linear_dual2D_row(X1, X2, 2.0, -0.5, 0.25, 8)
    assert np.array_equal(Y, (np.float32(2) * X1 + np.float32(-0.5) * X2) + np.float32(0.25))
    # with (1, 1, 0) the result is the single rounding of the exact sum
    rng = np.random.default_rng(5)
    X1 = rng.standard_normal((7, 12)).astype(np.float32) * 1e3
    X2 = rng.standard_normal(12).astype(np.float32)
    Y = O.ref_loops.linear_dual2D_row(X1, X2, 1.0, 1.0, 0.0, 12)
    assert np.array_equal(Y, (X1.astype(np.float64) + X2.astype(np.float64)).astype(np.float32))


def test_biased_argument_errors_without_gpu(pkg):
    lib = pkg.cu32.load()
    s = (ctypes.c_int64 * 1)(0)
    P = lambda a: ctypes.cast(a, ctypes.POINTER(ctypes.c_float))
    ok = 0x10000
    f = lib.cu32_matMul_biased
    assert f(s, 1, P(ok), P(ok), P(ok), None, 8, 8, 8, 8) == -1           # null bias
    assert f(s, 1, P(ok), P(ok), P(ok), P(ok), 8, 8, 8, 0) == -2          # width out of range
    assert f(s, 1, P(ok), P(ok), P(ok), P(ok), 8, 8, 8, 9) == -2
    assert f(s, 1, P(ok), P(ok), P(ok), P(ok + 4), 8, 8, 8, 8) == -4      # bias not 16-byte aligned
    g = lib.cu32_SKbuf_summary_biased
    assert g(0, P(ok), P(ok), None, 1, 64, 8, 8) == -1
    assert g(0, P(ok), P(ok), P(ok), 1, 64, 8, 9) == -2                   # width > row length
    assert g(0, P(ok), P(ok), P(ok), 1, 60, 8, 8) == -2                   # sizeC not a whole number of rows
    assert g(0, P(ok), P(ok), P(ok), 1, 72, 6, 6) == -4                   # row length not a multiple of 4
    h = lib.cu32_conv3D_GemmR_biased
    assert h(s, 1, P(ok), 8, 8, P(ok), P(ok), 3, 3, P(ok), 8, 8, 2, 8, 8, 1, 1, 1, 1, None, 8) == -1


# ------------------------------------------------------------------ GPU: bit-exact against the two-step sequence
def _bias_then_pad(O, C, bias, width):
    return O.ref_loops.linear_dual2D_row(C.reshape(-1, C.shape[-1]), bias, 1.0, 1.0, 0.0, width).reshape(C.shape)


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(132, 260, 96, 258), (512, 512, 256, 512), (300, 36, 200, 33), (64, 1028, 72, 1028)])
@pytest.mark.parametrize("mma", [False, True])
def test_matmul_biased_equals_two_step_sequence(pkg, O, cuda, shape, mma):
    import gpu_util as G
    N, M, K, width = shape
    A, B = G.rand_pm1((N, K), 41), G.rand_pm1((K, M), 42)
    B[:, width:] = 0                                     # the engine keeps padding columns zero
    bias = np.zeros(M, np.float32)
    bias[:width] = np.random.default_rng(43).standard_normal(width).astype(np.float32)
    plain = G.matmul(pkg, "AB", A, B, N, M, K, mma=mma)
    want = _bias_then_pad(O, plain, bias, width)
    dA, dB, dbias = G.dev(A), G.dev(B), G.dev(bias)
    out = G.Out(N * M)
    mm = pkg.cu32.Cuda_matMul
    (mm.matMul_mma_biased if mma else mm.matMul_biased)([G.stream()], 1, dA.data_ptr(), dB.data_ptr(), out.ptr,
                                                        dbias.data_ptr(), N, M, K, width)
    got = out.host((N, M))
    G.check_status(pkg)
    assert np.array_equal(got, want)
    if not mma:
        C64 = O.f64.matMul(A, B) + bias.astype(np.float64)
        C64[:, width:] = 0
        rep = O.report(got, C64)
        assert rep["frob"] <= 1e-6 and rep["elem"] <= 1e-4, rep


@pytest.mark.gpu
@pytest.mark.parametrize("tile", [0, 1, 2, 3, 4, 5])
def test_matmul_biased_every_tile(pkg, O, cuda, tile):
    import gpu_util as G
    pkg.cu32.tune("tile", tile)
    N, M, K, width = 300, 520, 136, 517
    A, B = G.rand_pm1((N, K), 44), G.rand_pm1((K, M), 45)
    bias = G.rand_pm1((M,), 46)
    plain = G.matmul(pkg, "AB", A, B, N, M, K)
    dA, dB, dbias = G.dev(A), G.dev(B), G.dev(bias)
    out = G.Out(N * M)
    pkg.cu32.Cuda_matMul.matMul_biased([G.stream()], 1, dA.data_ptr(), dB.data_ptr(), out.ptr, dbias.data_ptr(), N, M,
                                       K, width)
    got = out.host((N, M))
    G.check_status(pkg)
    assert np.array_equal(got, _bias_then_pad(O, plain, bias, width)), tile


@pytest.mark.gpu
@pytest.mark.parametrize("part", [0, 1, 5])
def test_skbuf_summary_biased(pkg, O, cuda, part):
    import gpu_util as G
    N, M, width = 36, 40, 38
    rng = np.random.default_rng(47)
    C = rng.standard_normal((N, M)).astype(np.float32)
    Cbuf = rng.standard_normal((max(part, 1), N, M)).astype(np.float32)
    bias = rng.standard_normal(M).astype(np.float32)
    want = _bias_then_pad(O, O.ref_loops.buf_summary(Cbuf[:part], C, part, N * M).reshape(N, M), bias, width)
    dC, dCbuf, dbias = G.dev(C), G.dev(Cbuf), G.dev(bias)
    pkg.cu32.Cuda_matMul.SKbuf_summary_biased(G.stream(), dCbuf.data_ptr(), dC.data_ptr(), dbias.data_ptr(), part,
                                              N * M, M, width)
    cuda.cuda.synchronize()
    assert np.array_equal(dC.cpu().numpy(), want)


@pytest.mark.gpu
def test_splitk_then_biased_summary_matches_engine_sequence(pkg, O, cuda):
    """matMulSK + SKbuf_summary_biased == matMulSK + SKbuf_summary + linear_dual2D_row (engine :1641-1688)."""
    import gpu_util as G
    N, M, K, GZ, width = 132, 260, 2052, 4, 258
    A, B = G.rand_pm1((N, K), 48), G.rand_pm1((K, M), 49)
    bias = G.rand_pm1((M,), 50)
    C, C0, Cbuf = G.matmul_sk(pkg, "AB", A, B, N, M, K, GZ)          # summed by the plain SKbuf_summary
    want = _bias_then_pad(O, C, bias, width)
    dC, dCbuf, dbias = G.dev(C0), G.dev(Cbuf), G.dev(bias)
    pkg.cu32.Cuda_matMul.SKbuf_summary_biased(G.stream(), dCbuf.data_ptr(), dC.data_ptr(), dbias.data_ptr(), GZ - 1,
                                              N * M, M, width)
    cuda.cuda.synchronize()
    assert np.array_equal(dC.cpu().numpy(), want)


@pytest.mark.gpu
@pytest.mark.parametrize("case", [(4, 12, 12, 16, 24, 3, 3, 1, 1, 1, 1, 22), (2, 9, 9, 8, 64, 3, 3, 2, 2, 1, 1, 64),
                                  (4, 10, 10, 32, 132, 1, 1, 1, 1, 0, 0, 130)])
def test_conv_biased_equals_two_step_sequence(pkg, O, cuda, case):
    import gpu_util as G
    torch = cuda
    N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw, width = case
    rng = np.random.default_rng(51)
    X = rng.standard_normal((N, IH, IW, IC)).astype(np.float32)
    W = (rng.standard_normal((OC, FH, FW, IC)) * 0.1).astype(np.float32)
    W[width:] = 0
    bias = rng.standard_normal(OC).astype(np.float32)
    OH, OW = (IH + 2 * ph - FH) // sh + 1, (IW + 2 * pw - FW) // sw + 1
    plain = G.conv(pkg, "conv3D_GemmR", X, W, sh, sw, ph, pw)
    want = _bias_then_pad(O, plain, bias, width)
    dX, dW, dbias = G.dev(X), G.dev(W), G.dev(bias)
    dCW = torch.empty(W.size, device="cuda")
    out = G.Out(N * OH * OW * OC)
    pkg.cu32.Cuda_conv3D.conv3D_GemmR_biased([G.stream()], 1, dX.data_ptr(), IH, IW, dW.data_ptr(), dCW.data_ptr(), FH, FW,
                                             out.ptr, OH, OW, N, IC, OC, sh, sw, ph, pw, dbias.data_ptr(), width)
    got = out.host((N, OH, OW, OC))
    G.check_status(pkg)
    assert np.array_equal(got, want)


@pytest.mark.gpu
def test_fullconnect_sweep_of_the_reference_test(pkg, O, cuda):
    """The reference's fully-connected test compares fullconnect(X, W) followed by add_row with fullconnect(X, W, B)
    for every X of 1..128 x 1..128 (test/cuda/Cuda_fullconect_test.java:47-49), demanding identical values.  Here the
    same comparison at the native level for every padded extent 4..128: the fused native against the plain native
    followed by one FP32 add of the bias on the device, bit for bit, pad columns zero."""
    import gpu_util as G
    torch = cuda
    mm = pkg.cu32.Cuda_matMul
    s = [G.stream()]
    g = torch.Generator(device="cuda").manual_seed(75)
    X = torch.randn(128 * 128, device="cuda", generator=g)
    Wt = torch.randn(128 * 128, device="cuda", generator=g)
    Bv = torch.randn(128, device="cuda", generator=g)
    plain = torch.empty(128 * 128, device="cuda")
    fused = G.Out(128 * 128)
    bad = torch.zeros((), device="cuda", dtype=torch.int64)
    for N in range(4, 129, 4):
        for M in range(4, 129, 4):            # K = M, as in the reference test (W is IW x IW)
            width = M - (N // 4) % 4          # true widths 0 to 3 below the padded one
            A = X[:N * M].view(N, M)
            W = Wt[:M * M].view(M, M).clone()
            W[:, width:] = 0                  # the engine keeps pad columns of the weights at zero
            C = plain[:N * M].view(N, M)
            F = fused.view[:N * M].view(N, M)
            F.fill_(float("nan"))
            mm.matMul(s, 1, A.data_ptr(), W.data_ptr(), C.data_ptr(), N, M, M)
            mm.matMul_biased(s, 1, A.data_ptr(), W.data_ptr(), F.data_ptr(), Bv.data_ptr(), N, M, M, width)
            want = C + Bv[:M]
            want[:, width:] = 0
            bad += (F != want).sum()
    assert int(bad.item()) == 0
    fused.host((128 * 128,))   # canaries
    G.check_status(pkg)


@pytest.mark.gpu
@pytest.mark.parametrize("geom", [(3, 3, 1, 1, 1, 1), (4, 4, 2, 2, 1, 1), (5, 5, 2, 2, 2, 2)])
def test_conv_biased_channel_sweep_of_the_reference_test(pkg, O, cuda, geom):
    """The reference's biased-convolution test sweeps the output channels 1..128 on a 4 x 16 x 16 x 16 input for
    3x3 stride 1, 4x4 stride 2 and 5x5 stride 2 (test/cuda/conv3D/Cuda_conv3D_biased_test.java:68-99); the engine pads
    the count to a multiple of 4 and passes the true count as the bias width.  Every padded count 4..128 with a true
    width 0 to 3 below it: FP64 parity of the fused native, pad channels zero."""
    import gpu_util as G
    torch = cuda
    FH, FW, sh, sw, ph, pw = geom
    N, IH, IW, IC = 4, 16, 16, 16
    OH, OW = (IH + 2 * ph - FH) // sh + 1, (IW + 2 * pw - FW) // sw + 1
    rng = np.random.default_rng(73)
    X = rng.random((N, IH, IW, IC), dtype=np.float32)
    dX = G.dev(X)
    for OC in range(4, 129, 4):
        width = OC - (OC // 4) % 4
        W = rng.random((OC, FH, FW, IC), dtype=np.float32)
        W[width:] = 0.0
        bias = rng.random(OC, dtype=np.float32)
        want = O.f64.conv3D(X, W, OH, OW, sh, sw, ph, pw) + bias.astype(np.float64)
        want[..., width:] = 0.0
        dW, dbias = G.dev(W), G.dev(bias)
        dCW = torch.empty(W.size, device="cuda")
        pkg.cu32.Cuda_conv3D.kernel_remode(G.stream(), dW.data_ptr(), dCW.data_ptr(), FH, FW, OC, IC)
        out = G.Out(N * OH * OW * OC)
        pkg.cu32.Cuda_conv3D.conv3D_GemmR_biased([G.stream()], 1, dX.data_ptr(), IH, IW, dW.data_ptr(), dCW.data_ptr(), FH, FW,
                                                 out.ptr, OH, OW, N, IC, OC, sh, sw, ph, pw, dbias.data_ptr(), width)
        got = out.host((N, OH, OW, OC))
        G.check_status(pkg)
        assert not got[..., width:].any(), (geom, OC, width)
        rep = O.report(got, want)
        assert rep["frob"] <= 1e-6 and rep["elem"] <= 1e-4, (geom, OC, rep)


@pytest.mark.gpu
def test_bias_kernel_restatement_against_reference_kernel(pkg, O, cuda):
    """Pins the restated linear_dual2D_row: the reference's own kernel, compiled from the reference tree for
    sm_100a (oracle/_ref/libref_function.so), gives the same bits on the same inputs."""
    import gpu_util as G
    ref = O.ref_native("function")
    if ref is None:
        pytest.skip("oracle/_ref/libref_function.so not built")
    rng = np.random.default_rng(52)
    for (height, stride, width) in [(3, 8, 6), (40, 260, 258), (700, 132, 132), (5, 4, 1)]:
        X1 = (rng.standard_normal((height, stride)) * 100).astype(np.float32)
        X2 = rng.standard_normal(stride).astype(np.float32)
        d1, d2 = G.dev(X1), G.dev(X2)
        dY = cuda.empty((height, stride), device="cuda")
        fn = ref.ref_gpu_linear_dual2D_row
        fn.argtypes = [ctypes.c_longlong, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_float,
                       ctypes.c_float, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int]
        assert fn(G.stream(), d1.data_ptr(), d2.data_ptr(), stride, 1.0, 1.0, 0.0, dY.data_ptr(), height * stride, width,
                  stride) == 0
        cuda.cuda.synchronize()
        assert np.array_equal(dY.cpu().numpy(), O.ref_loops.linear_dual2D_row(X1, X2, 1.0, 1.0, 0.0, width))


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(256, 512, 1024), (64, 128, 32768)])
def test_fullconnect_layer_forward_and_backward_through_the_engine_mirror(pkg, O, cuda, shape):
    """One fully-connected layer the way the Java engine runs it: forward Y = X*W + b (matMul_biased, fused here),
    weight gradient dW = X^T * dY (matMulT1, split-K by the engine's rule) and data gradient dX = dY * W^T
    (matMulT2) - the contractions behind fullconnect / fullconnect_deltaW / fullconnect_deltaX
    (Engine.java:1425-1467), all through natives this library exports."""
    import gpu_util as G
    torch = cuda
    batch, IW, OW = shape            # K of the weight gradient is the batch
    keep = []

    def malloc(n):
        t = torch.empty(n, device="cuda")
        keep.append(t)
        return t.data_ptr(), t
    eng = pkg.engine.Cu32Engine(148, malloc, [G.stream()])
    g = torch.Generator().manual_seed(61)
    X = torch.randn((batch, IW), generator=g)
    W = torch.randn((IW, OW), generator=g) * 0.05
    b = torch.randn(OW, generator=g)
    dY = torch.randn((batch, OW), generator=g)
    dX_, dW_, db_, ddY = X.cuda(), W.cuda(), b.cuda(), dY.cuda()
    Y = G.Out(batch * OW)
    eng.matMul_biased(Y.ptr, dX_.data_ptr(), dW_.data_ptr(), batch, OW, IW, db_.data_ptr(), OW)
    gW = G.Out(IW * OW)
    gz = eng.matMulT1(gW.ptr, dX_.data_ptr(), ddY.data_ptr(), IW, OW, batch)
    gX = G.Out(batch * IW)
    eng.matMulT2(gX.ptr, ddY.data_ptr(), dW_.data_ptr(), batch, IW, OW)
    G.check_status(pkg)
    X64, W64, dY64 = X.double().numpy(), W.double().numpy(), dY.double().numpy()
    for name, got, want in (("forward", Y.host((batch, OW)), X64 @ W64 + b.double().numpy()),
                            ("deltaW", gW.host((IW, OW)), X64.T @ dY64),
                            ("deltaX", gX.host((batch, IW)), dY64 @ W64.T)):
        rep = O.report(got, want)
        assert rep["frob"] <= 1e-6 and rep["elem"] <= 1e-4, (name, gz, rep)
    if batch >= 32768:
        assert gz > 1          # the long-K weight gradient takes the split-K branch
