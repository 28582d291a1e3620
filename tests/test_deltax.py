"""Data gradient of the stride-1 convolution (the Cuda_dconv3D_deltaX natives that need no stride handling).

Oracle: the reference's own CPU check loop deconv3D_deltaX_img2col_s1 (Cuda_dconv3D_deltaX/test.cuh:154-196),
restated in oracle/cu32_oracle.c, plus an FP64 version.  The restatement is pinned three ways: bit for bit
against the reference routine when oracle/_ref/libref_deltax.so has been built from the reference tree, against
the forward-convolution oracle (itself pinned) through the identity
    deltaX(deltaY, W; p) = conv(deltaY, rot180(W) with channels swapped; pad = F - 1 - p),
and against hand-computed answers."""
import ctypes

import numpy as np
import pytest


def _dims(N, IH, IW, IC, OC, FH, FW, ph, pw):
    return IH + 2 * ph - FH + 1, IW + 2 * pw - FW + 1


# ------------------------------------------------------------------ CPU
def test_deltax_oracle_known_answer(O):
    # one output pixel, 1 channel in / out, 3x3 filter: deltaX is deltaY times the filter laid around the pixel
    W = np.arange(1, 10, dtype=np.float32).reshape(1, 3, 3, 1)
    dY = np.zeros((1, 3, 3, 1), np.float32); dY[0, 1, 1, 0] = 2.0
    dX = O.ref_loops.deconv3D_deltaX_img2col_s1(dY, W, 3, 3, 1, 1)
    assert np.array_equal(dX[0, :, :, 0], 2.0 * W[0, :, :, 0])
    # no padding: a 2x2 deltaY of ones against a 2x2 filter gives the full correlation on a 3x3 input
    W = np.array([[1, 2], [3, 4]], np.float32).reshape(1, 2, 2, 1)
    dX = O.ref_loops.deconv3D_deltaX_img2col_s1(np.ones((1, 2, 2, 1), np.float32), W, 3, 3, 0, 0)
    assert np.array_equal(dX[0, :, :, 0], np.array([[1, 3, 2], [4, 10, 6], [3, 7, 4]], np.float32))


@pytest.mark.parametrize("case", [(2, 6, 5, 4, 8, 3, 3, 1, 1), (1, 7, 7, 8, 4, 5, 3, 2, 0), (2, 4, 4, 4, 4, 1, 1, 0, 0),
                                  (1, 9, 8, 12, 8, 2, 4, 1, 3)])
def test_deltax_oracle_is_the_forward_oracle_on_the_rotated_filter(O, case):
    N, IH, IW, IC, OC, FH, FW, ph, pw = case
    OH, OW = _dims(*case)
    rng = np.random.default_rng(3)
    dY = rng.standard_normal((N, OH, OW, OC)).astype(np.float32)
    W = rng.standard_normal((OC, FH, FW, IC)).astype(np.float32)
    Wr = np.ascontiguousarray(W[:, ::-1, ::-1, :].transpose(3, 1, 2, 0))      # [IC][FH][FW][OC], rotated
    want64 = O.f64.conv3D(dY, Wr, IH, IW, 1, 1, FH - 1 - ph, FW - 1 - pw)
    got64 = O.f64.deconv3D_deltaX_s1(dY, W, IH, IW, ph, pw)
    assert np.abs(got64 - want64).max() <= 1e-12 * max(1.0, np.abs(want64).max())
    got32 = O.ref_loops.deconv3D_deltaX_img2col_s1(dY, W, IH, IW, ph, pw)
    assert O.frob_rel(got32, want64) <= 2e-6
    # the forward check loop of the reference (double accumulator) on the rotated filter agrees to FP32 rounding
    fwd = O.ref_loops.conv3D_img2col(dY, Wr, IH, IW, 1, 1, FH - 1 - ph, FW - 1 - pw)
    assert O.frob_rel(fwd, want64) <= 1e-6


def test_deltax_oracle_against_reference_routine_when_built(O):
    ref = O.ref_native("deltax")
    if ref is None:
        pytest.skip("oracle/_ref/libref_deltax.so not built (python oracle/build_ref.py --deltax)")
    rng = np.random.default_rng(4)
    fp = ctypes.POINTER(ctypes.c_float)
    for case in [(2, 6, 5, 4, 8, 3, 3, 1, 1), (1, 8, 8, 8, 12, 5, 5, 2, 2), (3, 5, 7, 4, 4, 1, 1, 0, 0)]:
        N, IH, IW, IC, OC, FH, FW, ph, pw = case
        OH, OW = _dims(*case)
        dY = rng.standard_normal((N, OH, OW, OC)).astype(np.float32)
        W = rng.standard_normal((OC, FH, FW, IC)).astype(np.float32)
        out = np.zeros((N, IH, IW, IC), np.float32)
        ref.ref_cpu_deconv3D_deltaX_img2col_s1(dY.ctypes.data_as(fp), OH, OW, W.ctypes.data_as(fp), FH, FW,
                                               out.ctypes.data_as(fp), IH, IW, N, IC, OC, ph, pw)
        assert np.array_equal(out, O.ref_loops.deconv3D_deltaX_img2col_s1(dY, W, IH, IW, ph, pw)), case


def test_deltax_oracle_against_golden_fixture(O, golden):
    """tests/golden/golden_deltax.npz holds the outputs of the reference's own check loop on seeded inputs."""
    data = np.load(golden.HERE / "golden_deltax.npz")
    for name, (N, IH, IW, IC, OC, FH, FW, ph, pw) in golden.DELTAX_CASES.items():
        OH, OW = IH + 2 * ph - FH + 1, IW + 2 * pw - FW + 1
        dY, W = golden.golden_inputs(name, [(N, OH, OW, OC), (OC, FH, FW, IC)])
        assert np.array_equal(O.ref_loops.deconv3D_deltaX_img2col_s1(dY, W, IH, IW, ph, pw), data[name]), name


def test_deltax_argument_errors_without_gpu(pkg):
    lib = pkg.cu32.load()
    s = (ctypes.c_int64 * 1)(0)
    P = lambda a: ctypes.cast(a, ctypes.POINTER(ctypes.c_float))
    ok = 0x10000
    f = lib.cu32_dconv3D_deltaX_s1
    #           dY  OH OW  W  FH FW  dX  IH IW  N  IC OC ph pw
    assert f(s, 1, P(ok), 8, 8, P(ok), 3, 3, P(ok), 9, 8, 2, 8, 8, 1, 1) == -2      # IH inconsistent with OH, FH, ph
    assert f(s, 1, P(ok), 8, 8, P(ok), 3, 3, P(ok), 4, 4, 2, 8, 8, 3, 3) == -5      # padding beyond the filter reach
    assert f(s, 1, None, 8, 8, P(ok), 3, 3, P(ok), 8, 8, 2, 8, 8, 1, 1) == -1
    assert f(s, 1, P(ok), 8, 8, P(ok), 3, 3, P(ok), 8, 8, 2, 6, 8, 1, 1) == -4      # IC % 4
    assert f(s, 1, P(ok), 8, 8, P(ok), 3, 3, P(ok), 8, 8, 2, 8, 6, 1, 1) == -4      # OC % 4
    assert lib.cu32_dconv3D_deltaX_s1_SGM(s, 1, P(ok), 8, 8, P(ok), 3, 3, P(ok), 8, 8, 2, 8, 8, 1, 1, 0) == -8


# ------------------------------------------------------------------ GPU
def _run(pkg, entry, dY, W, IH, IW, ph, pw, GM_slice=64):
    import gpu_util as G
    dx = pkg.cu32.Cuda_dconv3D_deltaX
    N, OH, OW, OC = dY.shape
    _, FH, FW, IC = W.shape
    ddY, dW = G.dev(dY), G.dev(W)
    out = G.Out(N * IH * IW * IC)
    s = [G.stream()]
    base = [s, 1, ddY.data_ptr(), OH, OW, dW.data_ptr(), FH, FW, out.ptr, IH, IW, N, IC, OC, ph, pw]
    if entry in ("dconv3D_deltaX_s1", "dconv3D_deltaX_s1_texture"):
        getattr(dx, entry)(*base)
    elif entry in ("dconv3D_deltaX_s1_SGM", "dconv3D_deltaX_s1_texture_SGM"):
        getattr(dx, entry)(*base, GM_slice)
    elif entry == "dconv3D_deltaX_V2_s1":
        dx.dconv3D_deltaX_V2_s1(True, *base)
    elif entry in ("Im2col_Winograd_s8_texture", "Im2col_Winograd_s16_texture"):
        assert getattr(dx, entry)(True, *base) is True
    elif entry in ("Im2col_Winograd_s8_texture_SGM", "Im2col_Winograd_s16_texture_SGM"):
        assert getattr(dx, entry)(False, *base, GM_slice) is True
    elif entry in ("dconv3D_deltaX_W1", "dconv3D_deltaX_W1_SGM"):
        args = [s, 1, ddY.data_ptr(), dW.data_ptr(), out.ptr, IH, IW, N, IC, OC]
        getattr(dx, entry)(*(args + ([GM_slice] if entry.endswith("SGM") else [])))
    else:
        raise ValueError(entry)
    Y = out.host((N, IH, IW, IC))
    G.check_status(pkg)
    return Y


DX_CASES = [
    # N, IH, IW, IC, OC, FH, FW, ph, pw
    (4, 9, 9, 8, 12, 3, 3, 1, 1),
    (4, 28, 28, 64, 64, 3, 3, 1, 1),
    (8, 14, 14, 256, 32, 3, 3, 1, 1),
    (2, 11, 10, 4, 8, 5, 3, 2, 1),
    (2, 32, 32, 16, 36, 7, 7, 3, 3),
    (4, 10, 10, 16, 8, 3, 3, 0, 0),
    (3, 8, 12, 132, 260, 2, 4, 1, 2),
]


@pytest.mark.gpu
@pytest.mark.parametrize("case", DX_CASES)
def test_deltax_s1(pkg, O, cuda, case):
    N, IH, IW, IC, OC, FH, FW, ph, pw = case
    OH, OW = _dims(*case)
    rng = np.random.default_rng(61)
    dY = rng.standard_normal((N, OH, OW, OC)).astype(np.float32)
    W = (rng.standard_normal((OC, FH, FW, IC)) * np.sqrt(2.0 / (FH * FW * OC))).astype(np.float32)
    got = _run(pkg, "dconv3D_deltaX_s1", dY, W, IH, IW, ph, pw)
    rep = O.report(got, O.f64.deconv3D_deltaX_s1(dY, W, IH, IW, ph, pw))
    assert rep["frob"] <= 1e-6 and rep["elem"] <= 1e-4, (case, rep)
    if N * IH * IW * IC * OC * FH * FW <= 40e6:
        assert O.frob_rel(got, O.ref_loops.deconv3D_deltaX_img2col_s1(dY, W, IH, IW, ph, pw)) <= 2e-6


@pytest.mark.gpu
def test_deltax_entry_point_aliases_and_W1(pkg, O, cuda):
    rng = np.random.default_rng(62)
    N, IH, IW, IC, OC, FH, FW, ph, pw = 4, 12, 14, 24, 40, 3, 3, 1, 1
    OH, OW = _dims(N, IH, IW, IC, OC, FH, FW, ph, pw)
    dY = rng.standard_normal((N, OH, OW, OC)).astype(np.float32)
    W = rng.standard_normal((OC, FH, FW, IC)).astype(np.float32) * 0.1
    base = _run(pkg, "dconv3D_deltaX_s1", dY, W, IH, IW, ph, pw)
    for entry in ("dconv3D_deltaX_s1_texture", "dconv3D_deltaX_s1_SGM", "dconv3D_deltaX_s1_texture_SGM",
                  "dconv3D_deltaX_V2_s1", "Im2col_Winograd_s8_texture", "Im2col_Winograd_s8_texture_SGM",
                  "Im2col_Winograd_s16_texture", "Im2col_Winograd_s16_texture_SGM"):
        assert np.array_equal(_run(pkg, entry, dY, W, IH, IW, ph, pw), base), entry
    W1 = rng.standard_normal((OC, 1, 1, IC)).astype(np.float32)
    dY1 = rng.standard_normal((N, IH, IW, OC)).astype(np.float32)
    want = O.f64.deconv3D_deltaX_s1(dY1, W1, IH, IW, 0, 0)
    for entry in ("dconv3D_deltaX_W1", "dconv3D_deltaX_W1_SGM"):
        rep = O.report(_run(pkg, entry, dY1, W1, IH, IW, 0, 0), want)
        assert rep["frob"] <= 1e-6 and rep["elem"] <= 1e-4, (entry, rep)


@pytest.mark.gpu
@pytest.mark.parametrize("tile", [0, 1, 2, 3, 4, 8])
def test_deltax_every_tile_same_bits(pkg, O, cuda, tile):
    rng = np.random.default_rng(63)
    N, IH, IW, IC, OC, FH, FW, ph, pw = 4, 20, 20, 136, 72, 3, 3, 1, 1
    OH, OW = _dims(N, IH, IW, IC, OC, FH, FW, ph, pw)
    dY = rng.standard_normal((N, OH, OW, OC)).astype(np.float32)
    W = rng.standard_normal((OC, FH, FW, IC)).astype(np.float32) * 0.05
    pkg.cu32.tune("tile", 4)
    base = _run(pkg, "dconv3D_deltaX_s1", dY, W, IH, IW, ph, pw)
    rep = O.report(base, O.f64.deconv3D_deltaX_s1(dY, W, IH, IW, ph, pw))
    assert rep["frob"] <= 1e-6, rep
    pkg.cu32.tune("tile", tile)
    for _ in range(6):
        assert np.array_equal(_run(pkg, "dconv3D_deltaX_s1", dY, W, IH, IW, ph, pw), base), tile


@pytest.mark.gpu
def test_deltax_is_the_gradient_of_the_forward_entry_point(pkg, O, cuda):
    """<conv(X, W), dY> == <X, deltaX(dY, W)>: the two entry points are adjoint to each other."""
    import gpu_util as G
    rng = np.random.default_rng(64)
    N, IH, IW, IC, OC, FH, FW, ph, pw = 3, 13, 11, 16, 24, 3, 5, 1, 2
    OH, OW = _dims(N, IH, IW, IC, OC, FH, FW, ph, pw)
    X = rng.standard_normal((N, IH, IW, IC)).astype(np.float32)
    W = rng.standard_normal((OC, FH, FW, IC)).astype(np.float32) * 0.1
    dY = rng.standard_normal((N, OH, OW, OC)).astype(np.float32)
    Y = G.conv(pkg, "conv3D_GemmR", X, W, 1, 1, ph, pw)
    dX = _run(pkg, "dconv3D_deltaX_s1", dY, W, IH, IW, ph, pw)
    lhs = float((Y.astype(np.float64) * dY).sum()); rhs = float((X.astype(np.float64) * dX).sum())
    assert abs(lhs - rhs) <= 1e-5 * max(abs(lhs), abs(rhs), 1.0), (lhs, rhs)


@pytest.mark.gpu
def test_deltax_against_reference_kernels(pkg, O, cuda):
    import gpu_util as G
    torch = cuda
    ref = O.ref_native("deltax")
    if ref is None:
        pytest.skip("oracle/_ref/libref_deltax.so not built (python oracle/build_ref.py --deltax)")
    rng = np.random.default_rng(65)
    N, IH, IW, IC, OC, FH, FW, ph, pw = 8, 28, 28, 64, 64, 3, 3, 1, 1
    OH, OW = _dims(N, IH, IW, IC, OC, FH, FW, ph, pw)
    dY = rng.standard_normal((N, OH, OW, OC)).astype(np.float32)
    W = rng.standard_normal((OC, FH, FW, IC)).astype(np.float32) * 0.05
    ddY, dW = G.dev(dY), G.dev(W)
    dR = torch.zeros((N, IH, IW, IC), device="cuda")
    streams = (ctypes.c_longlong * 10)(*([G.stream()] * 10))
    vp = lambda t: ctypes.c_void_p(t.data_ptr())
    assert ref.ref_gpu_dconv3D_deltaX_s1(streams, 10, vp(ddY), OH, OW, vp(dW), FH, FW, vp(dR), IH, IW, N, IC, OC, ph, pw) == 0
    torch.cuda.synchronize()
    R = dR.cpu().numpy()
    got = _run(pkg, "dconv3D_deltaX_s1", dY, W, IH, IW, ph, pw)
    want = O.f64.deconv3D_deltaX_s1(dY, W, IH, IW, ph, pw)
    e_ref, e_our = O.frob_rel(R, want), O.frob_rel(got, want)
    assert e_ref <= 5e-6, e_ref
    assert e_our <= 1e-6 and O.frob_rel(got, R) <= 5e-6, (e_our, e_ref)


@pytest.mark.gpu
def test_deltax_against_golden_fixture(pkg, O, cuda, golden):
    data = np.load(golden.HERE / "golden_deltax.npz")
    for name, (N, IH, IW, IC, OC, FH, FW, ph, pw) in golden.DELTAX_CASES.items():
        OH, OW = IH + 2 * ph - FH + 1, IW + 2 * pw - FW + 1
        dY, W = golden.golden_inputs(name, [(N, OH, OW, OC), (OC, FH, FW, IC)])
        entry = "dconv3D_deltaX_W1" if (FH, FW) == (1, 1) else "dconv3D_deltaX_s1"
        got = _run(pkg, entry, dY, W, IH, IW, ph, pw)
        assert O.frob_rel(got, data[name]) <= 2e-6, name          # the golden output carries FP32 accumulation error
        assert O.same_percent(got, data[name], 1e-5) >= 0.999, name  # the reference's own gate, non-negative inputs


@pytest.mark.gpu
def test_conv_layer_forward_and_data_gradient_through_the_engine_mirror(pkg, O, cuda):
    import gpu_util as G
    torch = cuda
    keep = []

    def malloc(n):
        t = torch.empty(n, device="cuda")
        keep.append(t)
        return t.data_ptr(), t
    eng = pkg.engine.Cu32Engine(148, malloc, [G.stream()])
    rng = np.random.default_rng(66)
    for (N, IH, IW, IC, OC, F, p) in [(4, 14, 14, 32, 64, 3, 1), (4, 10, 10, 16, 24, 1, 0)]:
        OH, OW = IH + 2 * p - F + 1, IW + 2 * p - F + 1
        X = rng.standard_normal((N, IH, IW, IC)).astype(np.float32)
        W = (rng.standard_normal((OC, F, F, IC)) * 0.1).astype(np.float32)
        dY = rng.standard_normal((N, OH, OW, OC)).astype(np.float32)
        dX_, dW_, ddY = G.dev(X), G.dev(W), G.dev(dY)
        Y = G.Out(N * OH * OW * OC)
        eng.conv3D(Y.ptr, OH, OW, dX_.data_ptr(), IH, IW, dW_.data_ptr(), F, F, N, IC, OC, 1, 1, p, p)
        gX = G.Out(N * IH * IW * IC)
        eng.conv3D_deltaX(gX.ptr, IH, IW, ddY.data_ptr(), OH, OW, dW_.data_ptr(), F, F, N, IC, OC, 1, 1, p, p)
        G.check_status(pkg)
        for name, got, want in (("forward", Y.host((N, OH, OW, OC)), O.f64.conv3D(X, W, OH, OW, 1, 1, p, p)),
                                ("deltaX", gX.host((N, IH, IW, IC)), O.f64.deconv3D_deltaX_s1(dY, W, IH, IW, p, p))):
            rep = O.report(got, want)
            assert rep["frob"] <= 1e-6 and rep["elem"] <= 1e-4, (name, F, rep)
    with pytest.raises(NotImplementedError):
        eng.conv3D_deltaX(0, 8, 8, 0, 4, 4, 0, 3, 3, 1, 4, 4, 2, 2, 1, 1)
