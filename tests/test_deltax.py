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
    assert f(s, 1, P(ok), 8, 8, P(ok), 3, 3, P(ok), 0, 8, 2, 8, 8, 1, 1) == -2      # no rows
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
@pytest.mark.parametrize("tile", [0, 1, 2, 3, 4, 5])
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
    for (N, IH, IW, IC, OC, F, p, st) in [(4, 14, 14, 32, 64, 3, 1, 1), (4, 10, 10, 16, 24, 1, 0, 1),
                                          (4, 14, 14, 32, 64, 3, 1, 2), (2, 15, 15, 16, 24, 5, 2, 3)]:
        OH, OW = (IH + 2 * p - F) // st + 1, (IW + 2 * p - F) // st + 1
        X = rng.standard_normal((N, IH, IW, IC)).astype(np.float32)
        W = (rng.standard_normal((OC, F, F, IC)) * 0.1).astype(np.float32)
        dY = rng.standard_normal((N, OH, OW, OC)).astype(np.float32)
        dX_, dW_, ddY = G.dev(X), G.dev(W), G.dev(dY)
        Y = G.Out(N * OH * OW * OC)
        eng.conv3D(Y.ptr, OH, OW, dX_.data_ptr(), IH, IW, dW_.data_ptr(), F, F, N, IC, OC, st, st, p, p)
        gX = G.Out(N * IH * IW * IC)
        eng.conv3D_deltaX(gX.ptr, IH, IW, ddY.data_ptr(), OH, OW, dW_.data_ptr(), F, F, N, IC, OC, st, st, p, p)
        G.check_status(pkg)
        for name, got, want in (("forward", Y.host((N, OH, OW, OC)), O.f64.conv3D(X, W, OH, OW, st, st, p, p)),
                                ("deltaX", gX.host((N, IH, IW, IC)), O.f64.deconv3D_deltaX(dY, W, IH, IW, st, st, p, p))):
            rep = O.report(got, want)
            assert rep["frob"] <= 1e-6 and rep["elem"] <= 1e-4, (name, F, st, rep)


# ================================================================== any stride
# The reference computes the data gradient of a strided convolution either by scatter-add from the forward
# filter (crossAdd) or by "kernel split": sh*sw stride-1 sub-problems over a rearranged copy CW of the filter
# that ks_remodev2 writes.  Oracle: the reference's any-stride CPU check loop (Cuda_dconv3D_deltaX/test.cuh:109-152),
# an FP64 version of it, and a restatement of the two rearrangement kernels.
def _sdims(N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw):
    return (IH + 2 * ph - FH) // sh + 1, (IW + 2 * pw - FW) // sw + 1


SDX_SMALL = [
    # N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw
    (2, 8, 8, 4, 8, 3, 3, 2, 2, 1, 1),
    (1, 11, 10, 4, 4, 5, 3, 2, 2, 2, 1),
    (2, 9, 7, 8, 4, 3, 3, 3, 3, 1, 1),
    (1, 12, 12, 4, 4, 1, 1, 2, 2, 0, 0),      # filter smaller than the stride: most pixels get no tap
    (2, 10, 13, 4, 8, 4, 4, 2, 1, 1, 2),      # stride in one direction only
    (1, 10, 10, 4, 4, 3, 3, 4, 4, 1, 1),
]


def test_strided_oracle_known_answer_and_stride_one(O):
    # 1x1 filter, stride 2: each deltaY pixel lands on the even input pixel, the others stay zero
    dY = np.arange(1, 5, dtype=np.float32).reshape(1, 2, 2, 1)
    W = np.full((1, 1, 1, 1), 3.0, np.float32)
    dX = O.ref_loops.deconv3D_deltaX_img2col(dY, W, 4, 4, 2, 2, 0, 0)
    want = np.zeros((4, 4), np.float32); want[0::2, 0::2] = 3.0 * dY[0, :, :, 0]
    assert np.array_equal(dX[0, :, :, 0], want)
    # with sh = sw = 1 the any-stride loop is the stride-1 loop, bit for bit
    rng = np.random.default_rng(8)
    for case in [(2, 6, 5, 4, 8, 3, 3, 1, 1), (1, 7, 7, 8, 4, 5, 3, 2, 0)]:
        N, IH, IW, IC, OC, FH, FW, ph, pw = case
        OH, OW = _dims(*case)
        dY = rng.standard_normal((N, OH, OW, OC)).astype(np.float32)
        W = rng.standard_normal((OC, FH, FW, IC)).astype(np.float32)
        assert np.array_equal(O.ref_loops.deconv3D_deltaX_img2col(dY, W, IH, IW, 1, 1, ph, pw),
                              O.ref_loops.deconv3D_deltaX_img2col_s1(dY, W, IH, IW, ph, pw))


@pytest.mark.parametrize("case", SDX_SMALL)
def test_strided_oracle_is_the_adjoint_of_the_forward_oracle(O, case):
    """<conv(X, W), dY> == <X, deltaX(dY, W)> for every X: checked in FP64 with the pinned forward oracle."""
    N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw = case
    OH, OW = _sdims(*case)
    rng = np.random.default_rng(9)
    X = rng.standard_normal((N, IH, IW, IC)).astype(np.float32)
    dY = rng.standard_normal((N, OH, OW, OC)).astype(np.float32)
    W = rng.standard_normal((OC, FH, FW, IC)).astype(np.float32)
    Y64 = O.f64.conv3D(X, W, OH, OW, sh, sw, ph, pw)
    dX64 = O.f64.deconv3D_deltaX(dY, W, IH, IW, sh, sw, ph, pw)
    lhs, rhs = float((Y64 * dY).sum()), float((X.astype(np.float64) * dX64).sum())
    assert abs(lhs - rhs) <= 1e-10 * max(1.0, abs(lhs))
    # and column by column: deltaX of a one-hot deltaY is the filter laid at the strided position
    got32 = O.ref_loops.deconv3D_deltaX_img2col(dY, W, IH, IW, sh, sw, ph, pw)
    assert O.frob_rel(got32, dX64) <= 2e-6


def _cw_phase(CW, W, sh, sw, y, x, v2):
    """The part of workspace CW that belongs to phase (y, x), as [CFH][CFW][OC][IC] with taps in filter order."""
    OC, FH, FW, IC = W.shape
    mCFH, mCFW = (FH + sh - 1) // sh, (FW + sw - 1) // sw
    CFH, CFW = (FH - y + sh - 1) // sh, (FW - x + sw - 1) // sw
    slot = CW[(y * sw + x) * OC * mCFH * mCFW * IC:][:OC * CFH * CFW * IC]
    if v2:
        return slot.reshape(CFH, CFW, OC, IC)[::-1, ::-1]
    return slot.reshape(OC, CFH, CFW, IC).transpose(1, 2, 0, 3)[::-1, ::-1]


@pytest.mark.parametrize("geom", [(3, 3, 2, 2), (5, 3, 2, 2), (7, 7, 2, 2), (3, 3, 3, 3), (4, 4, 2, 1), (1, 1, 2, 2),
                                  (2, 5, 3, 2)])
@pytest.mark.parametrize("v2", [True, False])
def test_ks_remode_oracle_holds_each_phase_sub_filter(O, geom, v2):
    FH, FW, sh, sw = geom
    OC, IC = 6, 4
    W = np.random.default_rng(10).standard_normal((OC, FH, FW, IC)).astype(np.float32)
    CW = O.ref_loops.ks_remode(W, sh, sw, v2=v2)
    mCFH, mCFW = (FH + sh - 1) // sh, (FW + sw - 1) // sw
    touched = 0
    for y in range(sh):
        for x in range(sw):
            if y >= FH or x >= FW:
                continue
            sub = W[:, y::sh, x::sw, :].transpose(1, 2, 0, 3)          # [CFH][CFW][OC][IC], filter order
            assert np.array_equal(_cw_phase(CW, W, sh, sw, y, x, v2), sub), (y, x)
            touched += sub.size
    # every filter element appears exactly once; the rest of each slot is untouched
    assert touched == W.size and np.count_nonzero(~np.isnan(CW)) == W.size
    assert CW.size == sh * sw * OC * mCFH * mCFW * IC


def test_strided_oracle_against_reference_routine_when_built(O):
    ref = O.ref_native("deltax")
    if ref is None or not hasattr(ref, "ref_cpu_deconv3D_deltaX_img2col"):
        pytest.skip("oracle/_ref/libref_deltax.so not built with the any-stride routines (python oracle/build_ref.py --deltax)")
    rng = np.random.default_rng(11)
    fp = ctypes.POINTER(ctypes.c_float)
    for case in SDX_SMALL:
        N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw = case
        OH, OW = _sdims(*case)
        dY = rng.standard_normal((N, OH, OW, OC)).astype(np.float32)
        W = rng.standard_normal((OC, FH, FW, IC)).astype(np.float32)
        out = np.zeros((N, IH, IW, IC), np.float32)
        ref.ref_cpu_deconv3D_deltaX_img2col(dY.ctypes.data_as(fp), OH, OW, W.ctypes.data_as(fp), FH, FW,
                                            out.ctypes.data_as(fp), IH, IW, N, IC, OC, sh, sw, ph, pw)
        assert np.array_equal(out, O.ref_loops.deconv3D_deltaX_img2col(dY, W, IH, IW, sh, sw, ph, pw)), case


def test_strided_argument_errors_without_gpu(pkg):
    lib = pkg.cu32.load()
    s = (ctypes.c_int64 * 1)(0)
    P = lambda a: ctypes.cast(a, ctypes.POINTER(ctypes.c_float))
    ok = 0x10000
    f = lib.cu32_dconv3D_deltaX_crossAdd
    #           dY  OH OW  W  FH FW  dX  IH IW  N  IC OC sh sw ph pw
    assert f(s, 1, P(ok), 4, 4, P(ok), 3, 3, P(ok), 0, 8, 2, 8, 8, 2, 2, 1, 1) == -2   # no rows
    assert f(s, 1, None, 4, 4, P(ok), 3, 3, P(ok), 8, 8, 2, 8, 8, 2, 2, 1, 1) == -1
    assert f(s, 1, P(ok), 4, 4, P(ok), 3, 3, P(ok), 8, 8, 2, 6, 8, 2, 2, 1, 1) == -4   # IC % 4
    assert f(s, 1, P(ok), 4, 4, P(ok), 3, 3, P(ok), 8, 8, 2, 8, 8, 0, 2, 1, 1) == -2   # stride 0
    assert lib.cu32_dconv3D_deltaX_crossAdd_SGM(s, 1, P(ok), 4, 4, P(ok), 3, 3, P(ok), 8, 8, 2, 8, 8, 2, 2, 1, 1, 0) == -8
    assert lib.cu32_dconv3D_deltaX_ksIms2R(s, 0, P(ok), 4, 4, P(ok), 3, 3, P(ok), 8, 8, 2, 8, 8, 1, 1) == -3   # no stream
    r = lib.cu32_ks_remodev2
    assert r(0, None, 3, 3, P(ok), 2, 2, 8, 8, 2, 2) == -1
    assert r(0, P(ok), 3, 3, P(ok), 3, 2, 8, 8, 2, 2) == -2        # CFH must be ceil(FH / sh)
    assert lib.cu32_ks_remode(0, P(ok), 3, 3, P(ok), 2, 2, 8, 8, 0, 2) == -2


# ------------------------------------------------------------------ GPU, any stride
def _remode_dev(pkg, W, sh, sw, v2=True, fill=float("nan")):
    """ks_remode / ks_remodev2 through the mirror; returns the device workspace (prefilled with `fill`)."""
    import gpu_util as G
    import torch
    OC, FH, FW, IC = W.shape
    CFH, CFW = (FH + sh - 1) // sh, (FW + sw - 1) // sw
    dW = G.dev(W)
    dCW = torch.full((sh * sw * OC * CFH * CFW * IC,), fill, device="cuda", dtype=torch.float32)
    fn = pkg.cu32.Cuda_dconv3D_deltaX.ks_remodev2 if v2 else pkg.cu32.Cuda_dconv3D_deltaX.ks_remode
    fn(G.stream(), dW.data_ptr(), FH, FW, dCW.data_ptr(), CFH, CFW, OC, IC, sh, sw)
    torch.cuda.synchronize()
    return dCW


def _run_strided(pkg, entry, dY, W, IH, IW, sh, sw, ph, pw, GM_slice=64):
    import gpu_util as G
    dx = pkg.cu32.Cuda_dconv3D_deltaX
    N, OH, OW, OC = dY.shape
    _, FH, FW, IC = W.shape
    ddY = G.dev(dY)
    filt = G.dev(W) if entry.startswith("crossAdd") else _remode_dev(pkg, W, sh, sw)
    out = G.Out(N * IH * IW * IC)
    base = [[G.stream()], 1, ddY.data_ptr(), OH, OW, filt.data_ptr(), FH, FW, out.ptr, IH, IW, N, IC, OC]
    tail = [ph, pw] if "Ims2R" in entry else [sh, sw, ph, pw]
    if entry.endswith("SGM"):
        tail.append(GM_slice)
    if entry == "ksV2_Ims2R":
        dx.dconv3D_deltaX_ksV2_Ims2R(True, *base, *tail)
    else:
        getattr(dx, "dconv3D_deltaX_" + entry)(*base, *tail)
    X = out.host((N, IH, IW, IC))
    G.check_status(pkg)
    return X


SDX_CASES = SDX_SMALL + [
    (4, 16, 16, 32, 64, 3, 3, 2, 2, 1, 1),
    (4, 32, 32, 16, 32, 7, 7, 2, 2, 3, 3),        # the 7x7 stride-2 stem of a residual network
    (4, 8, 8, 256, 64, 2, 2, 2, 2, 0, 0),         # non-overlapping 2x2 (a learned down-sampling)
    (2, 15, 17, 36, 40, 3, 3, 3, 3, 1, 1),        # ragged channels, extents not multiples of the stride
    (2, 14, 13, 64, 128, 4, 4, 2, 1, 1, 2),
    (8, 56, 56, 64, 128, 3, 3, 2, 2, 1, 1),       # a residual network's down-sampling 3x3
    (2, 9, 9, 132, 260, 3, 3, 2, 2, 1, 1),        # channel tails in both operands
]


@pytest.mark.gpu
@pytest.mark.parametrize("case", SDX_CASES)
def test_strided_deltax(pkg, O, cuda, case):
    N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw = case
    OH, OW = _sdims(*case)
    rng = np.random.default_rng(23)
    dY = rng.standard_normal((N, OH, OW, OC)).astype(np.float32)
    W = (rng.standard_normal((OC, FH, FW, IC)) * 0.1).astype(np.float32)
    want = O.f64.deconv3D_deltaX(dY, W, IH, IW, sh, sw, ph, pw)
    got = _run_strided(pkg, "crossAdd", dY, W, IH, IW, sh, sw, ph, pw)
    assert np.isfinite(got).all()
    rep = O.report(got, want)
    assert rep["frob"] <= 1e-6 and rep["elem"] <= 1e-4, (case, rep)
    # pixels that no filter tap reaches are exactly zero
    assert np.array_equal(got[want == 0], np.zeros_like(got[want == 0]))
    # the kernel-split native on the rearranged filter gives the same bits
    ks = _run_strided(pkg, "kernelSplit", dY, W, IH, IW, sh, sw, ph, pw)
    assert np.array_equal(ks, got)
    if N * IH * IW * IC * OC * FH * FW <= 4e7:       # the reference's FP32 loop, where it finishes in seconds
        loop = O.ref_loops.deconv3D_deltaX_img2col(dY, W, IH, IW, sh, sw, ph, pw)
        assert O.frob_rel(got, loop) <= 2e-6


@pytest.mark.gpu
@pytest.mark.parametrize("tile", [-1, 0, 3])
def test_strided_phases_in_one_launch_give_the_bits_of_one_launch_per_phase(pkg, O, cuda, tile):
    """With 2 to 4 phases the kernel takes tile j of every phase in turn inside one launch
    (cu32_tune("phase_fused", 1), the default); phases of unequal size leave tiles without work at the end of the
    smaller ones.  Same bits as one launch per phase, with and without the fused bias row, and FP64 parity."""
    import gpu_util as G
    rng = np.random.default_rng(29)
    for (N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw) in [
        (1, 33, 33, 128, 64, 3, 3, 2, 2, 1, 1),      # 17x17 = 289 pixels (two 256-row tiles) against 16x16 (one)
        (3, 57, 57, 64, 96, 3, 3, 2, 2, 1, 1),       # several tiles per CTA pair, phases of 841 / 812 / 784 pixels per image
        (2, 21, 40, 36, 40, 5, 3, 2, 1, 2, 1),       # two phases only, 5 and 3... taps apart
        (2, 19, 23, 32, 32, 2, 3, 2, 2, 0, 1),       # a phase with a single tap row
    ]:
        OH, OW = (IH + 2 * ph - FH) // sh + 1, (IW + 2 * pw - FW) // sw + 1
        dY = rng.standard_normal((N, OH, OW, OC)).astype(np.float32)
        W = (rng.standard_normal((OC, FH, FW, IC)) * 0.1).astype(np.float32)
        want = O.f64.deconv3D_deltaX(dY, W, IH, IW, sh, sw, ph, pw)
        res = {}
        for fused in (1, 0):
            pkg.cu32.tune("phase_fused", fused)
            pkg.cu32.tune("tile", tile)
            res[fused] = [_run_strided(pkg, nm, dY, W, IH, IW, sh, sw, ph, pw) for nm in ("crossAdd", "kernelSplit")]
        pkg.cu32.tune("phase_fused", 1)
        pkg.cu32.tune("tile", -1)
        for a, b in zip(res[1], res[0]):
            assert np.array_equal(a, b), (tile, N, IH, IW, sh, sw)
        assert np.array_equal(res[1][0], res[1][1])
        rep = O.report(res[1][0], want)
        assert rep["frob"] <= 1e-6 and rep["elem"] <= 1e-4, (tile, rep)


@pytest.mark.gpu
def test_extents_that_no_forward_convolution_gives(pkg, O, cuda):
    """The reference's data-gradient kernels take (IH, IW) and (OH, OW) as given; its own test pairs IH = OH = 64
    with an 8x8 filter and padding 4 (Cuda_conv3D_dX_test.java:178, :216), which no forward convolution produces.
    Rows of deltaY the sum would need outside [0, OH) count as zeros, rows it never reaches are never read:
    FP64 parity and the reference's check loop, stride 1 and strided entry points."""
    rng = np.random.default_rng(41)
    for (N, IH, IW, OH, OW, IC, OC, FH, FW, sh, sw, ph, pw) in [
        (2, 16, 16, 16, 16, 16, 24, 8, 8, 1, 1, 4, 4),     # the reference test's pairing, scaled down
        (2, 12, 9, 9, 9, 8, 8, 3, 3, 1, 1, 1, 1),          # deltaX taller than the forward input
        (2, 7, 9, 9, 9, 8, 8, 3, 3, 1, 1, 1, 1),           # and shorter
        (2, 19, 17, 8, 8, 16, 8, 3, 3, 2, 2, 1, 1),        # strided: forward gives OH = 10 and 9
        (1, 12, 12, 8, 7, 8, 12, 5, 5, 2, 2, 2, 2),        # strided: forward gives 6
        (2, 9, 10, 5, 4, 8, 8, 3, 2, 3, 2, 0, 1),
    ]:
        dY = rng.random((N, OH, OW, OC), dtype=np.float32)
        W = rng.random((OC, FH, FW, IC), dtype=np.float32)
        want = O.f64.deconv3D_deltaX(dY, W, IH, IW, sh, sw, ph, pw)
        loop = O.ref_loops.deconv3D_deltaX_img2col(dY, W, IH, IW, sh, sw, ph, pw)
        got = [_run_strided(pkg, nm, dY, W, IH, IW, sh, sw, ph, pw) for nm in ("crossAdd", "kernelSplit")]
        if sh == 1 and sw == 1:
            got.append(_run(pkg, "dconv3D_deltaX_s1", dY, W, IH, IW, ph, pw))
        for g in got:
            rep = O.report(g, want)
            assert rep["frob"] <= 1e-6 and rep["elem"] <= 1e-4, ((N, IH, IW, OH, OW, FH, FW, sh, sw, ph, pw), rep)
            assert O.frob_rel(g, loop) <= 2e-6
            assert np.array_equal(g, got[0])


@pytest.mark.gpu
def test_strided_entry_points_give_the_same_bits(pkg, O, cuda):
    rng = np.random.default_rng(21)
    N, IH, IW, IC, OC, FH, FW, ph, pw = 3, 12, 14, 24, 40, 3, 3, 1, 1
    for (sh, sw, names) in [
        (2, 2, ["kernelSplit", "kernelSplit_SGM", "ksImsR", "ksImsR_SGM", "ksImsR_texture", "ksImsR_texture_SGM",
                "ksIms2R", "ksIms2R_SGM", "ksIms2R_texture", "ksIms2R_texture_SGM", "ksV2_Ims2R", "crossAdd_SGM"]),
        (3, 2, ["kernelSplit", "kernelSplit_SGM", "ksImsR", "ksImsR_SGM", "ksImsR_texture", "ksImsR_texture_SGM",
                "crossAdd_SGM"]),
    ]:
        OH, OW = (IH + 2 * ph - FH) // sh + 1, (IW + 2 * pw - FW) // sw + 1
        dY = rng.standard_normal((N, OH, OW, OC)).astype(np.float32)
        W = rng.standard_normal((OC, FH, FW, IC)).astype(np.float32)
        base = _run_strided(pkg, "crossAdd", dY, W, IH, IW, sh, sw, ph, pw)
        assert O.frob_rel(base, O.f64.deconv3D_deltaX(dY, W, IH, IW, sh, sw, ph, pw)) <= 1e-6
        for nm in names:
            assert np.array_equal(_run_strided(pkg, nm, dY, W, IH, IW, sh, sw, ph, pw), base), (sh, sw, nm)


@pytest.mark.gpu
@pytest.mark.parametrize("geom", [(3, 3, 2, 2), (5, 3, 2, 2), (7, 7, 2, 2), (3, 3, 3, 3), (4, 4, 2, 1), (1, 1, 2, 2),
                                  (2, 5, 3, 2)])
def test_ks_remode_kernels_bit_exact(pkg, O, cuda, geom):
    import gpu_util as G
    FH, FW, sh, sw = geom
    OC, IC = 20, 12
    W = np.random.default_rng(22).standard_normal((OC, FH, FW, IC)).astype(np.float32)
    ref = O.ref_native("deltax")
    for v2 in (True, False):
        got = _remode_dev(pkg, W, sh, sw, v2=v2).cpu().numpy()
        want = O.ref_loops.ks_remode(W, sh, sw, v2=v2)
        assert np.array_equal(got, want, equal_nan=True), (geom, v2)
        if ref is not None and hasattr(ref, "ref_gpu_ks_remodev2") and OC % 4 == 0 and IC % 4 == 0:
            # the reference's own rearrangement kernels on the same filter
            dW = G.dev(W)
            dR = cuda.full((got.size,), float("nan"), device="cuda")
            fn = ref.ref_gpu_ks_remodev2 if v2 else ref.ref_gpu_ks_remode
            CFH, CFW = (FH + sh - 1) // sh, (FW + sw - 1) // sw
            assert fn(ctypes.c_longlong(G.stream()), ctypes.c_void_p(dW.data_ptr()), FH, FW,
                      ctypes.c_void_p(dR.data_ptr()), CFH, CFW, OC, IC, sh, sw) == 0
            cuda.cuda.synchronize()
            R = dR.cpu().numpy()
            live = ~np.isnan(want)        # the reference leaves the unused tail of a slot as it found it
            assert np.array_equal(R[live], got[live]), (geom, v2)


@pytest.mark.gpu
def test_strided_deltax_against_reference_kernels(pkg, O, cuda):
    """The reference's scatter-add kernels for strides > 1, compiled for this GPU, on the same inputs."""
    import gpu_util as G
    torch = cuda
    ref = O.ref_native("deltax")
    if ref is None or not hasattr(ref, "ref_gpu_dconv3D_deltaX_crossAdd"):
        pytest.skip("oracle/_ref/libref_deltax.so not built with the any-stride routines (python oracle/build_ref.py --deltax)")
    rng = np.random.default_rng(66)
    for case in [(4, 28, 28, 64, 64, 3, 3, 2, 2, 1, 1), (2, 15, 17, 16, 32, 5, 5, 3, 3, 2, 2)]:
        N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw = case
        OH, OW = _sdims(*case)
        dY = rng.standard_normal((N, OH, OW, OC)).astype(np.float32)
        W = (rng.standard_normal((OC, FH, FW, IC)) * 0.05).astype(np.float32)
        ddY, dW = G.dev(dY), G.dev(W)
        dR = torch.full((N, IH, IW, IC), float("nan"), device="cuda")
        streams = (ctypes.c_longlong * 10)(*([G.stream()] * 10))
        vp = lambda t: ctypes.c_void_p(t.data_ptr())
        assert ref.ref_gpu_dconv3D_deltaX_crossAdd(streams, 10, vp(ddY), OH, OW, vp(dW), FH, FW, vp(dR), IH, IW, N, IC,
                                                   OC, sh, sw, ph, pw) == 0
        torch.cuda.synchronize()
        R = dR.cpu().numpy()
        got = _run_strided(pkg, "crossAdd", dY, W, IH, IW, sh, sw, ph, pw)
        want = O.f64.deconv3D_deltaX(dY, W, IH, IW, sh, sw, ph, pw)
        e_ref, e_our = O.frob_rel(R, want), O.frob_rel(got, want)
        assert e_ref <= 5e-6, (case, e_ref)
        assert e_our <= 1e-6 and O.frob_rel(got, R) <= 5e-6, (case, e_our, e_ref)


@pytest.mark.gpu
def test_strided_deltax_is_the_gradient_of_the_forward_entry_point(pkg, O, cuda):
    """<conv3D(X, W), dY> == <X, deltaX(dY, W)> with both sides computed by this library."""
    import gpu_util as G
    rng = np.random.default_rng(67)
    N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw = 4, 17, 16, 32, 48, 3, 3, 2, 2, 1, 1
    OH, OW = (IH + 2 * ph - FH) // sh + 1, (IW + 2 * pw - FW) // sw + 1
    X = rng.standard_normal((N, IH, IW, IC)).astype(np.float32)
    W = (rng.standard_normal((OC, FH, FW, IC)) * 0.1).astype(np.float32)
    dY = rng.standard_normal((N, OH, OW, OC)).astype(np.float32)
    Y = G.conv(pkg, "conv3D_GemmR", X, W, sh, sw, ph, pw)
    dX = _run_strided(pkg, "kernelSplit", dY, W, IH, IW, sh, sw, ph, pw)
    lhs = float((Y.astype(np.float64) * dY).sum())
    rhs = float((X.astype(np.float64) * dX).sum())
    scale = float(np.sqrt((Y.astype(np.float64) ** 2).sum() * (dY.astype(np.float64) ** 2).sum()))
    assert abs(lhs - rhs) <= 2e-6 * scale, (lhs, rhs, scale)


def test_strided_oracle_against_golden_fixture(O, golden):
    """tests/golden/golden_deltax_strided.npz: outputs of the reference's own any-stride check loop on seeded inputs."""
    data = np.load(golden.HERE / "golden_deltax_strided.npz")
    assert set(data.files) == set(golden.DELTAX_STRIDED_CASES)
    for name, case in golden.DELTAX_STRIDED_CASES.items():
        N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw = case
        OH, OW = _sdims(*case)
        dY, W = golden.golden_inputs(name, [(N, OH, OW, OC), (OC, FH, FW, IC)])
        assert np.array_equal(O.ref_loops.deconv3D_deltaX_img2col(dY, W, IH, IW, sh, sw, ph, pw), data[name]), name


@pytest.mark.gpu
def test_strided_deltax_against_golden_fixture(pkg, O, cuda, golden):
    data = np.load(golden.HERE / "golden_deltax_strided.npz")
    for name, case in golden.DELTAX_STRIDED_CASES.items():
        N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw = case
        OH, OW = _sdims(*case)
        dY, W = golden.golden_inputs(name, [(N, OH, OW, OC), (OC, FH, FW, IC)])
        for entry in ("crossAdd", "ksImsR"):
            got = _run_strided(pkg, entry, dY, W, IH, IW, sh, sw, ph, pw)
            assert O.frob_rel(got, data[name]) <= 2e-6, (name, entry)   # the golden output carries FP32 accumulation error
            assert O.same_percent(got, data[name], 1e-5) >= 0.999, (name, entry)


@pytest.mark.gpu
def test_strided_deltax_repeats_bit_for_bit_on_every_tile(pkg, O, cuda):
    rng = np.random.default_rng(68)
    N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw = 8, 28, 28, 96, 64, 3, 3, 2, 2, 1, 1
    OH, OW = (IH + 2 * ph - FH) // sh + 1, (IW + 2 * pw - FW) // sw + 1
    dY = rng.standard_normal((N, OH, OW, OC)).astype(np.float32)
    W = (rng.standard_normal((OC, FH, FW, IC)) * 0.1).astype(np.float32)
    try:
        pkg.cu32.tune("tile", 4)
        base = _run_strided(pkg, "ksIms2R", dY, W, IH, IW, sh, sw, ph, pw)
        assert O.frob_rel(base, O.f64.deconv3D_deltaX(dY, W, IH, IW, sh, sw, ph, pw)) <= 1e-6
        for tile in (0, 1, 2, 3, 4, 5):
            pkg.cu32.tune("tile", tile)
            for rep in range(6):
                R = _run_strided(pkg, "crossAdd" if rep & 1 else "ksIms2R", dY, W, IH, IW, sh, sw, ph, pw)
                assert np.array_equal(R, base), (tile, rep, int((R != base).sum()))
    finally:
        pkg.cu32.tune("tile", -1)


# ------------------------------------------------------------------ bias row fused into the data gradient
@pytest.mark.gpu
@pytest.mark.parametrize("case", [
    # N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw, width
    (4, 12, 12, 32, 48, 3, 3, 1, 1, 1, 1, 32),
    (2, 9, 10, 132, 64, 3, 3, 1, 1, 1, 1, 130),      # padded channels: columns >= width come out 0
    (3, 8, 8, 24, 16, 1, 1, 1, 1, 0, 0, 24),         # 1x1: the plain contraction
    (4, 16, 16, 32, 64, 3, 3, 2, 2, 1, 1, 32),       # stride 2 through the kernel-split workspace
    (2, 15, 17, 36, 40, 3, 3, 3, 3, 1, 1, 34),
    (2, 14, 13, 64, 128, 4, 4, 2, 1, 1, 2, 64),
])
def test_deltax_biased_is_the_unbiased_native_followed_by_the_bias_kernel(pkg, O, cuda, case):
    """The transposed convolution's forward pass with bias: the fused entry points must store the bits of the
    data-gradient native followed by linear_dual2D_row(Y, bias, 1, 1, 0)."""
    import gpu_util as G
    N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw, width = case
    OH, OW = (IH + 2 * ph - FH) // sh + 1, (IW + 2 * pw - FW) // sw + 1
    rng = np.random.default_rng(69)
    dY = rng.standard_normal((N, OH, OW, OC)).astype(np.float32)
    W = (rng.standard_normal((OC, FH, FW, IC)) * 0.1).astype(np.float32)
    bias = rng.standard_normal(IC).astype(np.float32)
    dx = pkg.cu32.Cuda_dconv3D_deltaX
    ddY, dB = G.dev(dY), G.dev(bias)
    out = G.Out(N * IH * IW * IC)
    if sh == 1 and sw == 1:
        plain = _run(pkg, "dconv3D_deltaX_W1" if (FH, FW, ph, pw) == (1, 1, 0, 0) else "dconv3D_deltaX_s1", dY, W, IH, IW, ph, pw)
        dW = G.dev(W)
        dx.dconv3D_deltaX_s1_biased([G.stream()], 1, ddY.data_ptr(), OH, OW, dW.data_ptr(), FH, FW, out.ptr, IH, IW, N, IC, OC,
                                    ph, pw, dB.data_ptr(), width)
    else:
        plain = _run_strided(pkg, "ksImsR", dY, W, IH, IW, sh, sw, ph, pw)
        dCW = _remode_dev(pkg, W, sh, sw)
        dx.dconv3D_deltaX_ksImsR_biased([G.stream()], 1, ddY.data_ptr(), OH, OW, dCW.data_ptr(), FH, FW, out.ptr, IH, IW, N, IC,
                                        OC, sh, sw, ph, pw, dB.data_ptr(), width)
    fused = out.host((N, IH, IW, IC))
    G.check_status(pkg)
    want = O.ref_loops.linear_dual2D_row(plain.reshape(-1, IC), bias, 1.0, 1.0, 0.0, width).reshape(fused.shape)
    assert np.array_equal(fused, want)
    if width < IC:
        assert not fused[..., width:].any()


@pytest.mark.gpu
@pytest.mark.parametrize("geom", [(3, 3, 1, 1, 1, 1), (4, 4, 2, 2, 1, 1), (5, 5, 2, 2, 2, 2)])
def test_transposed_convolution_channel_sweep_of_the_reference_test(pkg, O, cuda, geom):
    """The reference's transposed-convolution test sweeps the output channels 1..128 on a 4 x 16 x 16 x 16 input for
    3x3 stride 1, 4x4 stride 2 and 5x5 stride 2 (test/cuda/conv3D/Cuda_deconv3D_biased_test.java:83-114).  The engine
    pads the channel count to a multiple of 4 and passes the true count as the bias width; here every padded count
    4..128 with a true width 0 to 3 below it, FP64 parity of the fused native, pad channels zero.  (The transposed convolution's input is the data gradient's deltaY, its output deltaX.)"""
    import gpu_util as G
    FH, FW, sh, sw, ph, pw = geom
    N, OH, OW, OC = 4, 16, 16, 16                      # the transposed convolution's input
    IH, IW = (OH - 1) * sh + FH - 2 * ph, (OW - 1) * sw + FW - 2 * pw
    rng = np.random.default_rng(71)
    dY = rng.random((N, OH, OW, OC), dtype=np.float32)
    dx = pkg.cu32.Cuda_dconv3D_deltaX
    ddY = G.dev(dY)
    for IC in range(4, 129, 4):                        # the transposed convolution's output channels, padded
        width = IC - (IC // 4) % 4
        W = rng.random((OC, FH, FW, IC), dtype=np.float32)
        W[..., width:] = 0.0
        bias = rng.random(IC, dtype=np.float32)
        want = O.f64.deconv3D_deltaX(dY, W, IH, IW, sh, sw, ph, pw) + bias.astype(np.float64)
        want[..., width:] = 0.0
        out = G.Out(N * IH * IW * IC)
        dB = G.dev(bias)
        if sh == 1:
            dW = G.dev(W)
            dx.dconv3D_deltaX_s1_biased([G.stream()], 1, ddY.data_ptr(), OH, OW, dW.data_ptr(), FH, FW, out.ptr, IH, IW, N,
                                        IC, OC, ph, pw, dB.data_ptr(), width)
        else:
            dCW = _remode_dev(pkg, W, sh, sw)
            dx.dconv3D_deltaX_ksImsR_biased([G.stream()], 1, ddY.data_ptr(), OH, OW, dCW.data_ptr(), FH, FW, out.ptr, IH, IW,
                                            N, IC, OC, sh, sw, ph, pw, dB.data_ptr(), width)
        got = out.host((N, IH, IW, IC))
        G.check_status(pkg)
        assert not got[..., width:].any(), (geom, IC, width)
        rep = O.report(got, want)
        assert rep["frob"] <= 1e-6 and rep["elem"] <= 1e-4, (geom, IC, rep)

