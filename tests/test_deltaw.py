"""Weight gradient of the convolution (the natives of Cuda_dconv3D_deltaW).

The reference's CUDA source for these natives is not published; the oracle is a restatement of the Java check loop
its own test uses (Tense.deconv3d_deltaW_naive) plus an FP64 version.  Neither can be run against reference code
here (no JVM), so the FP64 oracle is pinned through the pinned forward-convolution oracle instead: the weight
gradient is linear in the filter, so deltaW[oc, fh, fw, ic] must equal <conv(X, E), deltaY> for the one-hot filter E
at (oc, fh, fw, ic) - checked for every element of small cases - and the check loop must agree with FP64 to FP32
rounding."""
import ctypes

import numpy as np
import pytest


def _odims(IH, IW, FH, FW, sh, sw, ph, pw):
    return (IH + 2 * ph - FH) // sh + 1, (IW + 2 * pw - FW) // sw + 1


DW_SMALL = [
    # N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw
    (2, 6, 5, 4, 4, 3, 3, 1, 1, 1, 1),
    (2, 7, 8, 4, 8, 3, 2, 2, 2, 1, 0),
    (1, 9, 9, 4, 4, 5, 5, 3, 2, 2, 2),
    (3, 4, 4, 8, 4, 1, 1, 1, 1, 0, 0),
]


@pytest.mark.parametrize("case", DW_SMALL)
def test_deltaw_oracle_is_the_derivative_of_the_forward_oracle(O, case):
    N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw = case
    OH, OW = _odims(IH, IW, FH, FW, sh, sw, ph, pw)
    rng = np.random.default_rng(31)
    X = rng.standard_normal((N, IH, IW, IC)).astype(np.float32)
    dY = rng.standard_normal((N, OH, OW, OC)).astype(np.float32)
    dW64 = O.f64.deconv3D_deltaW(X, dY, FH, FW, sh, sw, ph, pw)
    dY64 = dY.astype(np.float64)
    for oc in range(OC):
        for fh in range(FH):
            for fw in range(FW):
                for ic in range(IC):
                    E = np.zeros((OC, FH, FW, IC), np.float32); E[oc, fh, fw, ic] = 1.0
                    want = float((O.f64.conv3D(X, E, OH, OW, sh, sw, ph, pw) * dY64).sum())
                    assert abs(dW64[oc, fh, fw, ic] - want) <= 1e-12 * max(1.0, abs(want)), (oc, fh, fw, ic)
    loop = O.ref_loops.deconv3D_deltaW_naive(X, dY, FH, FW, sh, sw, ph, pw)
    assert O.frob_rel(loop, dW64) <= 1e-7      # double accumulator: only the products and the final cast round


def test_deltaw_oracle_known_answer(O):
    # one image, one channel each way, 2x2 filter, stride 1, no padding: deltaW[fh, fw] = sum of the 2x2 window sums
    X = np.arange(9, dtype=np.float32).reshape(1, 3, 3, 1)
    dY = np.ones((1, 2, 2, 1), np.float32)
    dW = O.ref_loops.deconv3D_deltaW_naive(X, dY, 2, 2, 1, 1, 0, 0)
    assert np.array_equal(dW[0, :, :, 0], np.array([[8, 12], [20, 24]], np.float32))


def test_deltaw_argument_errors_without_gpu(pkg):
    lib = pkg.cu32.load()
    s = (ctypes.c_int64 * 1)(0)
    P = lambda a: ctypes.cast(a, ctypes.POINTER(ctypes.c_float))
    ok = 0x10000
    f = lib.cu32_dconv3D_deltaW_GemmSK
    #              GZ   X  IH IW  dY  OH OW  dW   buf  FH FW N  IC OC sh sw ph pw
    assert f(s, 1, 2, P(ok), 8, 8, P(ok), 8, 8, P(ok), None, 3, 3, 2, 8, 8, 1, 1, 1, 1) == -1     # GridZ > 1 needs the buffer
    assert f(s, 1, 0, P(ok), 8, 8, P(ok), 8, 8, P(ok), P(ok), 3, 3, 2, 8, 8, 1, 1, 1, 1) == -8
    assert f(s, 1, 1, P(ok), 8, 8, P(ok), 0, 8, P(ok), P(ok), 3, 3, 2, 8, 8, 1, 1, 1, 1) == -2    # no rows
    assert f(s, 1, 1, P(ok), 8, 8, P(ok), 8, 8, P(ok), P(ok), 3, 3, 2, 6, 8, 1, 1, 1, 1) == -4    # IC % 4
    assert f(s, 0, 1, P(ok), 8, 8, P(ok), 8, 8, P(ok), P(ok), 3, 3, 2, 8, 8, 1, 1, 1, 1) == -3
    assert lib.cu32_dconv3D_deltaW(s, 1, None, 8, 8, P(ok), 8, 8, P(ok), 3, 3, 2, 8, 8, 1, 1, 1, 1) == -1
    assert lib.cu32_dconv3D_deltaW_buf_summary(0, None, P(ok), 1, 16) == -1


# ------------------------------------------------------------------ GPU
def _run(pkg, entry, X, dY, FH, FW, sh, sw, ph, pw, GZ=1):
    import gpu_util as G
    import torch
    dw = pkg.cu32.Cuda_dconv3D_deltaW
    N, IH, IW, IC = X.shape
    _, OH, OW, OC = dY.shape
    dX_, ddY = G.dev(X), G.dev(dY)
    size = OC * FH * FW * IC
    out = G.Out(size)
    buf = torch.full((max(GZ - 1, 1) * size,), float("nan"), device="cuda")
    s = [G.stream()]
    if entry == "dconv3D_deltaW":
        dw.dconv3D_deltaW(s, 1, dX_.data_ptr(), IH, IW, ddY.data_ptr(), OH, OW, out.ptr, FH, FW, N, IC, OC, sh, sw, ph, pw)
    elif entry == "dconv3D_deltaW_W1":
        dw.dconv3D_deltaW_W1(s, 1, dX_.data_ptr(), IH, IW, ddY.data_ptr(), out.ptr, N, IC, OC)
    elif entry in ("dconv3D_deltaW_GemmSK", "dconv3D_deltaW_GemmV2SK"):
        getattr(dw, entry)(s, 1, GZ, dX_.data_ptr(), IH, IW, ddY.data_ptr(), OH, OW, out.ptr, buf.data_ptr(), FH, FW,
                           N, IC, OC, sh, sw, ph, pw)
    elif entry == "dconv3D_deltaW_GemmSK_W1":
        dw.dconv3D_deltaW_GemmSK_W1(s, 1, GZ, dX_.data_ptr(), IH, IW, ddY.data_ptr(), out.ptr, buf.data_ptr(), N, IC, OC)
    elif entry.startswith("Im2col_WinogradV2_SHW_s16"):
        assert getattr(dw, entry)(s, 1, GZ, OH, OW, 0, dX_.data_ptr(), IH, IW, ddY.data_ptr(), OH, OW, out.ptr,
                                  buf.data_ptr(), FH, FW, N, IC, OC, ph, pw, 6) is True
    elif entry.startswith("Im2col_WinogradV2_SHW"):
        assert getattr(dw, entry)(s, 1, GZ, OH, OW, dX_.data_ptr(), IH, IW, ddY.data_ptr(), OH, OW, out.ptr,
                                  buf.data_ptr(), FH, FW, N, IC, OC, ph, pw, 6) is True
    else:
        raise ValueError(entry)
    if GZ > 1:
        dw.buf_summary(s[0], buf.data_ptr(), out.ptr, GZ - 1, size)
    R = out.host((OC, FH, FW, IC))
    G.check_status(pkg)
    return R


DW_CASES = DW_SMALL + [
    (4, 14, 14, 32, 64, 3, 3, 1, 1, 1, 1),
    (8, 28, 28, 64, 64, 3, 3, 1, 1, 1, 1),
    (4, 16, 16, 16, 32, 3, 3, 2, 2, 1, 1),
    (2, 32, 32, 16, 36, 7, 7, 2, 2, 3, 3),
    (2, 11, 10, 132, 260, 3, 3, 1, 1, 1, 1),      # channel tails on both sides
    (3, 9, 12, 4, 8, 2, 4, 1, 2, 1, 2),
    (5, 7, 7, 256, 32, 3, 3, 1, 1, 0, 0),          # pixel count not a multiple of the 32-pixel k-block
    (4, 10, 10, 48, 24, 1, 1, 1, 1, 0, 0),         # 1x1: the plain A^T*B contraction
    (4, 10, 10, 48, 24, 1, 1, 2, 2, 0, 0),         # 1x1 with a stride: the im2col walk skips pixels
]


@pytest.mark.gpu
@pytest.mark.parametrize("case", DW_CASES)
def test_deltaw(pkg, O, cuda, case):
    N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw = case
    OH, OW = _odims(IH, IW, FH, FW, sh, sw, ph, pw)
    rng = np.random.default_rng(32)
    X = rng.standard_normal((N, IH, IW, IC)).astype(np.float32)
    dY = rng.standard_normal((N, OH, OW, OC)).astype(np.float32)
    want = O.f64.deconv3D_deltaW(X, dY, FH, FW, sh, sw, ph, pw)
    got = _run(pkg, "dconv3D_deltaW", X, dY, FH, FW, sh, sw, ph, pw)
    rep = O.report(got, want)
    assert np.isfinite(got).all() and rep["frob"] <= 1e-6 and rep["elem"] <= 1e-4, (case, rep)
    for GZ in (2, 5):
        sk = _run(pkg, "dconv3D_deltaW_GemmSK", X, dY, FH, FW, sh, sw, ph, pw, GZ=GZ)
        rep = O.report(sk, want)
        assert np.isfinite(sk).all() and rep["frob"] <= 1e-6 and rep["elem"] <= 1e-4, (case, GZ, rep)
    if N * OH * OW * IC * OC * FH * FW <= 4e7:
        loop = O.ref_loops.deconv3D_deltaW_naive(X, dY, FH, FW, sh, sw, ph, pw)
        assert O.frob_rel(got, loop) <= 1e-6
        assert O.same_percent(np.abs(got), np.abs(loop), 1e-3) >= 0.999     # the gate of the reference's own Java test


@pytest.mark.gpu
def test_deltaw_extents_that_no_forward_convolution_gives(pkg, O, cuda):
    """(IH, IW) and (OH, OW) are taken as given, as by the reference's natives (its tests pass both): input pixels
    outside X count as zeros.  FP64 parity, plain and split-K."""
    rng = np.random.default_rng(43)
    for (N, IH, IW, OH, OW, IC, OC, FH, FW, sh, sw, ph, pw) in [
        (2, 16, 16, 16, 16, 16, 24, 8, 8, 1, 1, 4, 4),     # the data-gradient test's pairing of the reference
        (2, 12, 9, 9, 9, 8, 8, 3, 3, 1, 1, 1, 1),
        (2, 7, 9, 9, 9, 8, 8, 3, 3, 1, 1, 1, 1),
        (2, 19, 17, 8, 8, 16, 8, 3, 3, 2, 2, 1, 1),
        (1, 12, 12, 8, 7, 8, 12, 5, 5, 2, 2, 2, 2),
    ]:
        X = rng.standard_normal((N, IH, IW, IC)).astype(np.float32)
        dY = rng.standard_normal((N, OH, OW, OC)).astype(np.float32)
        want = O.f64.deconv3D_deltaW(X, dY, FH, FW, sh, sw, ph, pw)
        for entry, GZ in (("dconv3D_deltaW", 1), ("dconv3D_deltaW_GemmSK", 3)):
            got = _run(pkg, entry, X, dY, FH, FW, sh, sw, ph, pw, GZ=GZ)
            rep = O.report(got, want)
            assert np.isfinite(got).all() and rep["frob"] <= 1e-6 and rep["elem"] <= 1e-4, ((IH, OH, FH, sh, ph), entry, rep)


@pytest.mark.gpu
def test_deltaw_entry_points(pkg, O, cuda):
    rng = np.random.default_rng(33)
    N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw = 4, 12, 12, 24, 40, 3, 3, 1, 1, 1, 1
    X = rng.standard_normal((N, IH, IW, IC)).astype(np.float32)
    dY = rng.standard_normal((N, IH, IW, OC)).astype(np.float32)
    want = O.f64.deconv3D_deltaW(X, dY, FH, FW, sh, sw, ph, pw)
    base = _run(pkg, "dconv3D_deltaW_GemmSK", X, dY, FH, FW, sh, sw, ph, pw, GZ=3)
    assert O.frob_rel(base, want) <= 1e-6
    for entry in ("dconv3D_deltaW_GemmV2SK", "Im2col_WinogradV2_SHW_s4_texture", "Im2col_WinogradV2_SHW_s8_texture",
                  "Im2col_WinogradV2_SHW_s16_texture"):
        assert np.array_equal(_run(pkg, entry, X, dY, FH, FW, sh, sw, ph, pw, GZ=3), base), entry
    # 1x1 natives
    dY1 = rng.standard_normal((N, IH, IW, OC)).astype(np.float32)
    want1 = O.f64.deconv3D_deltaW(X, dY1, 1, 1, 1, 1, 0, 0)
    a = _run(pkg, "dconv3D_deltaW_W1", X, dY1, 1, 1, 1, 1, 0, 0)
    b = _run(pkg, "dconv3D_deltaW_GemmSK_W1", X, dY1, 1, 1, 1, 1, 0, 0, GZ=4)
    assert O.frob_rel(a, want1) <= 1e-6 and O.frob_rel(b, want1) <= 1e-6


@pytest.mark.gpu
def test_deltaw_is_the_gradient_of_the_forward_entry_point(pkg, O, cuda):
    """<conv3D(X, W), dY> == <W, deltaW(X, dY)> with both sides computed by this library."""
    import gpu_util as G
    rng = np.random.default_rng(34)
    N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw = 4, 15, 14, 32, 48, 3, 3, 2, 2, 1, 1
    OH, OW = _odims(IH, IW, FH, FW, sh, sw, ph, pw)
    X = rng.standard_normal((N, IH, IW, IC)).astype(np.float32)
    W = (rng.standard_normal((OC, FH, FW, IC)) * 0.1).astype(np.float32)
    dY = rng.standard_normal((N, OH, OW, OC)).astype(np.float32)
    Y = G.conv(pkg, "conv3D_GemmR", X, W, sh, sw, ph, pw)
    dW = _run(pkg, "dconv3D_deltaW_GemmSK", X, dY, FH, FW, sh, sw, ph, pw, GZ=4)
    lhs = float((Y.astype(np.float64) * dY).sum())
    rhs = float((W.astype(np.float64) * dW).sum())
    scale = float(np.sqrt((Y.astype(np.float64) ** 2).sum() * (dY.astype(np.float64) ** 2).sum()))
    assert abs(lhs - rhs) <= 2e-6 * scale, (lhs, rhs, scale)


@pytest.mark.gpu
def test_conv_layer_weight_gradient_through_the_engine_mirror(pkg, O, cuda):
    import gpu_util as G
    torch = cuda
    keep = []

    def malloc(n):
        t = torch.full((n,), float("nan"), device="cuda")
        keep.append(t)
        return t.data_ptr(), t
    eng = pkg.engine.Cu32Engine(148, malloc, [G.stream()])
    rng = np.random.default_rng(35)
    for (N, IH, IW, IC, OC, F, p, st) in [(8, 14, 14, 32, 64, 3, 1, 1), (4, 10, 10, 16, 24, 1, 0, 1),
                                          (8, 14, 14, 32, 64, 3, 1, 2)]:
        OH, OW = (IH + 2 * p - F) // st + 1, (IW + 2 * p - F) // st + 1
        X = rng.standard_normal((N, IH, IW, IC)).astype(np.float32)
        dY = rng.standard_normal((N, OH, OW, OC)).astype(np.float32)
        dX_, ddY = G.dev(X), G.dev(dY)
        gW = G.Out(OC * F * F * IC)
        gz = eng.conv3D_deltaW(gW.ptr, F, F, dX_.data_ptr(), IH, IW, ddY.data_ptr(), OH, OW, N, IC, OC, st, st, p, p)
        G.check_status(pkg)
        rep = O.report(gW.host((OC, F, F, IC)), O.f64.deconv3D_deltaW(X, dY, F, F, st, st, p, p))
        assert rep["frob"] <= 1e-6 and rep["elem"] <= 1e-4, (F, st, gz, rep)


@pytest.mark.gpu
def test_deltaw_repeats_bit_for_bit_on_every_tile(pkg, O, cuda):
    """Same reduction order on every tile shape and in every run: an unfenced hand-over between the im2col loads,
    the split and the tensor core would show up as a few differing elements in one run of many."""
    rng = np.random.default_rng(36)
    N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw = 8, 28, 28, 64, 96, 3, 3, 1, 1, 1, 1
    X = rng.standard_normal((N, IH, IW, IC)).astype(np.float32)
    dY = rng.standard_normal((N, IH, IW, OC)).astype(np.float32)
    try:
        pkg.cu32.tune("tile", 4)
        base = _run(pkg, "dconv3D_deltaW_GemmSK", X, dY, FH, FW, sh, sw, ph, pw, GZ=4)
        assert O.frob_rel(base, O.f64.deconv3D_deltaW(X, dY, FH, FW, sh, sw, ph, pw)) <= 1e-6
        for tile in (0, 1, 2, 3, 4, 5):
            pkg.cu32.tune("tile", tile)
            for rep in range(6):
                R = _run(pkg, "dconv3D_deltaW_GemmSK", X, dY, FH, FW, sh, sw, ph, pw, GZ=4)
                assert np.array_equal(R, base), (tile, rep, int((R != base).sum()))
    finally:
        pkg.cu32.tune("tile", -1)
