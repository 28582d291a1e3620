"""Geometries no im2col tensor map can express - strides above 8, window corners beyond +-128, padding beyond the
filter reach, filters wider than 16 on the data-gradient natives - are served by the kernel's gather path (the
producer warp builds the same shared-memory tile with plain loads).  The reference computes any geometry
(Cuda_conv3D/conv3D.cuh:866-1070 has no such limits), so these entry points must not refuse one.

Two kinds of checks: (1) on ordinary geometries the gather path, forced by a tuning key, returns the bits of the
tensor-map path - same tiles, same operand values, same order; (2) on the geometries only it can serve, the result
meets the contraction tolerance against the FP64 oracle."""
import numpy as np
import pytest

import gpu_util as G
import test_deltax as DX
import test_deltaw as DW

pytestmark = pytest.mark.gpu


def _accurate(O, Y, Y64, what):
    assert np.isfinite(Y).all(), what
    rep = O.report(Y, Y64)
    assert rep["frob"] <= 1e-6 and rep["elem"] <= 1e-4, (what, rep)


def test_gather_path_returns_the_bits_of_the_tensor_map_path(pkg, O, cuda):
    rng = np.random.default_rng(41)
    X = rng.standard_normal((4, 13, 11, 36)).astype(np.float32)
    W = (rng.standard_normal((40, 3, 3, 36)) * 0.1).astype(np.float32)
    dY = rng.standard_normal((4, 7, 6, 40)).astype(np.float32)        # conv of X with stride 2, pad 1
    dY1 = rng.standard_normal((4, 13, 11, 40)).astype(np.float32)     # stride 1, pad 1
    runs = {
        "conv s1": lambda: G.conv(pkg, "conv3D_GemmR", X, W, 1, 1, 1, 1),
        "conv s2": lambda: G.conv(pkg, "conv3D_GemmR", X, W, 2, 2, 1, 1),
        "deltaX s1": lambda: DX._run(pkg, "dconv3D_deltaX_s1", dY1, W, 13, 11, 1, 1),
        "deltaX s2": lambda: DX._run_strided(pkg, "crossAdd", dY, W, 13, 11, 2, 2, 1, 1),
        "deltaW s2": lambda: DW._run(pkg, "dconv3D_deltaW_GemmSK", X, dY, 3, 3, 2, 2, 1, 1, GZ=3),
    }
    for tile in (-1, 1, 4):
        pkg.cu32.tune("tile", tile)
        for name, fn in runs.items():
            pkg.cu32.tune("gather", 0)
            base = fn()
            pkg.cu32.tune("gather", 1)
            got = fn()
            pkg.cu32.tune("gather", 0)
            assert np.array_equal(got, base), (name, tile, int((got != base).sum()))


@pytest.mark.parametrize("case", [
    # N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw
    (2, 40, 50, 8, 12, 3, 3, 9, 12, 1, 1),        # strides beyond the tensor map's three bits
    (2, 30, 30, 4, 8, 5, 5, 10, 11, 2, 2),
    (1, 12, 12, 8, 8, 3, 3, 1, 1, 5, 5),          # padding beyond the filter size: a border of pure padding
    (1, 6, 6, 4, 8, 3, 3, 1, 1, 130, 130),        # window corners beyond -128
    (1, 24, 24, 4, 4, 17, 17, 1, 1, 8, 8),        # 17 x 17 filter
])
def test_forward_convolution_any_geometry(pkg, O, cuda, case):
    N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw = case
    rng = np.random.default_rng(43)
    X = rng.standard_normal((N, IH, IW, IC)).astype(np.float32)
    W = (rng.standard_normal((OC, FH, FW, IC)) * np.sqrt(2.0 / (FH * FW * IC))).astype(np.float32)
    OH, OW = (IH + 2 * ph - FH) // sh + 1, (IW + 2 * pw - FW) // sw + 1
    Y = G.conv(pkg, "conv3D_GemmR", X, W, sh, sw, ph, pw)
    _accurate(O, Y, O.f64.conv3D(X, W, OH, OW, sh, sw, ph, pw), f"conv {case}")
    assert np.array_equal(G.conv(pkg, "conv3D", X, W, sh, sw, ph, pw), Y)


@pytest.mark.parametrize("case", [
    # N, IH, IW, IC, OC, FH, FW, ph, pw   (stride 1)
    (1, 24, 24, 8, 8, 17, 17, 8, 8),              # filter wider than 16
    (2, 8, 9, 8, 12, 3, 3, 3, 3),                 # padding beyond the filter reach: the outer pixels of deltaY never contribute
    (1, 20, 18, 4, 4, 19, 17, 9, 8),
])
def test_data_gradient_stride_one_any_geometry(pkg, O, cuda, case):
    N, IH, IW, IC, OC, FH, FW, ph, pw = case
    OH, OW = IH + 2 * ph - FH + 1, IW + 2 * pw - FW + 1
    rng = np.random.default_rng(47)
    dY = rng.standard_normal((N, OH, OW, OC)).astype(np.float32)
    W = (rng.standard_normal((OC, FH, FW, IC)) * 0.1).astype(np.float32)
    dXg = DX._run(pkg, "dconv3D_deltaX_s1", dY, W, IH, IW, ph, pw)
    _accurate(O, dXg, O.f64.deconv3D_deltaX(dY, W, IH, IW, 1, 1, ph, pw), f"deltaX s1 {case}")


@pytest.mark.parametrize("case", [
    # N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw
    (2, 40, 37, 8, 8, 3, 3, 17, 18, 1, 1),        # strides beyond 16; most phases meet no tap
    (1, 35, 35, 4, 8, 20, 20, 17, 17, 2, 2),      # and a filter longer than the stride
    (2, 30, 30, 4, 8, 5, 5, 10, 11, 2, 2),
])
def test_data_gradient_any_stride(pkg, O, cuda, case):
    N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw = case
    OH, OW = (IH + 2 * ph - FH) // sh + 1, (IW + 2 * pw - FW) // sw + 1
    # the natives require extents the forward convolution would give back exactly
    IH, IW = (OH - 1) * sh + FH - 2 * ph, (OW - 1) * sw + FW - 2 * pw
    rng = np.random.default_rng(53)
    dY = rng.standard_normal((N, OH, OW, OC)).astype(np.float32)
    W = (rng.standard_normal((OC, FH, FW, IC)) * 0.1).astype(np.float32)
    want = O.f64.deconv3D_deltaX(dY, W, IH, IW, sh, sw, ph, pw)
    for entry in ("crossAdd", "kernelSplit"):
        got = DX._run_strided(pkg, entry, dY, W, IH, IW, sh, sw, ph, pw)
        _accurate(O, got, want, f"{entry} {case}")


@pytest.mark.parametrize("case", [
    # N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw
    (2, 40, 50, 8, 12, 3, 3, 9, 12, 1, 1),
    (4, 30, 30, 4, 8, 5, 5, 10, 11, 2, 2),
    (2, 12, 12, 8, 8, 3, 3, 1, 1, 5, 5),
])
def test_weight_gradient_any_geometry(pkg, O, cuda, case):
    N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw = case
    OH, OW = (IH + 2 * ph - FH) // sh + 1, (IW + 2 * pw - FW) // sw + 1
    rng = np.random.default_rng(59)
    X = rng.standard_normal((N, IH, IW, IC)).astype(np.float32)
    dY = rng.standard_normal((N, OH, OW, OC)).astype(np.float32)
    want = O.f64.deconv3D_deltaW(X, dY, FH, FW, sh, sw, ph, pw)
    for gz in (1, 3):
        got = DW._run(pkg, "dconv3D_deltaW_GemmSK" if gz > 1 else "dconv3D_deltaW", X, dY, FH, FW, sh, sw, ph, pw, GZ=gz)
        _accurate(O, got, want, f"deltaW GZ={gz} {case}")
