"""Seeded random shapes through every operator family: small enough for a full FP64 check of
each case, chosen to hit the corners of the persistent tile loop (fewer tiles than CTAs, one
tile per CTA pair, ragged last tiles in both directions, K shorter than one k-block, split-K
slices without work, batches of one, odd strides and paddings)."""
import numpy as np
import pytest
import torch

import gpu_util as G

pytestmark = pytest.mark.gpu


def _acc(O, C, C64, what):
    assert np.isfinite(C).all(), what
    rep = O.report(C, C64)
    assert rep["frob"] <= 1e-6 and rep["elem"] <= 1e-4, (what, rep)


def test_fuzz_matmul(pkg, O, cuda):
    rng = np.random.default_rng(2024)
    for case in range(40):
        form = ["AB", "T1", "T2"][case % 3]
        N = int(rng.integers(1, 200)) * 4
        M = int(rng.integers(1, 200)) * 4
        K = int(rng.choice([4, 8, 28, 32, 36, 64, 100, 256, 516, 1000]))
        if case % 7 == 0:
            N = int(rng.choice([4, 8, 128, 256, 1024, 2052]))
        sa, sb = G.mm_shapes(form, N, M, K)
        A = rng.standard_normal(sa).astype(np.float32)
        B = rng.standard_normal(sb).astype(np.float32)
        if case % 4 == 3 and K >= 64:
            GZ = int(rng.choice([2, 3, 5, 8, 16]))
            C, _, _ = G.matmul_sk(pkg, form, A, B, N, M, K, GZ)
            _acc(O, C, G.f64_matmul(O, form, A, B), f"SK {form} {N}x{M}x{K} GZ={GZ}")
        else:
            C = G.matmul(pkg, form, A, B, N, M, K)
            _acc(O, C, G.f64_matmul(O, form, A, B), f"{form} {N}x{M}x{K}")


def test_fuzz_batched(pkg, O, cuda):
    bm = pkg.cu32.Cuda_batchMatMul
    rng = np.random.default_rng(7)
    s = [G.stream()]
    for case in range(24):
        Batch = int(rng.choice([1, 2, 3, 7, 16, 150, 301]))
        N = int(rng.integers(1, 140))
        M = int(rng.integers(1, 70)) * 4
        K = int(rng.integers(1, 40)) * 4
        kind = case % 3
        if kind == 0:
            AK = K + int(rng.choice([0, 4, 8]))
            A = np.zeros((Batch, N, AK), np.float32); A[:, :, :K] = rng.standard_normal((Batch, N, K))
            B = rng.standard_normal((Batch, K, M)).astype(np.float32)
            out = G.Out(Batch * N * M)
            dA, dB = G.dev(A), G.dev(B)
            bm.batchMatMul(s, 1, dA.data_ptr(), dB.data_ptr(), out.ptr, Batch, N, M, K, AK)
            _acc(O, out.host((Batch, N, M)), O.f64.batchMatMul(A, B, K), f"bmm {Batch}x{N}x{M}x{K}/{AK}")
        elif kind == 1:
            AN = (N + 3) // 4 * 4 + int(rng.choice([0, 4]))
            A = np.zeros((Batch, K, AN), np.float32); A[:, :, :N] = rng.standard_normal((Batch, K, N))
            B = rng.standard_normal((Batch, K, M)).astype(np.float32)
            out = G.Out(Batch * N * M)
            dA, dB = G.dev(A), G.dev(B)
            bm.batchMatMulT1(s, 1, dA.data_ptr(), dB.data_ptr(), out.ptr, Batch, N, AN, M, K)
            _acc(O, out.host((Batch, N, M)), O.f64.batchMatMulT1(A, B, N), f"bmmT1 {Batch}x{N}x{M}x{K}/{AN}")
        else:
            BM = max(1, M - int(rng.choice([0, 1, 2, 3])))
            A = rng.standard_normal((Batch, N, K)).astype(np.float32)
            B = rng.standard_normal((Batch, BM, K)).astype(np.float32)
            out = G.Out(Batch * N * M)
            dA, dB = G.dev(A), G.dev(B)
            bm.batchMatMulT2(s, 1, dA.data_ptr(), dB.data_ptr(), out.ptr, Batch, N, M, BM, K)
            C = out.host((Batch, N, M))
            _acc(O, C, O.f64.batchMatMulT2(A, B, M), f"bmmT2 {Batch}x{N}x{BM}/{M}x{K}")
            assert np.all(C[:, :, BM:] == 0)
    G.check_status(pkg)


def test_fuzz_conv(pkg, O, cuda):
    rng = np.random.default_rng(99)
    for case in range(20):
        N = int(rng.choice([4, 8, 12]))
        IH, IW = int(rng.integers(5, 20)), int(rng.integers(5, 20))
        IC = int(rng.choice([4, 8, 12, 32, 36, 64, 68]))
        OC = int(rng.choice([4, 8, 36, 64, 132, 260]))
        FH, FW = int(rng.integers(1, 6)), int(rng.integers(1, 6))
        FH, FW = min(FH, IH), min(FW, IW)
        sh, sw = int(rng.integers(1, 4)), int(rng.integers(1, 4))
        ph, pw = int(rng.integers(0, FH)), int(rng.integers(0, FW))
        X = rng.standard_normal((N, IH, IW, IC)).astype(np.float32)
        W = (rng.standard_normal((OC, FH, FW, IC)) / np.sqrt(FH * FW * IC)).astype(np.float32)
        OH, OW = (IH + 2 * ph - FH) // sh + 1, (IW + 2 * pw - FW) // sw + 1
        Y = G.conv(pkg, "conv3D_GemmR", X, W, sh, sw, ph, pw)
        _acc(O, Y, O.f64.conv3D(X, W, OH, OW, sh, sw, ph, pw), f"conv N{N} {IH}x{IW}x{IC}->{OC} f{FH}x{FW} s{sh},{sw} p{ph},{pw}")


def test_fuzz_biased(pkg, O, cuda):
    """Random shapes and widths through the fused bias entry points: same bits as the two-step sequence
    (contraction, then the restated linear_dual2D_row)."""
    mm, cv = pkg.cu32.Cuda_matMul, pkg.cu32.Cuda_conv3D
    rng = np.random.default_rng(77)
    s = [G.stream()]
    for case in range(24):
        N = int(rng.integers(1, 160)) * 4
        M = int(rng.integers(1, 160)) * 4
        K = int(rng.choice([4, 32, 36, 100, 516]))
        width = M - int(rng.choice([0, 0, 1, 2, 3]))
        A = rng.standard_normal((N, K)).astype(np.float32)
        B = rng.standard_normal((K, M)).astype(np.float32)
        B[:, width:] = 0
        bias = rng.standard_normal(M).astype(np.float32)
        plain = G.matmul(pkg, "AB", A, B, N, M, K)
        want = O.ref_loops.linear_dual2D_row(plain, bias, 1.0, 1.0, 0.0, width)
        dA, dB, db = G.dev(A), G.dev(B), G.dev(bias)
        out = G.Out(N * M)
        mm.matMul_biased(s, 1, dA.data_ptr(), dB.data_ptr(), out.ptr, db.data_ptr(), N, M, K, width)
        assert np.array_equal(out.host((N, M)), want), (N, M, K, width)
    for case in range(8):
        N, IH, IW = int(rng.integers(1, 5)), int(rng.integers(5, 14)), int(rng.integers(5, 14))
        IC, OC = int(rng.integers(1, 10)) * 4, int(rng.integers(1, 40)) * 4
        F = int(rng.choice([1, 3, 5])); st = int(rng.choice([1, 2])); pad = F // 2
        width = OC - int(rng.choice([0, 1, 3]))
        X = rng.standard_normal((N, IH, IW, IC)).astype(np.float32)
        W = (rng.standard_normal((OC, F, F, IC)) * 0.1).astype(np.float32)
        W[width:] = 0
        bias = rng.standard_normal(OC).astype(np.float32)
        OH, OW = (IH + 2 * pad - F) // st + 1, (IW + 2 * pad - F) // st + 1
        plain = G.conv(pkg, "conv3D_GemmR", X, W, st, st, pad, pad)
        want = O.ref_loops.linear_dual2D_row(plain.reshape(-1, OC), bias, 1.0, 1.0, 0.0, width).reshape(plain.shape)
        dX, dW, db = G.dev(X), G.dev(W), G.dev(bias)
        dCW = torch.empty(W.size, device="cuda")
        out = G.Out(N * OH * OW * OC)
        cv.conv3D_GemmR_biased(s, 1, dX.data_ptr(), IH, IW, dW.data_ptr(), dCW.data_ptr(), F, F, out.ptr, OH, OW, N, IC, OC,
                               st, st, pad, pad, db.data_ptr(), width)
        assert np.array_equal(out.host((N, OH, OW, OC)), want), (N, IH, IW, IC, OC, F, st, width)
    G.check_status(pkg)


def test_fuzz_deltax(pkg, O, cuda):
    """Random stride-1 geometries through the data-gradient entry point, each against the FP64 oracle."""
    dx = pkg.cu32.Cuda_dconv3D_deltaX
    rng = np.random.default_rng(88)
    s = [G.stream()]
    for case in range(30):
        N = int(rng.integers(1, 6))
        FH, FW = int(rng.integers(1, 8)), int(rng.integers(1, 8))
        ph, pw = int(rng.integers(0, FH)), int(rng.integers(0, FW))
        IH = int(rng.integers(max(1, FH - 2 * ph), 20 + FH))
        IW = int(rng.integers(max(1, FW - 2 * pw), 20 + FW))
        OH, OW = IH + 2 * ph - FH + 1, IW + 2 * pw - FW + 1
        if OH < 1 or OW < 1:
            continue
        IC, OC = int(rng.integers(1, 48)) * 4, int(rng.integers(1, 48)) * 4
        dY = rng.standard_normal((N, OH, OW, OC)).astype(np.float32)
        W = (rng.standard_normal((OC, FH, FW, IC)) * 0.1).astype(np.float32)
        ddY, dW = G.dev(dY), G.dev(W)
        out = G.Out(N * IH * IW * IC)
        dx.dconv3D_deltaX_s1(s, 1, ddY.data_ptr(), OH, OW, dW.data_ptr(), FH, FW, out.ptr, IH, IW, N, IC, OC, ph, pw)
        _acc(O, out.host((N, IH, IW, IC)), O.f64.deconv3D_deltaX_s1(dY, W, IH, IW, ph, pw),
             f"deltaX {(N, IH, IW, IC, OC, FH, FW, ph, pw)}")
    G.check_status(pkg)


def test_fuzz_deltax_strided(pkg, O, cuda):
    """Random geometries with strides up to 4 through the scatter-add-named and the kernel-split natives (which
    must agree bit for bit), each against the FP64 oracle.  Includes extents the stride does not divide, filters
    smaller than the stride and paddings up to the filter size."""
    dx = pkg.cu32.Cuda_dconv3D_deltaX
    rng = np.random.default_rng(89)
    s = [G.stream()]
    done = 0
    for case in range(60):
        N = int(rng.integers(1, 5))
        FH, FW = int(rng.integers(1, 8)), int(rng.integers(1, 8))
        sh, sw = int(rng.integers(1, 5)), int(rng.integers(1, 5))
        ph, pw = int(rng.integers(0, FH)), int(rng.integers(0, FW))
        IH = int(rng.integers(max(1, FH - 2 * ph), 24 + FH))
        IW = int(rng.integers(max(1, FW - 2 * pw), 24 + FW))
        if sh == 1 and sw == 1:
            sh = 2
        OH, OW = (IH + 2 * ph - FH) // sh + 1, (IW + 2 * pw - FW) // sw + 1
        IC, OC = int(rng.integers(1, 40)) * 4, int(rng.integers(1, 40)) * 4
        dY = rng.standard_normal((N, OH, OW, OC)).astype(np.float32)
        W = (rng.standard_normal((OC, FH, FW, IC)) * 0.1).astype(np.float32)
        ddY, dW = G.dev(dY), G.dev(W)
        geo = (N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw)
        out = G.Out(N * IH * IW * IC)
        dx.dconv3D_deltaX_crossAdd(s, 1, ddY.data_ptr(), OH, OW, dW.data_ptr(), FH, FW, out.ptr, IH, IW, N, IC, OC,
                                   sh, sw, ph, pw)
        got = out.host((N, IH, IW, IC))
        _acc(O, got, O.f64.deconv3D_deltaX(dY, W, IH, IW, sh, sw, ph, pw), f"strided deltaX {geo}")
        CFH, CFW = (FH + sh - 1) // sh, (FW + sw - 1) // sw
        dCW = torch.full((sh * sw * OC * CFH * CFW * IC,), float("nan"), device="cuda")
        dx.ks_remodev2(s[0], dW.data_ptr(), FH, FW, dCW.data_ptr(), CFH, CFW, OC, IC, sh, sw)
        out2 = G.Out(N * IH * IW * IC)
        dx.dconv3D_deltaX_ksImsR(s, 1, ddY.data_ptr(), OH, OW, dCW.data_ptr(), FH, FW, out2.ptr, IH, IW, N, IC, OC,
                                 sh, sw, ph, pw)
        assert np.array_equal(out2.host((N, IH, IW, IC)), got), f"kernel split vs in-place filter {geo}"
        done += 1
    assert done == 60
    G.check_status(pkg)


def test_fuzz_deltaw(pkg, O, cuda):
    """Random geometries (strides up to 3, any padding below the filter size, channel tails, pixel counts that are
    not multiples of the 32-pixel k-block, more split-K slices than k-blocks) through the weight-gradient natives."""
    dw = pkg.cu32.Cuda_dconv3D_deltaW
    rng = np.random.default_rng(90)
    s = [G.stream()]
    for case in range(40):
        N = int(rng.integers(1, 6))
        FH, FW = int(rng.integers(1, 6)), int(rng.integers(1, 6))
        sh, sw = int(rng.integers(1, 4)), int(rng.integers(1, 4))
        ph, pw = int(rng.integers(0, FH)), int(rng.integers(0, FW))
        IH = int(rng.integers(max(1, FH - 2 * ph), 18 + FH))
        IW = int(rng.integers(max(1, FW - 2 * pw), 18 + FW))
        OH, OW = (IH + 2 * ph - FH) // sh + 1, (IW + 2 * pw - FW) // sw + 1
        IC, OC = int(rng.integers(1, 40)) * 4, int(rng.integers(1, 40)) * 4
        GZ = int(rng.choice([1, 2, 3, 7, 16]))
        X = rng.standard_normal((N, IH, IW, IC)).astype(np.float32)
        dY = rng.standard_normal((N, OH, OW, OC)).astype(np.float32)
        dX_, ddY = G.dev(X), G.dev(dY)
        size = OC * FH * FW * IC
        out = G.Out(size)
        buf = torch.full((max(GZ - 1, 1) * size,), float("nan"), device="cuda")
        dw.dconv3D_deltaW_GemmSK(s, 1, GZ, dX_.data_ptr(), IH, IW, ddY.data_ptr(), OH, OW, out.ptr, buf.data_ptr(), FH, FW,
                                 N, IC, OC, sh, sw, ph, pw)
        if GZ > 1:
            dw.buf_summary(s[0], buf.data_ptr(), out.ptr, GZ - 1, size)
        _acc(O, out.host((OC, FH, FW, IC)), O.f64.deconv3D_deltaW(X, dY, FH, FW, sh, sw, ph, pw),
             f"deltaW {(N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw, GZ)}")
    G.check_status(pkg)
