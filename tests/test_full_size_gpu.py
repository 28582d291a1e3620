"""Parity at the full benchmark configurations, and on the reference's own input distribution.

The configurations are too large for a full CPU oracle run inside a test, so each is checked by
  (1) sampled output rows / images / batches against the FP64 oracle on the CPU (the same tolerance as
      the small cases: relative Frobenius error <= 1e-6, elementwise <= 1e-4 with the rms floor), and
  (2) a checksum identity over the WHOLE output, evaluated in FP64: the sum over the columns (or the
      output channels) of the result equals the product with the column sums of the second operand, which
      catches a wrong or missing tile anywhere in the output.
The reference's own tests draw every input from [0, 1) (Cuda_matMul/test.cuh:19-24, ExRandom.java:341-347):
non-negative data is the worst case for an accumulator that truncates toward zero, so the long reductions
are checked on that distribution too, at the default chunk length.
"""
import numpy as np
import pytest
import torch

import gpu_util as G

pytestmark = pytest.mark.gpu

FROB_TOL, ELEM_TOL = 1e-6, 1e-4


def _accurate(O, C, C64, what):
    assert np.isfinite(C).all(), f"{what}: non-finite output (unwritten element?)"
    rep = O.report(C, C64)
    assert rep["frob"] <= FROB_TOL and rep["elem"] <= ELEM_TOL, f"{what}: {rep}"
    return rep


def _rel(a, b):
    return float((a - b).norm() / b.norm())


# ------------------------------------------------------------------ config 2, ragged
@pytest.mark.parametrize("form", ["AB", "T1", "T2"])
def test_config2_ragged_engine_padded(pkg, O, cuda, form):
    """Logical 8191 x 4097 x 3000 as the engine presents it: N=8192, M=4100, K=3000 with zero pad lanes in the
    inputs.  Tails in every dimension at full scale; the pad lanes of C come out as zeros."""
    w = pkg.workloads.config2_ragged(form)
    N, M, K = w.N, w.M, w.K
    lN, lM, lK = w.logical
    dA, dB = w.A.cuda(), w.B.cuda()
    out = G.Out(N * M)
    fn = {"AB": pkg.cu32.Cuda_matMul.matMul, "T1": pkg.cu32.Cuda_matMul.matMulT1, "T2": pkg.cu32.Cuda_matMul.matMulT2}[form]
    fn([G.stream()], 1, dA.data_ptr(), dB.data_ptr(), out.ptr, N, M, K)
    G.check_status(pkg)
    dC = out.view.view(N, M)
    A, B = w.A.numpy(), w.B.numpy()
    rows = np.unique(np.concatenate([np.linspace(0, lN - 1, 40).astype(int), [127, 128, 255, 256, lN - 1, N - 1]]))
    Arows = A[:, rows].T if form == "T1" else A[rows]
    Bm = B.T if form == "T2" else B
    C64 = Arows.astype(np.float64) @ Bm.astype(np.float64)
    C = dC[torch.as_tensor(rows, device="cuda")].cpu().numpy()
    _accurate(O, C, C64, f"config 2 ragged {form} sampled rows")
    # pad lanes: columns lM.. and rows lN.. are exact zeros
    assert bool((dC[:, lM:] == 0).all()) and bool((dC[lN:, :] == 0).all())
    # checksum over the whole output
    A64 = torch.from_numpy(A.T.copy() if form == "T1" else A).double().cuda()
    bsum = torch.from_numpy(Bm.astype(np.float64).sum(1)).cuda()
    assert _rel(dC.double().sum(1), A64 @ bsum) <= 1e-6, form
    out.host((N, M))   # canaries around the output


# ------------------------------------------------------------------ config 3 at batch 1024
def test_config3_full_batch(pkg, O, cuda):
    w = pkg.workloads.config3()
    bm = pkg.cu32.Cuda_batchMatMul
    s = [G.stream()]
    Bt, L, D = w.Batch, w.L, w.D
    dQ, dK, dV = w.Q.cuda(), w.K.cuda(), w.V.cuda()
    S = G.Out(Bt * L * L)
    bm.batchMatMulT2(s, 1, dQ.data_ptr(), dK.data_ptr(), S.ptr, Bt, L, L, L, D)
    G.check_status(pkg)
    dS = S.view.view(Bt, L, L)
    sample = [0, 1, 73, 511, 512, 1000, Bt - 1]
    Sh = dS[torch.as_tensor(sample, device="cuda")].cpu().numpy()
    _accurate(O, Sh, O.f64.batchMatMulT2(w.Q.numpy()[sample], w.K.numpy()[sample]), "config 3 Q K^T sampled batches")
    ksum = dK.double().sum(1)                                        # [Bt, D]
    assert _rel(dS.double().sum(2), torch.einsum("bnd,bd->bn", dQ.double(), ksum)) <= 1e-6
    # P = softmax rows in FP32, an input of the second product (the oracle sees the same FP32 P)
    dP = torch.softmax(dS / (D ** 0.5), dim=-1)
    Oo = G.Out(Bt * L * D)
    bm.batchMatMul(s, 1, dP.data_ptr(), dV.data_ptr(), Oo.ptr, Bt, L, D, L, L)
    G.check_status(pkg)
    dO = Oo.view.view(Bt, L, D)
    Ph = dP[torch.as_tensor(sample, device="cuda")].cpu().numpy()
    Oh = dO[torch.as_tensor(sample, device="cuda")].cpu().numpy()
    _accurate(O, Oh, O.f64.batchMatMul(Ph, w.V.numpy()[sample]), "config 3 P V sampled batches")
    vsum = dV.double().sum(2)                                        # [Bt, L]
    assert _rel(dO.double().sum(2), torch.einsum("bnk,bk->bn", dP.double(), vsum)) <= 1e-6
    S.host((Bt, L * L))      # canaries around both outputs
    Oo.host((Bt, L * D))


# ------------------------------------------------------------------ config 4 at 256 images
def test_config4_full_256_images(pkg, O, cuda):
    w = pkg.workloads.config4()
    d = w.dims
    cv = pkg.cu32.Cuda_conv3D
    dX, dW = w.X.cuda(), w.W.cuda()
    dCW = torch.empty(w.W.numel(), device="cuda")
    out = G.Out(d["N"] * d["OH"] * d["OW"] * d["OC"])
    s = [G.stream()]
    cv.kernel_remode(s[0], dW.data_ptr(), dCW.data_ptr(), d["FH"], d["FW"], d["OC"], d["IC"])
    cv.conv3D_GemmR(s, 1, dX.data_ptr(), d["IH"], d["IW"], dW.data_ptr(), dCW.data_ptr(), d["FH"], d["FW"], out.ptr,
                    d["OH"], d["OW"], d["N"], d["IC"], d["OC"], w.sh, w.sw, w.ph, w.pw)
    G.check_status(pkg)
    dY = out.view.view(d["N"], d["OH"], d["OW"], d["OC"])
    X, W = w.X.numpy(), w.W.numpy()
    for img in (0, 131, d["N"] - 1):
        Y64 = O.f64.conv3D(X[img:img + 1], W, d["OH"], d["OW"], w.sh, w.sw, w.ph, w.pw)
        _accurate(O, dY[img:img + 1].cpu().numpy(), Y64, f"config 4 image {img}")
    # checksum: the sum over output channels is the convolution with the channel-summed filter
    Wsum = W.astype(np.float64).sum(0, keepdims=True)
    want = O.f64.conv3D(X, Wsum, d["OH"], d["OW"], w.sh, w.sw, w.ph, w.pw)[..., 0]
    got = dY.double().sum(3).cpu().numpy()
    assert np.linalg.norm(got - want) / np.linalg.norm(want) <= 1e-6
    out.host((d["N"], d["OH"] * d["OW"] * d["OC"]))


# ------------------------------------------------------------------ config 5 at full K
def test_config5_full_size_through_the_engine_rule(pkg, O, cuda):
    """512 x 512 x 1 048 576 A^T*B with the split count the Java engine's rule gives, then SKbuf_summary."""
    w = pkg.workloads.config5()
    N, M, K = w.N, w.M, w.K
    mm = pkg.cu32.Cuda_matMul
    GZ = pkg.engine.matMulT1_gridZ(N, M, K, 148)
    assert GZ > 1
    dA, dB = w.A.cuda(), w.B.cuda()
    out = G.Out(N * M)
    buf = G.Out((GZ - 1) * N * M)
    s = [G.stream()]
    mm.matMulT1SK(s, 1, GZ, dA.data_ptr(), dB.data_ptr(), out.ptr, buf.ptr, N, M, K)
    mm.SKbuf_summary(s[0], buf.ptr, out.ptr, GZ - 1, N * M)
    G.check_status(pkg)
    C = out.host((N, M))
    assert np.isfinite(buf.host((GZ - 1, N * M))).all()
    A, B = w.A.numpy(), w.B.numpy()
    rows = np.linspace(0, N - 1, 12).astype(int)
    C64 = A[:, rows].astype(np.float64).T @ B.astype(np.float64)
    _accurate(O, C[rows], C64, "config 5 sampled rows")
    want = (dA.double().T @ dB.double().sum(1)).cpu().numpy()
    got = C.astype(np.float64).sum(1)
    assert np.linalg.norm(got - want) / np.linalg.norm(want) <= 1e-6


# ------------------------------------------------------------------ the reference's input distribution at long K
@pytest.mark.parametrize("K", [8192, 65536, 131072])
def test_nonnegative_inputs_long_reduction(pkg, O, cuda, K):
    """[0, 1) inputs, three forms, default chunk length: relative Frobenius error against FP64 within the
    budget, with the margin stated here (the truncating accumulator gives non-negative data a systematic
    error that does not grow with K)."""
    assert pkg.cu32.get_tune("kc") == 2
    N, M = 256, 384
    rng = np.random.default_rng(K)
    for form in ("AB", "T1", "T2"):
        sa, sb = G.mm_shapes(form, N, M, K)
        A, B = rng.random(sa, dtype=np.float32), rng.random(sb, dtype=np.float32)
        C = G.matmul(pkg, form, A, B, N, M, K)
        C64 = G.f64_matmul(O, form, A, B)
        rep = _accurate(O, C, C64, f"[0,1) {form} K={K}")
        assert rep["frob"] <= 9e-7, (form, K, rep)
        # and the reference's own acceptance gate against its FP32 loop is far away from failing
        if K == 8192:
            assert O.same_percent(C, G.ref_matmul(O, form, A, B, N, M, K), 1e-5) >= 0.999


def test_nonnegative_inputs_split_k(pkg, O, cuda):
    """The long-K weight-gradient shape on [0, 1) data through split-K and the compensated summation."""
    N, M, K = 128, 256, 262144
    rng = np.random.default_rng(11)
    A, B = rng.random((K, N), dtype=np.float32), rng.random((K, M), dtype=np.float32)
    GZ = pkg.engine.matMulT1_gridZ(N, M, K, 148)
    C, _, _ = G.matmul_sk(pkg, "T1", A, B, N, M, K, GZ)
    rep = _accurate(O, C, O.f64.matMulT1(A, B), f"[0,1) split-K GZ={GZ}")
    assert rep["frob"] <= 9e-7, rep


# ------------------------------------------------------------------ the reference's remainder sweep
@pytest.mark.parametrize("form", ["AB", "T1", "T2"])
def test_remainder_sweep_every_multiple_of_four(pkg, O, cuda, form):
    """The reference sweeps n, m over 1..255 (engine-padded to multiples of 4) at k around 128 and 512
    (Cuda_matMul_test.java:135-141).  Here: every N, M in 4, 8, ..., 260 x K in {128, 132, 512, 516},
    [0, 1) inputs, each product verified on the device against an FP64 product of the same operands;
    the worst case and the canaries around the output are checked once per K."""
    fn = {"AB": pkg.cu32.Cuda_matMul.matMul, "T1": pkg.cu32.Cuda_matMul.matMulT1, "T2": pkg.cu32.Cuda_matMul.matMulT2}[form]
    s = [G.stream()]
    g = torch.Generator(device="cuda").manual_seed(1234)
    DMAX, KMAX = 260, 516
    fa = torch.rand(DMAX * KMAX, device="cuda", generator=g)
    fb = torch.rand(DMAX * KMAX, device="cuda", generator=g)
    out = G.Out(DMAX * DMAX)
    for K in (128, 132, 512, 516):
        worst = torch.zeros((), device="cuda", dtype=torch.float64)
        bad = torch.zeros((), device="cuda", dtype=torch.int64)
        for N in range(4, DMAX + 1, 4):
            for M in range(4, DMAX + 1, 4):
                sa, sb = G.mm_shapes(form, N, M, K)
                A = fa[:sa[0] * sa[1]].view(sa)
                B = fb[:sb[0] * sb[1]].view(sb)
                C = out.view[:N * M].view(N, M)
                C.fill_(float("nan"))
                fn(s, 1, A.data_ptr(), B.data_ptr(), C.data_ptr(), N, M, K)
                A64 = A.double().T if form == "T1" else A.double()
                B64 = B.double().T if form == "T2" else B.double()
                ref = A64 @ B64
                err = (C.double() - ref).norm() / ref.norm()
                worst = torch.maximum(worst, torch.nan_to_num(err, nan=1.0))
                bad += (~torch.isfinite(C)).sum()
        assert int(bad.item()) == 0, (form, K)
        assert float(worst.item()) <= FROB_TOL, (form, K, float(worst.item()))
        out.host((DMAX * DMAX,))   # canaries
        G.check_status(pkg)


@pytest.mark.parametrize("form", ["AB", "T1", "T2"])
def test_batched_remainder_sweep_of_the_reference_test(pkg, O, cuda, form):
    """The reference's batched test sweeps K = 7..9, N = 1..82, M = 1..96 at batch 5 x 3
    (test/cuda/matMul/Cuda_batchMatMul_test.java:120-123) through the engine, which pads every tensor's last
    dimension to a multiple of 4 with zeros and leaves the others as they are.  Here the same sweep as the natives
    see it: every row count, the padded extents as pitches (AK, AN, CM), the true ones as logical sizes (BK, CN, BM);
    each product verified on the device against an FP64 product, pad columns of C asserted zero."""
    bm = pkg.cu32.Cuda_batchMatMul
    s = [G.stream()]
    g = torch.Generator(device="cuda").manual_seed(4321)
    Batch = 15
    pad4 = lambda x: (x + 3) // 4 * 4
    out = G.Out(Batch * 84 * 96)
    worst = torch.zeros((), device="cuda", dtype=torch.float64)
    bad = torch.zeros((), device="cuda", dtype=torch.int64)
    for K in (7, 8, 9):
        Kp = pad4(K)
        for N in range(1, 83, 3 if form != "AB" else 1):
            Np = pad4(N)
            for M in range(1, 97, 5):
                Mp = pad4(M)
                if form == "AB":      # A[b][N][Kp] (zeros beyond K), B[b][K][Mp] (zeros beyond M)
                    A = torch.rand((Batch, N, Kp), device="cuda", generator=g); A[:, :, K:] = 0
                    B = torch.rand((Batch, K, Mp), device="cuda", generator=g); B[:, :, M:] = 0
                    C = out.view[:Batch * N * Mp].view(Batch, N, Mp); C.fill_(float("nan"))
                    bm.batchMatMul(s, 1, A.data_ptr(), B.data_ptr(), C.data_ptr(), Batch, N, Mp, K, Kp)
                    ref = A.double() @ torch.nn.functional.pad(B.double(), (0, 0, 0, Kp - K))
                elif form == "T1":    # A[b][K][Np] (zeros beyond N), B[b][K][Mp]; C[b][N][Mp]
                    A = torch.rand((Batch, K, Np), device="cuda", generator=g); A[:, :, N:] = 0
                    B = torch.rand((Batch, K, Mp), device="cuda", generator=g); B[:, :, M:] = 0
                    C = out.view[:Batch * N * Mp].view(Batch, N, Mp); C.fill_(float("nan"))
                    bm.batchMatMulT1(s, 1, A.data_ptr(), B.data_ptr(), C.data_ptr(), Batch, N, Np, Mp, K)
                    ref = A.double().transpose(1, 2)[:, :N, :] @ B.double()
                else:                 # A[b][N][Kp], B[b][M][Kp] (zeros beyond K); C[b][N][Mp], columns M.. zero
                    A = torch.rand((Batch, N, Kp), device="cuda", generator=g); A[:, :, K:] = 0
                    B = torch.rand((Batch, M, Kp), device="cuda", generator=g); B[:, :, K:] = 0
                    C = out.view[:Batch * N * Mp].view(Batch, N, Mp); C.fill_(float("nan"))
                    bm.batchMatMulT2(s, 1, A.data_ptr(), B.data_ptr(), C.data_ptr(), Batch, N, Mp, M, Kp)
                    ref = torch.nn.functional.pad(A.double() @ B.double().transpose(1, 2), (0, Mp - M))
                    bad += (C[:, :, M:] != 0).sum()
                err = (C.double() - ref).norm() / ref.norm()
                worst = torch.maximum(worst, torch.nan_to_num(err, nan=1.0))
                bad += (~torch.isfinite(C)).sum()
    assert int(bad.item()) == 0, form
    assert float(worst.item()) <= FROB_TOL, (form, float(worst.item()))
    out.host((Batch * 84 * 96,))   # canaries
    G.check_status(pkg)

