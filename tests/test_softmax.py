"""Attention scores in one pass: P = softmax_rows(alpha * Q K^T) (cu32_batchMatMulT2_softmax).

The reference's attention block (nn/unit/complex/block/ImageMHA.java:67-68) runs batchMatMulT2, linear2D (the
1/sqrt(d) scale), and softmax2D = row_max + row_softmax + div2D_field (CudaFloat32EngineBase.java:5738-5775).
The fused entry point computes the same values per element - x' = fma(x, alpha, 0), e = expf(x' - max),
p = e * (1 / sum) - but sums each row in a different order and takes the maximum over the valid columns only, so
it is not a bit target: tolerance against the three-kernel sequence 2e-6 relative per element (a few units in the
last place of e and of the row sum), against the FP64 softmax of the FP64 scores relative Frobenius 1e-6 and
1e-4 elementwise (floored at the rms), the same budget as the contractions.
"""
import ctypes

import numpy as np
import pytest


def test_softmax_oracle_known_answers(O):
    x = np.array([[0.0, 0.0, 0.0, 0.0], [1.0, 2.0, 3.0, 0.0], [-1000.0, 0.0, -1000.0, -1000.0]], np.float32)
    y = O.ref_loops.softmax2D(x)
    assert np.array_equal(y[0], np.full(4, 0.25, np.float32))
    e = np.exp(np.array([1.0, 2.0, 3.0, 0.0]) - 3.0)
    assert np.allclose(y[1], e / e.sum(), rtol=3e-7, atol=0)
    assert np.array_equal(y[2], np.array([0, 1, 0, 0], np.float32))
    # pitch padding: columns >= width come out 0 and do not take part in the sum
    xp = np.array([[1.0, 2.0, 3.0, 0.0, 0.0, 0.0, 0.0, 0.0]], np.float32)
    yp = O.ref_loops.softmax2D(xp, 3)
    e3 = np.exp(np.array([1.0, 2.0, 3.0]) - 3.0)
    assert np.allclose(yp[0, :3], e3 / e3.sum(), rtol=3e-7, atol=0) and np.all(yp[0, 3:] == 0)
    rng = np.random.default_rng(5)
    X = (rng.standard_normal((40, 132)) * 3).astype(np.float32)
    assert np.abs(O.ref_loops.softmax2D(X, 130) - O.f64.softmax_rows(X.astype(np.float64), 1.0, 130)).max() <= 2e-7


def test_softmax_argument_errors_without_gpu(pkg):
    lib = pkg.cu32.load()
    s = (ctypes.c_int64 * 1)(0)
    P = lambda a: ctypes.cast(a, ctypes.POINTER(ctypes.c_float))
    ok = 0x10000
    f = lib.cu32_batchMatMulT2_softmax
    assert f(s, 1, None, P(ok), P(ok), 4, 8, 8, 8, 8, 0.125) == -1
    assert f(s, 1, P(ok), P(ok), P(ok), 0, 8, 8, 8, 8, 0.125) == -2
    assert f(s, 0, P(ok), P(ok), P(ok), 4, 8, 8, 8, 8, 0.125) == -3
    assert f(s, 1, P(ok), P(ok), P(ok), 4, 8, 4, 8, 8, 0.125) == -2      # CM < BM
    assert f(s, 1, P(ok), P(ok), P(ok), 4, 8, 8, 8, 6, 0.125) == -4      # K not a multiple of 4
    assert f(s, 1, P(ok), P(ok + 4), P(ok), 4, 8, 8, 8, 8, 0.125) == -4


CASES = [
    # Batch, N, CM, BM, K
    (6, 96, 80, 80, 64),         # one tile per row block
    (3, 130, 72, 68, 36),        # ragged rows, padded pitch, K tail
    (5, 256, 512, 512, 64),      # the benchmark's shape, fewer batches: rows span both TMEM buffers
    (2, 300, 512, 510, 64),      # pitch padding in the second buffer
    (2, 300, 512, 510, 128),     # reduction longer than one chunk: scaled product + in-place row softmax
    (9, 40, 260, 260, 32),       # second buffer nearly empty
    (2, 64, 516, 516, 64),       # rows longer than 512 columns: scaled product + in-place row softmax
    (2, 72, 256, 256, 192),      # reduction longer than one chunk: the same two-step path
]


def _fused(pkg, Q, Kt, CM, alpha):
    import gpu_util as G
    Batch, N, K = Q.shape
    BM = Kt.shape[1]
    dQ, dK = G.dev(Q), G.dev(Kt)
    out = G.Out(Batch * N * CM)
    pkg.cu32.Cuda_batchMatMul.batchMatMulT2_softmax([G.stream()], 1, dQ.data_ptr(), dK.data_ptr(), out.ptr, Batch, N, CM, BM,
                                                   K, alpha)
    P = out.host((Batch, N, CM))
    G.check_status(pkg)
    return P


@pytest.mark.gpu
@pytest.mark.parametrize("case", CASES)
def test_fused_scores_softmax(pkg, O, cuda, case):
    import gpu_util as G
    Batch, N, CM, BM, K = case
    rng = np.random.default_rng(sum(case))
    Q = rng.standard_normal((Batch, N, K)).astype(np.float32)
    Kt = rng.standard_normal((Batch, BM, K)).astype(np.float32)
    alpha = 1.0 / np.sqrt(K)
    P = _fused(pkg, Q, Kt, CM, alpha)
    assert np.isfinite(P).all()
    assert np.all(P[:, :, BM:] == 0)
    assert np.abs(P[:, :, :BM].astype(np.float64).sum(-1) - 1.0).max() <= 2e-6
    # against FP64
    S64 = O.f64.batchMatMulT2(Q, Kt, CM)
    P64 = O.f64.softmax_rows(S64, alpha, BM)
    rep = O.report(P, P64)
    assert rep["frob"] <= 1e-6 and rep["elem"] <= 1e-4, rep
    # against the engine's sequence on this library's scaled product: oracle restatement of softmax2D
    dQ, dK = G.dev(Q), G.dev(Kt)
    S = G.Out(Batch * N * CM)
    pkg.cu32.Cuda_batchMatMul.batchMatMulT2_scaled([G.stream()], 1, dQ.data_ptr(), dK.data_ptr(), S.ptr, Batch, N, CM, BM, K, alpha)
    Pseq = O.ref_loops.softmax2D(S.host((Batch, N, CM)), BM)
    G.check_status(pkg)
    big = Pseq > 1e-30
    assert (np.abs(P - Pseq)[big] / Pseq[big]).max() <= 2e-6
    assert np.abs(P - Pseq).max() <= 2e-7


@pytest.mark.gpu
def test_fused_scores_width_sweep_of_the_reference_test(pkg, O, cuda):
    """The reference's softmax test sweeps heights 2..20 x widths 2..256, heights 100..105 x widths 40..64 and
    1024 x 1024 (test/cuda/function/Cuda_function_softmax_test.java:60-66), inputs in [0, 0.7).  Here every width of
    that sweep (the engine's pitch = the width rounded up to 4) for a few of its heights, as the row length of the
    fused scores; verified on the device against the FP64 softmax of the FP64 scores: rows sum to 1, pad columns are
    zero, relative Frobenius error <= 1e-6."""
    import gpu_util as G
    torch = cuda
    g = torch.Generator(device="cuda").manual_seed(77)
    Batch, K = 3, 64
    alpha = 1.0 / 8.0
    worst = torch.zeros((), device="cuda", dtype=torch.float64)
    bad = torch.zeros((), device="cuda", dtype=torch.int64)
    out = G.Out(Batch * 105 * 1024)
    cases = [(h, w) for h in (2, 7, 20) for w in range(2, 257)] + [(h, w) for h in (100, 105) for w in range(40, 65)]
    cases.append((64, 1024))      # rows longer than the two TMEM buffers: the two-step path
    for (h, w) in cases:
        CM = (w + 3) // 4 * 4
        Q = torch.rand((Batch, h, K), device="cuda", generator=g) * 0.7
        Kt = torch.rand((Batch, w, K), device="cuda", generator=g) * 0.7
        P = out.view[:Batch * h * CM].view(Batch, h, CM)
        P.fill_(float("nan"))
        pkg.cu32.Cuda_batchMatMul.batchMatMulT2_softmax([G.stream()], 1, Q.data_ptr(), Kt.data_ptr(), P.data_ptr(), Batch, h, CM,
                                                       w, K, alpha)
        ref = torch.softmax((Q.double() @ Kt.double().transpose(1, 2)) * alpha, dim=-1)
        err = (P[:, :, :w].double() - ref).norm() / ref.norm()
        worst = torch.maximum(worst, torch.nan_to_num(err, nan=1.0))
        bad += (P[:, :, w:] != 0).sum() + (~torch.isfinite(P)).sum()
        bad += ((P[:, :, :w].double().sum(-1) - 1.0).abs() > 2e-6).sum()
    assert int(bad.item()) == 0
    assert float(worst.item()) <= 1e-6, float(worst.item())
    out.host((Batch * 105 * 1024,))   # canaries
    G.check_status(pkg)


@pytest.mark.gpu
def test_fused_scores_softmax_against_the_reference_kernels(pkg, O, cuda):
    """The reference's own kernels on this GPU: linear2D, row_max, row_softmax, div2D_field on this library's
    unscaled product (the product itself is compared with the reference elsewhere)."""
    import torch
    import gpu_util as G
    red, fun = O.ref_native("reduce"), O.ref_native("function")
    if red is None or fun is None or not hasattr(fun, "ref_gpu_div2D_field"):
        pytest.skip("oracle/_ref/libref_reduce.so / libref_function.so not built")
    FP = ctypes.POINTER(ctypes.c_float)
    ptr = lambda t: ctypes.cast(ctypes.c_void_p(t.data_ptr()), FP)
    for (Batch, N, CM, BM, K) in [(4, 128, 512, 512, 64), (3, 130, 72, 68, 36), (2, 300, 512, 510, 64), (2, 64, 516, 516, 128)]:
        rng = np.random.default_rng(K + N)
        Q = rng.standard_normal((Batch, N, K)).astype(np.float32)
        Kt = rng.standard_normal((Batch, BM, K)).astype(np.float32)
        alpha = float(np.float32(1.0 / np.sqrt(K)))
        P = _fused(pkg, Q, Kt, CM, alpha)
        dQ, dK = G.dev(Q), G.dev(Kt)
        rows = Batch * N
        S = torch.zeros((rows, CM), device="cuda")
        pkg.cu32.Cuda_batchMatMul.batchMatMulT2([G.stream()], 1, dQ.data_ptr(), dK.data_ptr(), S.data_ptr(), Batch, N, CM, BM, K)
        st = ctypes.c_longlong(G.stream())
        X = torch.empty_like(S)
        assert fun.ref_gpu_linear2D(st, ctypes.c_float(alpha), ptr(S), ctypes.c_float(0.0), ptr(X), rows * CM, BM, CM) == 0
        nextM = max(CM >> 8, 1)
        V = torch.zeros(nextM * ((rows + 3) // 4 * 4) + 16, device="cuda")
        mx = torch.zeros(rows + 16, device="cuda")
        Y = torch.empty_like(S)
        assert red.ref_gpu_row_max(st, ptr(X), rows, CM, ptr(V), ptr(mx), BM, CM) == 0
        assert red.ref_gpu_row_softmax(st, ptr(X), ptr(mx), ptr(Y), rows, CM, ptr(V), BM, CM) == 0
        assert fun.ref_gpu_div2D_field(st, ctypes.c_float(1.0), ptr(Y), ctypes.c_float(0.0), ctypes.c_float(1.0), ptr(V),
                                       ctypes.c_float(0.0), ctypes.c_float(0.0), CM, ptr(Y), rows * CM, BM, CM) == 0
        torch.cuda.synchronize()
        R = Y.cpu().numpy().reshape(Batch, N, CM)
        assert np.isfinite(R).all() and np.all(R[:, :, BM:] == 0)
        # the reference kernels and the oracle restatement of them agree (this is what pins the restatement)
        Rseq = O.ref_loops.softmax2D(X.cpu().numpy().reshape(Batch, N, CM), BM)
        assert np.abs(R - Rseq).max() <= 2e-7
        big = R > 1e-30
        assert (np.abs(P - R)[big] / R[big]).max() <= 2e-6
        assert np.abs(P - R).max() <= 3e-7
        G.check_status(pkg)


@pytest.mark.gpu
def test_attention_pair_with_fused_scores(pkg, O, cuda):
    """Config 3 at batch 16: P = softmax(Q K^T / 8) by the fused entry point, O = P V; against FP64 end to end."""
    import gpu_util as G
    w = pkg.workloads.config3(Batch=16)
    bm = pkg.cu32.Cuda_batchMatMul
    s = [G.stream()]
    dQ, dK, dV = w.Q.cuda(), w.K.cuda(), w.V.cuda()
    Pb = G.Out(w.Batch * w.L * w.L)
    alpha = 1.0 / (w.D ** 0.5)
    bm.batchMatMulT2_softmax(s, 1, dQ.data_ptr(), dK.data_ptr(), Pb.ptr, w.Batch, w.L, w.L, w.L, w.D, alpha)
    Oo = G.Out(w.Batch * w.L * w.D)
    bm.batchMatMul(s, 1, Pb.ptr, dV.data_ptr(), Oo.ptr, w.Batch, w.L, w.D, w.L, w.L)
    P = Pb.host((w.Batch, w.L, w.L))
    Oh = Oo.host((w.Batch, w.L, w.D))
    G.check_status(pkg)
    P64 = O.f64.softmax_rows(O.f64.batchMatMulT2(w.Q.numpy(), w.K.numpy()), alpha)
    rep = O.report(P, P64)
    assert rep["frob"] <= 1e-6 and rep["elem"] <= 1e-4, rep
    # the second product against FP64 on the FP32 P it was given (each operator has the 1e-6 budget) ...
    rep = O.report(Oh, O.f64.batchMatMul(P, w.V.numpy()))
    assert rep["frob"] <= 1e-6 and rep["elem"] <= 1e-4, rep
    # ... and the chain of the two against FP64 from the inputs: two budgets
    rep = O.report(Oh, np.matmul(P64, w.V.numpy().astype(np.float64)))
    assert rep["frob"] <= 2e-6 and rep["elem"] <= 2e-4, rep
