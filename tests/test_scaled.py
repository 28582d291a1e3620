"""Batched contraction with the attention block's scale fused into the store.

The reference's attention block computes P = softmax(sdiv(sqrt(d), Q x K)) (nn/unit/complex/block/ImageMHA.java:67-68);
sdiv is linear2D(1/sqrt(d), X, 0) (Engine.java:4002), a second kernel over the scores.  The *_scaled entry points
store fma(product, alpha, 0) directly, which must be the bits of that two-kernel sequence."""
import ctypes

import numpy as np
import pytest


def test_linear2D_oracle(O):
    x = np.array([1.5, -2.25, 0.0, -0.0, 3.0e-39, 7.0], np.float32)
    a = np.float32(1.0 / np.sqrt(np.float32(64.0)))
    y = O.ref_loops.linear2D(a, x, 0.0)
    assert np.array_equal(y, (x.astype(np.float64) * np.float64(a)).astype(np.float32))   # one rounding
    assert not np.signbit(y[3])                                                          # -0 * a + 0 = +0
    y = O.ref_loops.linear2D(np.float32(3.0), x, np.float32(0.5))
    assert np.array_equal(y, (x.astype(np.float64) * 3.0 + 0.5).astype(np.float32))


def test_scaled_argument_errors_without_gpu(pkg):
    lib = pkg.cu32.load()
    s = (ctypes.c_int64 * 1)(0)
    P = lambda a: ctypes.cast(a, ctypes.POINTER(ctypes.c_float))
    ok = 0x10000
    f = lib.cu32_batchMatMulT2_scaled
    assert f(s, 1, None, P(ok), P(ok), 4, 8, 8, 8, 8, 0.125) == -1
    assert f(s, 1, P(ok), P(ok), P(ok), 0, 8, 8, 8, 8, 0.125) == -2
    assert f(s, 0, P(ok), P(ok), P(ok), 4, 8, 8, 8, 8, 0.125) == -3
    assert f(s, 1, P(ok), P(ok), P(ok), 4, 8, 4, 8, 8, 0.125) == -2      # CM < BM


def _run(pkg, form, A, B, dims, alpha=None):
    import gpu_util as G
    bm = pkg.cu32.Cuda_batchMatMul
    Batch, d0, d1, d2, d3 = dims
    dA, dB = G.dev(A), G.dev(B)
    rows, cols = (d0, d1) if form != "T1" else (d0, d2)
    out = G.Out(Batch * rows * cols)
    name = {"AB": "batchMatMul", "T1": "batchMatMulT1", "T2": "batchMatMulT2"}[form]
    args = [[G.stream()], 1, dA.data_ptr(), dB.data_ptr(), out.ptr, Batch, d0, d1, d2, d3]
    if alpha is None:
        getattr(bm, name)(*args)
    else:
        getattr(bm, name + "_scaled")(*args, alpha)
    C = out.host((Batch, rows, cols))
    G.check_status(pkg)
    return C


@pytest.mark.gpu
@pytest.mark.parametrize("form,dims", [
    ("T2", (6, 96, 80, 80, 64)),       # Q x K^T: N=96, CM=BM=80, K=64
    ("T2", (3, 130, 72, 68, 36)),      # ragged, padded output pitch
    ("T1", (5, 64, 64, 96, 48)),       # the form the reference's own attention block calls (CN, AN, M, K)
    ("AB", (4, 100, 64, 72, 72)),      # P x V
    ("T2", (64, 512, 512, 512, 64)),   # the attention shape of the benchmark, fewer batches
])
def test_scaled_is_the_product_followed_by_the_scale_kernel(pkg, O, cuda, form, dims):
    import gpu_util as G
    rng = np.random.default_rng(41)
    Batch, d0, d1, d2, d3 = dims
    if form == "T2":
        A = rng.standard_normal((Batch, d0, d3)).astype(np.float32); B = rng.standard_normal((Batch, d2, d3)).astype(np.float32)
        want64 = np.einsum("bnk,bmk->bnm", A.astype(np.float64), B.astype(np.float64))
        want64 = np.pad(want64, ((0, 0), (0, 0), (0, d1 - d2)))
    elif form == "T1":
        A = rng.standard_normal((Batch, d3, d1)).astype(np.float32); B = rng.standard_normal((Batch, d3, d2)).astype(np.float32)
        want64 = np.einsum("bkn,bkm->bnm", A.astype(np.float64)[:, :, :d0], B.astype(np.float64))
    else:
        A = rng.standard_normal((Batch, d0, d3)).astype(np.float32); B = rng.standard_normal((Batch, d2, d1)).astype(np.float32)
        want64 = np.einsum("bnk,bkm->bnm", A.astype(np.float64)[:, :, :d2], B.astype(np.float64))
    alpha = float(np.float32(1.0) / np.sqrt(np.float32(d3)))
    plain = _run(pkg, form, A, B, dims)
    fused = _run(pkg, form, A, B, dims, alpha)
    assert np.array_equal(fused, O.ref_loops.linear2D(alpha, plain, 0.0))        # bits of the two-kernel sequence
    rep = O.report(fused, want64 * np.float64(np.float32(alpha)))
    assert rep["frob"] <= 1e-6 and rep["elem"] <= 1e-4, rep
    ref = O.ref_native("function")
    if ref is not None and hasattr(ref, "ref_gpu_linear2D"):
        # the reference's own linear2D kernel applied to the unscaled product
        t = G.dev(plain)
        n = plain.size
        cols = plain.shape[-1]
        assert ref.ref_gpu_linear2D(ctypes.c_longlong(G.stream()), ctypes.c_float(alpha), ctypes.c_void_p(t.data_ptr()),
                                    ctypes.c_float(0.0), ctypes.c_void_p(t.data_ptr()), n, cols, cols) == 0
        cuda.cuda.synchronize()
        assert np.array_equal(t.cpu().numpy(), fused)


@pytest.mark.gpu
def test_attention_scores_through_the_engine_mirror(pkg, O, cuda):
    """Q [Batch, d, L] and K [Batch, d, L] as the reference's attention block lays them out: scores = Q^T K / sqrt(d)."""
    import gpu_util as G
    torch = cuda
    eng = pkg.engine.Cu32Engine(148, lambda n: (0, None), [G.stream()])
    rng = np.random.default_rng(42)
    Batch, d, L = 8, 32, 96
    Q = rng.standard_normal((Batch, d, L)).astype(np.float32)
    K = rng.standard_normal((Batch, d, L)).astype(np.float32)
    dQ, dK = G.dev(Q), G.dev(K)
    out = G.Out(Batch * L * L)
    eng.batchMatMulT1_sdiv(out.ptr, dQ.data_ptr(), dK.data_ptr(), Batch, L, L, L, d, float(np.sqrt(d)))
    G.check_status(pkg)
    S = out.host((Batch, L, L))
    alpha = np.float32(1.0) / np.float32(np.sqrt(d))
    want = np.einsum("bkn,bkm->bnm", Q.astype(np.float64), K.astype(np.float64)) * np.float64(alpha)
    rep = O.report(S, want)
    assert rep["frob"] <= 1e-6 and rep["elem"] <= 1e-4, rep
