"""The CPU oracle against (1) the golden fixtures produced by the reference's own CPU
routines, (2) those routines themselves when oracle/_ref is built, (3) hand-computed known
answers, and (4) its own FP64 layer."""
import ctypes

import numpy as np
import pytest

FP = ctypes.POINTER(ctypes.c_float)


def _p(a):
    return a.ctypes.data_as(FP)


def test_known_answers_matmul(O):
    # 2x3 * 3x2, integers: exact in any precision
    A = np.array([[1, 2, 3], [4, 5, 6]], np.float32)
    B = np.array([[7, 8], [9, 10], [11, 12]], np.float32)
    want = np.array([[58, 64], [139, 154]], np.float32)
    assert np.array_equal(O.ref_loops.multiply(A, B, 2, 2, 3), want)
    assert np.array_equal(O.ref_loops.multiplyT1(A.T.copy(), B, 2, 2, 3), want)
    assert np.array_equal(O.ref_loops.multiplyT2(A, B.T.copy(), 2, 2, 3), want)
    assert np.array_equal(O.f64.matMul(A, B), want.astype(np.float64))


def test_known_answers_conv(O):
    # 1 image 3x3x1 of ones, one 3x3 filter of ones, pad 1: each output counts the taps inside
    X = np.ones((1, 3, 3, 1), np.float32)
    W = np.ones((1, 3, 3, 1), np.float32)
    want = np.array([[4, 6, 4], [6, 9, 6], [4, 6, 4]], np.float32).reshape(1, 3, 3, 1)
    assert np.array_equal(O.ref_loops.conv3D_naive(X, W, 3, 3, 1, 1, 1, 1), want)
    assert np.array_equal(O.ref_loops.conv3D_img2col(X, W, 3, 3, 1, 1, 1, 1), want)
    assert np.array_equal(O.f64.conv3D(X, W, 3, 3, 1, 1, 1, 1), want.astype(np.float64))


def test_known_answers_kahan_and_remode(O):
    # 1 + 2^-24 * 4096 added naively in FP32 stays 1; compensated summation recovers 1 + 2^-12
    part, size = 4096, 4
    C = np.ones(size, np.float32)
    Cbuf = np.full((part, size), 2.0 ** -24, np.float32)
    out = O.ref_loops.buf_summary(Cbuf, C, part, size)
    assert np.allclose(out, 1.0 + 2.0 ** -12, rtol=0, atol=2.0 ** -23)
    naive = C.copy()
    for p in range(part):
        naive = naive + Cbuf[p]
    assert np.array_equal(naive, C)
    W = np.arange(2 * 2 * 3 * 4, dtype=np.float32).reshape(2, 2, 3, 4)  # OC, FH, FW, IC
    CW = O.ref_loops.kernel_remode(W)
    assert CW.shape == (2, 3, 4, 2)
    assert np.array_equal(CW, W.transpose(1, 2, 3, 0))


def test_golden_matmul_bmm_bit_exact(O, golden):
    data = np.load(golden.HERE / "golden_matmul_bmm.npz")
    for name, (kind, N, M, K) in golden.MATMUL_CASES.items():
        A, B = golden.golden_inputs(name, golden.matmul_shapes(kind, N, M, K))
        fn = {"AB": O.ref_loops.multiply, "T1": O.ref_loops.multiplyT1, "T2": O.ref_loops.multiplyT2}[kind]
        assert np.array_equal(fn(A, B, N, M, K), data[name]), name
    for name, (kind, Batch, d0, d1, d2, d3) in golden.BMM_CASES.items():
        shapes, _ = golden.bmm_shapes(kind, Batch, d0, d1, d2, d3)
        A, B = golden.golden_inputs(name, shapes)
        fn = {"AB": O.ref_loops.bmm, "T1": O.ref_loops.bmmT1, "T2": O.ref_loops.bmmT2}[kind]
        assert np.array_equal(fn(A, B, Batch, d0, d1, d2, d3), data[name]), name


def test_golden_conv_bit_exact(O, golden):
    path = golden.HERE / "golden_conv.npz"
    if not path.exists():
        pytest.skip("conv fixtures not generated yet")
    data = np.load(path)
    for name, (N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw) in golden.CONV_CASES.items():
        X, W = golden.golden_inputs(name, [(N, IH, IW, IC), (OC, FH, FW, IC)])
        OH, OW = golden.conv_out(IH, FH, sh, ph), golden.conv_out(IW, FW, sw, pw)
        assert np.array_equal(O.ref_loops.conv3D_naive(X, W, OH, OW, sh, sw, ph, pw), data[name + "/naive"]), name
        assert np.array_equal(O.ref_loops.conv3D_img2col(X, W, OH, OW, sh, sw, ph, pw), data[name + "/img2col"]), name


def test_against_reference_routines_when_built(O):
    """Random shapes, restatement vs the reference's compiled loops: bit-identical."""
    mm = O.ref_native("matmul")
    bm = O.ref_native("bmm")
    if mm is None or bm is None:
        pytest.skip("oracle/_ref not built here")
    rng = np.random.default_rng(11)
    for _ in range(6):
        N, M, K = (int(rng.integers(1, 60)) for _ in range(3))
        A = rng.random((N, K), dtype=np.float32) - 0.5
        B = rng.random((K, M), dtype=np.float32) - 0.5
        C = np.zeros((N, M), np.float32)
        mm.ref_cpu_multiply(_p(A), _p(B), _p(C), N, M, K)
        assert np.array_equal(C, O.ref_loops.multiply(A, B, N, M, K))
        At = np.ascontiguousarray(A.T)
        C = np.zeros((N, M), np.float32)
        mm.ref_cpu_multiplyT1(_p(At), _p(B), _p(C), N, M, K)
        assert np.array_equal(C, O.ref_loops.multiplyT1(At, B, N, M, K))
        Bt = np.ascontiguousarray(B.T)
        C = np.zeros((N, M), np.float32)
        mm.ref_cpu_multiplyT2(_p(A), _p(Bt), _p(C), N, M, K)
        assert np.array_equal(C, O.ref_loops.multiplyT2(A, Bt, N, M, K))
    Batch, N, CM, BM, K = 3, 17, 24, 22, 12
    A = rng.random((Batch, N, K), dtype=np.float32)
    B = rng.random((Batch, BM, K), dtype=np.float32)
    C = np.zeros((Batch, N, CM), np.float32)
    bm.ref_cpu_bmmT2(_p(A), _p(B), _p(C), Batch, N, CM, BM, K)
    assert np.array_equal(C, O.ref_loops.bmmT2(A, B, Batch, N, CM, BM, K))
    # the reference's own same-percent gate agrees with the restated one
    a = rng.random(1000, dtype=np.float32)
    b = a * (1 + 3e-5 * rng.standard_normal(1000).astype(np.float32))
    assert abs(mm.ref_cpu_samePercent(_p(a), _p(b), 1000) - O.same_percent(a, b, 1e-5)) < 1e-7


def test_fp32_loops_close_to_fp64(O):
    rng = np.random.default_rng(5)
    N, M, K = 48, 40, 256
    A = (rng.random((N, K), dtype=np.float32) * 2 - 1)
    B = (rng.random((K, M), dtype=np.float32) * 2 - 1)
    C64 = O.f64.matMul(A, B)
    assert O.frob_rel(O.ref_loops.multiply(A, B, N, M, K), C64) < 1e-6
    assert O.frob_rel(O.ref_loops.multiplyT2(A, B.T.copy(), N, M, K), O.f64.matMulT2(A, B.T.copy())) < 1e-6
    Batch = 3
    Ab = rng.standard_normal((Batch, N, K)).astype(np.float32)
    Bb = rng.standard_normal((Batch, K, M)).astype(np.float32)
    assert O.frob_rel(O.ref_loops.bmm(Ab, Bb, Batch, N, M, K, K), O.f64.batchMatMul(Ab, Bb)) < 1e-6
    Abt = np.ascontiguousarray(Ab.transpose(0, 2, 1))
    assert O.frob_rel(O.ref_loops.bmmT1(Abt, Bb, Batch, N, N, M, K), O.f64.batchMatMulT1(Abt, Bb)) < 1e-6
    X = rng.standard_normal((2, 10, 9, 8)).astype(np.float32)
    W = rng.standard_normal((6, 3, 5, 8)).astype(np.float32)
    OH, OW = (10 + 2 - 3) // 2 + 1, (9 + 4 - 5) // 1 + 1
    Y64 = O.f64.conv3D(X, W, OH, OW, 2, 1, 1, 2)
    assert O.frob_rel(O.ref_loops.conv3D_naive(X, W, OH, OW, 2, 1, 1, 2), Y64) < 1e-6
    assert O.frob_rel(O.ref_loops.conv3D_img2col(X, W, OH, OW, 2, 1, 1, 2), Y64) < 1e-7


def test_metrics(O):
    C64 = np.array([1.0, -2.0, 0.0, 4.0])
    C = C64 + np.array([1e-6, 0, 1e-9, 0])
    assert abs(O.frob_rel(C, C64) - np.sqrt(1e-12 + 1e-18) / np.sqrt(21)) < 1e-12
    assert O.elem_rel(C, C64, 1e-3) == pytest.approx(1e-6, rel=1e-3)
    rms = np.sqrt(21 / 4)
    assert O.elem_rel(C, C64) == pytest.approx(1e-6 / rms, rel=1e-3)   # error on the element 1.0 < rms
    a = np.array([1.0, 2.0, 3.0, 0.0], np.float32)
    b = np.array([1.0, 2.00001, 3.1, 0.0], np.float32)
    assert O.same_percent(a, b, 1e-5) == pytest.approx(0.75)
    assert O.zero_percent(a) == pytest.approx(0.25)
