"""Parity of the CUDA path, called through the C ABI, with the CPU oracle.

Tolerances (FP32-accurate entry points), against the FP64 oracle:
    relative Frobenius error   <= 1e-6
    elementwise relative error <= 1e-4   (denominator floored at the rms of the oracle output:
                                          outputs are signed sums, some land next to zero, and an
                                          unfloored ratio is unbounded for any FP32 implementation)
and, on the non-negative inputs the reference's tests use, the reference's own acceptance gate
against its FP32 CPU loops:
    >= 99.9 % of elements within |a-b|/|a+b| < 1e-5          (Cuda_matMul/test.cuh:48-58, :328)
The TF32 fast mode (`_mma` entry points) has its own looser tolerance: frob <= 1e-3, elem <= 5e-3.
Bandwidth kernels (filter remode, split-K buffer summation) are bit-exact.
"""
import numpy as np
import pytest
import torch

import gpu_util as G

pytestmark = pytest.mark.gpu

FROB_TOL, ELEM_TOL = 1e-6, 1e-4
FAST_FROB_TOL, FAST_ELEM_TOL = 1e-3, 5e-3


def assert_accurate(O, C, C64, what=""):
    assert np.isfinite(C).all(), f"{what}: non-finite output (unwritten element?)"
    rep = O.report(C, C64)
    assert rep["frob"] <= FROB_TOL and rep["elem"] <= ELEM_TOL, f"{what}: {rep}"
    return rep


# ------------------------------------------------------------------ golden fixtures
def test_golden_matmul(pkg, O, cuda, golden):
    data = np.load(golden.HERE / "golden_matmul_bmm.npz")
    for name, (kind, N, M, K) in golden.MATMUL_CASES.items():
        A, B = golden.golden_inputs(name, golden.matmul_shapes(kind, N, M, K))
        C = G.matmul(pkg, kind, A, B, N, M, K)
        assert O.same_percent(C, data[name], 1e-5) >= 0.999, name
        assert_accurate(O, C, G.f64_matmul(O, kind, A, B), name)


def test_golden_bmm(pkg, O, cuda, golden):
    data = np.load(golden.HERE / "golden_matmul_bmm.npz")
    bm = pkg.cu32.Cuda_batchMatMul
    for name, (kind, Batch, d0, d1, d2, d3) in golden.BMM_CASES.items():
        shapes, cshape = golden.bmm_shapes(kind, Batch, d0, d1, d2, d3)
        A, B = golden.golden_inputs(name, shapes)
        dA, dB = G.dev(A), G.dev(B)
        out = G.Out(int(np.prod(cshape)))
        fn = {"AB": bm.batchMatMul, "T1": bm.batchMatMulT1, "T2": bm.batchMatMulT2}[kind]
        fn([G.stream()], 1, dA.data_ptr(), dB.data_ptr(), out.ptr, Batch, d0, d1, d2, d3)
        C = out.host(cshape)
        G.check_status(pkg)
        assert np.isfinite(C).all(), name
        assert O.same_percent(C, data[name], 1e-5) >= 0.999, name
        # the batched tests of the reference use an absolute 1e-2 criterion (Cuda_batchMatMul/test.cuh:69-89)
        assert O.same_percent(C, data[name], 1e-2, absolute=True) == 1.0, name
        if kind == "T2":  # pad columns BM..CM-1 come out zero
            assert np.all(C[:, :, d2:] == 0), name


def test_golden_conv(pkg, O, cuda, golden):
    path = golden.HERE / "golden_conv.npz"
    if not path.exists():
        pytest.skip("conv fixtures not generated")
    data = np.load(path)
    for name, (N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw) in golden.CONV_CASES.items():
        X, W = golden.golden_inputs(name, [(N, IH, IW, IC), (OC, FH, FW, IC)])
        Y = G.conv(pkg, "conv3D_GemmR", X, W, sh, sw, ph, pw)
        # the reference's conv gate: relative 1e-3 on >= 99 % and identical zero share (Cuda_conv3D/test.cuh:38-57, :913)
        assert O.same_percent(Y, data[name + "/img2col"], 1e-3) >= 0.99, name
        assert O.same_percent(Y, data[name + "/naive"], 1e-3) >= 0.99, name
        assert O.zero_percent(Y) == O.zero_percent(data[name + "/img2col"]), name


# ------------------------------------------------------------------ matMul family
SHAPES = [
    (4, 4, 4), (4, 8, 36), (8, 4, 32), (128, 128, 32), (128, 128, 64), (132, 124, 100), (256, 256, 256),
    (60, 516, 132), (516, 60, 128), (300, 260, 516), (1024, 64, 96), (64, 1024, 40), (388, 392, 1028),
]


@pytest.mark.parametrize("form", ["AB", "T1", "T2"])
def test_matmul_shapes(pkg, O, cuda, form):
    for i, (N, M, K) in enumerate(SHAPES):
        sa, sb = G.mm_shapes(form, N, M, K)
        A, B = G.rand_pm1(sa, 100 + i), G.rand_pm1(sb, 200 + i)
        C = G.matmul(pkg, form, A, B, N, M, K)
        assert_accurate(O, C, G.f64_matmul(O, form, A, B), f"{form} {N}x{M}x{K}")


def test_matmul_remainder_sweep(pkg, O, cuda):
    """A slice of the reference's exhaustive sweep (n, m in 1..255 padded to 4, k around 128 and
    512: Cuda_matMul_test.java:135-141), subsampled to keep the run short."""
    rng = np.random.default_rng(1)
    for _ in range(24):
        N = int(rng.integers(1, 64)) * 4
        M = int(rng.integers(1, 64)) * 4
        K = int(rng.choice([128, 132, 512, 516]))
        form = ["AB", "T1", "T2"][int(rng.integers(0, 3))]
        sa, sb = G.mm_shapes(form, N, M, K)
        A, B = rng.random(sa, dtype=np.float32), rng.random(sb, dtype=np.float32)  # [0,1) like the reference tests
        C = G.matmul(pkg, form, A, B, N, M, K)
        assert_accurate(O, C, G.f64_matmul(O, form, A, B), f"{form} {N}x{M}x{K}")
        assert O.same_percent(C, G.ref_matmul(O, form, A, B, N, M, K), 1e-5) >= 0.999


@pytest.mark.parametrize("tile", [0, 1, 2, 3, 4, 5])
def test_every_tile_configuration(pkg, O, cuda, tile):
    pkg.cu32.tune("tile", tile)
    for form in ("AB", "T1", "T2"):
        for (N, M, K) in [(256, 256, 128), (520, 772, 200), (132, 68, 64)]:
            sa, sb = G.mm_shapes(form, N, M, K)
            A, B = G.rand_pm1(sa, 7), G.rand_pm1(sb, 8)
            C = G.matmul(pkg, form, A, B, N, M, K)
            assert_accurate(O, C, G.f64_matmul(O, form, A, B), f"tile {tile} {form} {N}x{M}x{K}")
    # the same tile through the batched, split-K and convolution paths
    rng = np.random.default_rng(tile)
    Batch, N, M, K = 3, 200, 196, 100
    A = rng.standard_normal((Batch, N, K)).astype(np.float32)
    B = rng.standard_normal((Batch, K, M)).astype(np.float32)
    out = G.Out(Batch * N * M)
    dA, dB = G.dev(A), G.dev(B)
    pkg.cu32.Cuda_batchMatMul.batchMatMul([G.stream()], 1, dA.data_ptr(), dB.data_ptr(), out.ptr, Batch, N, M, K, K)
    assert_accurate(O, out.host((Batch, N, M)), O.f64.batchMatMul(A, B), f"tile {tile} bmm")
    A, B = G.rand_pm1((1028, 132), 3), G.rand_pm1((1028, 260), 4)
    C, _, _ = G.matmul_sk(pkg, "T1", A, B, 132, 260, 1028, 4)
    assert_accurate(O, C, O.f64.matMulT1(A, B), f"tile {tile} split-K T1")
    X = rng.standard_normal((4, 12, 12, 36)).astype(np.float32)
    W = rng.standard_normal((40, 3, 3, 36)).astype(np.float32) * 0.1
    assert_accurate(O, G.conv(pkg, "conv3D_GemmR", X, W, 1, 1, 1, 1), O.f64.conv3D(X, W, 12, 12, 1, 1, 1, 1), f"tile {tile} conv")


@pytest.mark.parametrize("kc", [1, 2, 3, 8, 1000])
def test_chunk_lengths(pkg, O, cuda, kc):
    """Any chunk length gives the same product (accuracy bound checked at moderate K)."""
    pkg.cu32.tune("kc", kc)
    N, M, K = 256, 384, 1000
    A, B = G.rand_pm1((N, K), 1), G.rand_pm1((K, M), 2)
    C = G.matmul(pkg, "AB", A, B, N, M, K)
    rep = O.report(C, O.f64.matMul(A, B))
    assert rep["frob"] <= 1e-5 and np.isfinite(C).all(), rep


def test_results_repeat_bit_for_bit_on_every_tile(pkg, O, cuda):
    """Every tile shape walks K in the same order, so all of them return the same bits, run after run.
    A hand-over that is not properly fenced (a lo tile read by the tensor core while a store to it is still in
    flight, a TMEM buffer recycled early) shows up here as a few hundred elements that differ in one run of many,
    long before it costs enough accuracy to fail a tolerance."""
    w = pkg.workloads.config4(N=8)
    X, W = w.X.numpy(), w.W.numpy()
    A, B = G.rand_pm1((1024, 2304), 1), G.rand_pm1((2304, 520), 2)
    cases = {"conv": lambda: G.conv(pkg, "conv3D_GemmR", X, W, 1, 1, 1, 1),
             "matMul": lambda: G.matmul(pkg, "AB", A, B, 1024, 520, 2304)}
    for name, fn in cases.items():
        pkg.cu32.tune("tile", 4)
        base = fn()
        for tile in (0, 1, 2, 3, 4, 5):
            pkg.cu32.tune("tile", tile)
            for rep in range(16):
                Y = fn()
                assert np.array_equal(Y, base), (name, tile, rep, int((Y != base).sum()), float(np.abs(Y - base).max()))


def test_extreme_extents(pkg, O, cuda):
    """Long thin problems: more row tiles, batches and split-K slices than a 16-bit grid axis could index,
    and a reduction of a million - the extents the tile index and the tensor maps have to carry."""
    torch = cuda
    mm, bm = pkg.cu32.Cuda_matMul, pkg.cu32.Cuda_batchMatMul
    s = [G.stream()]
    g = torch.Generator(device="cuda").manual_seed(99)
    # 1 Mi + 4 rows, 8 columns: 8193 row tiles of the 128-row tile
    N, M, K = (1 << 20) + 4, 8, 36
    A = torch.randn(N, K, device="cuda", generator=g); B = torch.randn(K, M, device="cuda", generator=g)
    C = torch.full((N, M), float("nan"), device="cuda")
    mm.matMul(s, 1, A.data_ptr(), B.data_ptr(), C.data_ptr(), N, M, K)
    ref = A.double() @ B.double()
    assert ((C.double() - ref).norm() / ref.norm()).item() <= 1e-6 and bool(torch.isfinite(C).all())
    # 70 000 batches of 4x4x4
    Bt = 70000
    Q = torch.randn(Bt, 4, 4, device="cuda", generator=g); Kt = torch.randn(Bt, 4, 4, device="cuda", generator=g)
    S = torch.full((Bt, 4, 4), float("nan"), device="cuda")
    bm.batchMatMulT2(s, 1, Q.data_ptr(), Kt.data_ptr(), S.data_ptr(), Bt, 4, 4, 4, 4)
    ref = Q.double() @ Kt.double().transpose(1, 2)
    assert ((S.double() - ref).norm() / ref.norm()).item() <= 1e-6 and bool(torch.isfinite(S).all())
    # K = 1 Mi through split-K with the engine's own slice count, 64x64 output
    N, M, K = 64, 64, 1 << 20
    A = torch.randn(K, N, device="cuda", generator=g); B = torch.randn(K, M, device="cuda", generator=g)
    GZ = pkg.engine.matMulT1_gridZ(N, M, K, 148)
    assert GZ > 1
    C = torch.full((N, M), float("nan"), device="cuda"); Cbuf = torch.full((GZ - 1, N, M), float("nan"), device="cuda")
    mm.matMulT1SK(s, 1, GZ, A.data_ptr(), B.data_ptr(), C.data_ptr(), Cbuf.data_ptr(), N, M, K)
    mm.SKbuf_summary(s[0], Cbuf.data_ptr(), C.data_ptr(), GZ - 1, N * M)
    ref = A.double().T @ B.double()
    assert ((C.double() - ref).norm() / ref.norm()).item() <= 1e-6 and bool(torch.isfinite(C).all())
    G.check_status(pkg)


def test_config1_full_size(pkg, O, cuda):
    w = pkg.workloads.config1()
    A, B = w.A.numpy(), w.B.numpy()
    C = G.matmul(pkg, "AB", A, B, w.N, w.M, w.K)
    assert_accurate(O, C, O.f64.matMul(A, B), "config 1")
    # against the reference's FP32 loop: both are FP32-accurate, so they agree to FP32 noise
    Cref = O.ref_loops.multiply(A, B, w.N, w.M, w.K)
    assert O.frob_rel(C, Cref) <= 2e-6
    assert O.frob_rel(C, O.f64.matMul(A, B)) <= O.frob_rel(Cref, O.f64.matMul(A, B))   # and closer to FP64 than it


@pytest.mark.parametrize("form", ["AB", "T1", "T2"])
@pytest.mark.parametrize("GZ", [2, 4, 16])
def test_splitk_protocol(pkg, O, cuda, form, GZ):
    """slice 0 -> C, slice z -> Cbuf[z-1]; every partial is written (no NaN left), their
    FP64 sum is the product, and SKbuf_summary leaves the product in C."""
    N, M, K = 132, 260, 2052
    sa, sb = G.mm_shapes(form, N, M, K)
    A, B = G.rand_pm1(sa, 31), G.rand_pm1(sb, 32)
    C, C0, Cbuf = G.matmul_sk(pkg, form, A, B, N, M, K, GZ)
    assert np.isfinite(C0).all() and np.isfinite(Cbuf).all()
    C64 = G.f64_matmul(O, form, A, B)
    assert O.frob_rel(C0.astype(np.float64) + Cbuf.astype(np.float64).sum(0), C64) <= FROB_TOL
    assert_accurate(O, C, C64, f"split-K {form} GZ={GZ}")
    assert np.array_equal(C, O.ref_loops.buf_summary(Cbuf.reshape(GZ - 1, -1), C0.ravel(), GZ - 1, N * M).reshape(N, M))


def test_splitk_more_slices_than_kblocks(pkg, O, cuda):
    N, M, K = 64, 64, 96   # 3 k-blocks, 16 slices: empty slices must write zeros
    A, B = G.rand_pm1((N, K), 1), G.rand_pm1((K, M), 2)
    C, C0, Cbuf = G.matmul_sk(pkg, "AB", A, B, N, M, K, 16)
    assert np.isfinite(Cbuf).all()
    assert_accurate(O, C, O.f64.matMul(A, B), "split-K with empty slices")


def test_engine_split_decision_end_to_end(pkg, O, cuda):
    """Drive the natives the way CudaFloat32EngineBase.matMulT1 does for a weight-gradient shape."""
    keep = []

    def malloc(n):
        t = torch.empty(n, device="cuda")
        keep.append(t)
        return t.data_ptr(), t
    eng = pkg.engine.Cu32Engine(148, malloc, [G.stream()])
    N, M, K = 256, 128, 16384
    g = torch.Generator().manual_seed(5)
    A = torch.randn((K, N), generator=g) * 0.01
    B = torch.randn((K, M), generator=g) * 0.01
    dA, dB = A.cuda(), B.cuda()
    out = G.Out(N * M)
    gz = eng.matMulT1(out.ptr, dA.data_ptr(), dB.data_ptr(), N, M, K)
    assert gz > 1
    C = out.host((N, M))
    G.check_status(pkg)
    assert_accurate(O, C, O.f64.matMulT1(A.numpy(), B.numpy()), f"engine matMulT1 gz={gz}")


def test_skbuf_summary_bit_exact(pkg, O, cuda):
    rng = np.random.default_rng(3)
    for part, size in [(1, 4), (3, 252), (15, 4096), (35, 1028)]:
        C = rng.standard_normal(size).astype(np.float32)
        Cbuf = (rng.standard_normal((part, size)) * 10.0 ** rng.integers(-6, 3, (part, 1))).astype(np.float32)
        dC, dB = G.dev(C), G.dev(Cbuf)
        pkg.cu32.Cuda_matMul.SKbuf_summary(G.stream(), dB.data_ptr(), dC.data_ptr(), part, size)
        torch.cuda.synchronize()
        assert np.array_equal(dC.cpu().numpy(), O.ref_loops.buf_summary(Cbuf, C, part, size))


@pytest.mark.parametrize("form", ["AB", "T1", "T2"])
def test_tf32_fast_mode(pkg, O, cuda, form):
    N, M, K = 256, 260, 512
    sa, sb = G.mm_shapes(form, N, M, K)
    A, B = G.rand_pm1(sa, 41), G.rand_pm1(sb, 42)
    C = G.matmul(pkg, form, A, B, N, M, K, mma=True)
    rep = O.report(C, G.f64_matmul(O, form, A, B))
    assert rep["frob"] <= FAST_FROB_TOL and rep["elem"] <= FAST_ELEM_TOL, rep
    assert rep["frob"] > 1e-5   # it really is the single-pass mode


# ------------------------------------------------------------------ batched family
def test_batched_forms(pkg, O, cuda):
    bm = pkg.cu32.Cuda_batchMatMul
    rng = np.random.default_rng(9)
    s = [G.stream()]
    # batchMatMul: N not a multiple of 4, AK > BK (A rows padded)
    for (Batch, N, M, BK, AK) in [(3, 37, 64, 30, 32), (8, 128, 132, 64, 64), (2, 250, 260, 100, 100), (5, 512, 64, 512, 512)]:
        A = rng.standard_normal((Batch, N, AK)).astype(np.float32)
        B = rng.standard_normal((Batch, BK, M)).astype(np.float32)
        out = G.Out(Batch * N * M)
        dA, dB = G.dev(A), G.dev(B)
        for fn in (bm.batchMatMul, bm.batchMatMul_texture):
            fn(s, 1, dA.data_ptr(), dB.data_ptr(), out.ptr, Batch, N, M, BK, AK)
            C = out.host((Batch, N, M))
            assert_accurate(O, C, O.f64.batchMatMul(A, B, BK), f"bmm {Batch}x{N}x{M}x{BK}")
    # batchMatMulT1: AN > CN
    for (Batch, CN, AN, M, K) in [(2, 50, 52, 24, 40), (4, 128, 128, 128, 96), (3, 130, 132, 68, 260)]:
        A = rng.standard_normal((Batch, K, AN)).astype(np.float32)
        B = rng.standard_normal((Batch, K, M)).astype(np.float32)
        out = G.Out(Batch * CN * M)
        dA, dB = G.dev(A), G.dev(B)
        bm.batchMatMulT1(s, 1, dA.data_ptr(), dB.data_ptr(), out.ptr, Batch, CN, AN, M, K)
        C = out.host((Batch, CN, M))
        assert_accurate(O, C, O.f64.batchMatMulT1(A, B, CN), f"bmmT1 {Batch}x{CN}x{M}x{K}")
    # batchMatMulT2: CM > BM (pad columns written as zero)
    for (Batch, N, CM, BM, K) in [(4, 33, 68, 66, 16), (2, 512, 512, 512, 64), (3, 100, 132, 130, 36)]:
        A = rng.standard_normal((Batch, N, K)).astype(np.float32)
        B = rng.standard_normal((Batch, BM, K)).astype(np.float32)
        out = G.Out(Batch * N * CM)
        dA, dB = G.dev(A), G.dev(B)
        for fn in (bm.batchMatMulT2, bm.batchMatMulT2_texture):
            fn(s, 1, dA.data_ptr(), dB.data_ptr(), out.ptr, Batch, N, CM, BM, K)
            C = out.host((Batch, N, CM))
            assert_accurate(O, C, O.f64.batchMatMulT2(A, B, CM), f"bmmT2 {Batch}x{N}x{BM}x{K}")
            assert np.all(C[:, :, BM:] == 0)
    G.check_status(pkg)


def test_attention_shaped_pair_reduced(pkg, O, cuda):
    """Config 3 at batch 16: S = Q K^T, P = softmax rows (FP32, as an input), O = P V."""
    w = pkg.workloads.config3(Batch=16)
    bm = pkg.cu32.Cuda_batchMatMul
    s = [G.stream()]
    dQ, dK, dV = w.Q.cuda(), w.K.cuda(), w.V.cuda()
    S = G.Out(w.Batch * w.L * w.L)
    bm.batchMatMulT2(s, 1, dQ.data_ptr(), dK.data_ptr(), S.ptr, w.Batch, w.L, w.L, w.L, w.D)
    Sh = S.host((w.Batch, w.L, w.L))
    assert_accurate(O, Sh, O.f64.batchMatMulT2(w.Q.numpy(), w.K.numpy()), "Q K^T")
    P = pkg.workloads.softmax_rows(torch.from_numpy(Sh), w.D)
    dP = P.cuda()
    Oo = G.Out(w.Batch * w.L * w.D)
    bm.batchMatMul(s, 1, dP.data_ptr(), dV.data_ptr(), Oo.ptr, w.Batch, w.L, w.D, w.L, w.L)
    assert_accurate(O, Oo.host((w.Batch, w.L, w.D)), O.f64.batchMatMul(P.numpy(), w.V.numpy()), "P V")
    G.check_status(pkg)


# ------------------------------------------------------------------ convolution
CONV_CASES = [
    # N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw
    (4, 9, 9, 8, 12, 3, 3, 1, 1, 1, 1),
    (4, 28, 28, 64, 64, 3, 3, 1, 1, 1, 1),
    (8, 14, 14, 32, 256, 3, 3, 1, 1, 1, 1),
    (4, 16, 16, 36, 40, 3, 3, 2, 2, 1, 1),
    (4, 11, 10, 4, 8, 5, 3, 2, 2, 2, 1),
    (4, 32, 32, 16, 32, 7, 7, 2, 2, 3, 3),
    (4, 12, 12, 128, 132, 1, 1, 1, 1, 0, 0),
    (4, 10, 10, 8, 16, 3, 3, 1, 1, 0, 0),
    (4, 8, 8, 256, 64, 2, 2, 2, 2, 0, 0),
]


@pytest.mark.parametrize("case", CONV_CASES)
def test_conv_gemmr(pkg, O, cuda, case):
    N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw = case
    rng = np.random.default_rng(17)
    X = rng.standard_normal((N, IH, IW, IC)).astype(np.float32)
    W = (rng.standard_normal((OC, FH, FW, IC)) * np.sqrt(2.0 / (FH * FW * IC))).astype(np.float32)
    OH, OW = (IH + 2 * ph - FH) // sh + 1, (IW + 2 * pw - FW) // sw + 1
    Y64 = O.f64.conv3D(X, W, OH, OW, sh, sw, ph, pw)
    Y = G.conv(pkg, "conv3D_GemmR", X, W, sh, sw, ph, pw)
    assert_accurate(O, Y, Y64, f"conv {case}")
    if N * OH * OW * OC * FH * FW * IC <= 60e6:
        Yref = O.ref_loops.conv3D_img2col(X, W, OH, OW, sh, sw, ph, pw)
        assert O.frob_rel(Y, Yref) <= 2e-6


# Feature-map and filter geometries the reference's own convolution test lists
# (test/cuda/conv3D/Cuda_conv3D_test.java:157-171, :183-189), at a batch the FP64 oracle finishes in a second or two;
# inputs as in that test: uniform [0, 1) (Vector.random_float_vector).
REF_TEST_CONV = [
    # N, IH, IW, IC, OC, FH, FW, ph, pw
    (1, 64, 64, 64, 64, 7, 7, 3, 3),
    (1, 64, 64, 64, 64, 9, 9, 4, 4),
    (1, 32, 32, 64, 64, 8, 8, 4, 4),
    (2, 32, 32, 64, 64, 1, 7, 0, 3),
    (2, 16, 16, 256, 256, 5, 5, 2, 2),
    (2, 16, 16, 128, 128, 3, 3, 1, 1),
    (4, 8, 8, 128, 256, 3, 3, 1, 1),
    (4, 8, 8, 256, 256, 5, 5, 2, 2),
    (1, 128, 128, 4, 64, 3, 3, 1, 1),        # the 3-channel input of that list, padded to 4 channels by the engine
    (2, 4, 4, 1024, 1024, 3, 3, 1, 1),
]


@pytest.mark.gpu
@pytest.mark.parametrize("case", REF_TEST_CONV)
def test_conv_geometries_of_the_reference_test(pkg, O, cuda, case):
    N, IH, IW, IC, OC, FH, FW, ph, pw = case
    rng = np.random.default_rng(IH * 131 + FH)
    X = rng.random((N, IH, IW, IC), dtype=np.float32)
    W = rng.random((OC, FH, FW, IC), dtype=np.float32)
    if IC == 4:
        X[..., 3] = 0.0
        W[..., 3] = 0.0
    OH, OW = IH + 2 * ph - FH + 1, IW + 2 * pw - FW + 1
    Y64 = O.f64.conv3D(X, W, OH, OW, 1, 1, ph, pw)
    Y = G.conv(pkg, "conv3D_GemmR", X, W, 1, 1, ph, pw)
    assert_accurate(O, Y, Y64, f"conv {case}")
    # the reference test's own gate: its CPU loop's result within 1e-3 relative for >= 99 % of the elements
    # (Cuda_conv3D/test.cuh:38-57, :913) - checked here against FP64, which that loop approximates
    rel = np.abs(Y - Y64) / np.maximum(np.abs(Y64), 1e-30)
    assert np.mean(rel <= 1e-3) >= 0.99


def test_conv_entry_point_aliases(pkg, O, cuda):
    rng = np.random.default_rng(18)
    X = rng.standard_normal((4, 12, 12, 16)).astype(np.float32)
    W = rng.standard_normal((24, 3, 3, 16)).astype(np.float32) * 0.1
    Y64 = O.f64.conv3D(X, W, 12, 12, 1, 1, 1, 1)
    base = G.conv(pkg, "conv3D_GemmR", X, W, 1, 1, 1, 1)
    assert_accurate(O, base, Y64, "GemmR")
    for entry in ("conv3D_GemmR_texture", "conv3D_GemmR_SGM", "conv3D_GemmR_texture_SGM", "conv3D", "conv3D_texture"):
        assert np.array_equal(G.conv(pkg, entry, X, W, 1, 1, 1, 1), base), entry
    Ynp = G.conv(pkg, "conv3D_np", X, W, 1, 1, 0, 0)
    assert_accurate(O, Ynp, O.f64.conv3D(X, W, 10, 10, 1, 1, 0, 0), "conv3D_np")
    W1 = rng.standard_normal((20, 1, 1, 16)).astype(np.float32)
    Y1 = O.f64.conv3D(X, W1, 12, 12, 1, 1, 0, 0)
    for entry in ("conv3D_W1", "conv3D_GemmR_W1", "conv3D_GemmR_W1_SGM"):
        assert_accurate(O, G.conv(pkg, entry, X, W1, 1, 1, 0, 0), Y1, entry)


V2_AND_WINOGRAD_ENTRIES = ("conv3DV2", "conv3D_GemmV2R", "conv3D_Im2col_Winograd_s8_R_texture",
                           "conv3D_Im2col_WinogradR_s8_texture_SGM", "conv3D_Im2col_Winograd_s16_R_texture",
                           "conv3D_Im2col_WinogradR_s16_texture_SGM")


@pytest.mark.parametrize("case", [
    # N, IH, IW, IC, OC, FH, FW, ph, pw  - stride-1 shapes the Java engine sends to the Im2col-Winograd natives:
    # IC % 8 == 0, N*OH >= 32, FW + OW > 8 (s8: 2 <= FW <= 9) or > 16 (s16: 7 <= FW <= 9)
    (4, 12, 12, 16, 64, 3, 3, 1, 1),
    (2, 16, 20, 8, 72, 5, 5, 2, 2),
    (2, 18, 18, 8, 32, 7, 7, 3, 3),
    (2, 16, 16, 8, 32, 9, 9, 4, 4),
    (4, 10, 14, 24, 64, 2, 4, 0, 1),
])
def test_v2_and_winograd_entry_points(pkg, O, cuda, case):
    """The reference's other forward-conv natives are the same convolution (they differ from GemmR only
    in rounding), so here they must return GemmR's bits and meet the same FP64 tolerance."""
    N, IH, IW, IC, OC, FH, FW, ph, pw = case
    rng = np.random.default_rng(23)
    X = rng.standard_normal((N, IH, IW, IC)).astype(np.float32)
    W = (rng.standard_normal((OC, FH, FW, IC)) * np.sqrt(2.0 / (FH * FW * IC))).astype(np.float32)
    OH, OW = IH + 2 * ph - FH + 1, IW + 2 * pw - FW + 1
    base = G.conv(pkg, "conv3D_GemmR", X, W, 1, 1, ph, pw)
    assert_accurate(O, base, O.f64.conv3D(X, W, OH, OW, 1, 1, ph, pw), f"GemmR {case}")
    for entry in V2_AND_WINOGRAD_ENTRIES:
        assert np.array_equal(G.conv(pkg, entry, X, W, 1, 1, ph, pw), base), entry


def test_v2_entry_points_strided(pkg, O, cuda):
    rng = np.random.default_rng(24)
    X = rng.standard_normal((4, 17, 15, 12)).astype(np.float32)
    W = rng.standard_normal((40, 3, 3, 12)).astype(np.float32) * 0.1
    base = G.conv(pkg, "conv3D_GemmR", X, W, 2, 2, 1, 1)
    assert_accurate(O, base, O.f64.conv3D(X, W, 9, 8, 2, 2, 1, 1), "GemmR s2")
    for entry in ("conv3DV2", "conv3D_GemmV2R"):
        assert np.array_equal(G.conv(pkg, entry, X, W, 2, 2, 1, 1), base), entry


def test_kernel_remode_bit_exact(pkg, O, cuda):
    rng = np.random.default_rng(19)
    for (OC, FH, FW, IC) in [(4, 1, 1, 4), (12, 3, 3, 8), (256, 3, 3, 64), (36, 5, 3, 20), (33, 2, 2, 7)]:
        W = rng.standard_normal((OC, FH, FW, IC)).astype(np.float32)
        dW = G.dev(W)
        out = G.Out(W.size)
        pkg.cu32.Cuda_conv3D.kernel_remode(G.stream(), dW.data_ptr(), out.ptr, FH, FW, OC, IC)
        assert np.array_equal(out.host((FH, FW, IC, OC)), O.ref_loops.kernel_remode(W))


def test_config4_reduced(pkg, O, cuda):
    """Config 4 geometry (28x28, 256 -> 256, 3x3 s1 p1) on 8 images."""
    w = pkg.workloads.config4(N=8)
    X, W = w.X.numpy(), w.W.numpy()
    Y = G.conv(pkg, "conv3D_GemmR", X, W, 1, 1, 1, 1)
    assert_accurate(O, Y, O.f64.conv3D(X, W, 28, 28, 1, 1, 1, 1), "config 4 (8 images)")


# ------------------------------------------------------------------ full-size properties
def test_config2_full_size_sampled_rows_and_checksum(pkg, O, cuda):
    """8192^3 is too large for a full CPU oracle run inside a test; check (1) 48 sampled rows of
    C against the FP64 oracle, and (2) the checksum identity C*1 = A*(B*1) over the whole output."""
    size = 8192
    for form in ("AB", "T1", "T2"):
        w = pkg.workloads.config2(form, size)
        dA, dB = w.A.cuda(), w.B.cuda()
        dC = torch.empty((size, size), device="cuda")
        fn = {"AB": pkg.cu32.Cuda_matMul.matMul, "T1": pkg.cu32.Cuda_matMul.matMulT1,
              "T2": pkg.cu32.Cuda_matMul.matMulT2}[form]
        fn([G.stream()], 1, dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), size, size, size)
        G.check_status(pkg)
        rows = np.linspace(0, size - 1, 48).astype(int)
        A, B = w.A.numpy(), w.B.numpy()
        Arows = A[:, rows].T if form == "T1" else A[rows]
        Bm = B.T if form == "T2" else B
        C64 = Arows.astype(np.float64) @ Bm.astype(np.float64)
        C = dC[torch.as_tensor(rows, device="cuda")].cpu().numpy()
        assert_accurate(O, C, C64, f"config 2 {form} sampled rows")
        rowsum = dC.double().sum(1).cpu().numpy()
        A64 = (A.T if form == "T1" else A).astype(np.float64)
        want = A64 @ Bm.astype(np.float64).sum(1)
        assert np.linalg.norm(rowsum - want) / np.linalg.norm(want) <= 1e-6, form
        del dA, dB, dC
