"""Host-side logic that needs no GPU: the mirrored Java heuristics, the C-ABI surface, and
argument validation (which happens before any CUDA call)."""
import ctypes
import re
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def java_blockNum(N, M):
    """Literal transcription of the loop structure in Cuda_matMul.java:18-38 for comparison."""
    def one(x):
        b = 0
        while True:
            if x > 127: b += x >> 7
            x &= 127
            if x == 0: break
            if x > 63: b += 1
            x &= 63
            if x == 0: break
            if x > 31: b += 1
            x &= 31
            if x == 0: break
            if x > 15: b += 1
            x &= 15
            if x == 0: break
            if x > 7: b += 1
            x &= 7
            if x == 0: break
            if x > 3: b += 1
            break
        return b
    return one(N) * one(M)


def test_blockNum_matches_java_loop(pkg):
    mm = pkg.cu32.Cuda_matMul
    for N in list(range(4, 600, 4)) + [1024, 8192, 4100]:
        for M in (4, 60, 128, 132, 252, 4100):
            assert mm.blockNum(N, M) == java_blockNum(N, M), (N, M)
    assert mm.blockNum(512, 512) == 16
    assert mm.blockNum(8192, 8192) == 4096


def test_nstream(pkg):
    mm = pkg.cu32.Cuda_matMul
    assert mm.nstream(1024, 1024) == 1          # powers of two: one rectangle
    assert mm.nstream(8192, 4100) == 2          # 4100 = 32*128 + 4
    assert mm.nstream(252, 252) == 10           # capped at 10
    assert mm.nstream(132, 128) == 2


def test_splitk_decisions(pkg):
    e = pkg.engine
    # big outputs never split
    assert e.matMul_gridZ(8192, 8192, 8192, 148) == 1
    assert e.matMul_gridZ(1024, 1024, 1024, 148) == 1
    # K below the threshold never splits
    assert e.matMul_gridZ(128, 128, 508, 148) == 1
    # the long-K weight-gradient shape is split into the maximum number of parts
    assert e.matMulT1_gridZ(512, 512, 1048576, 148) == 16
    assert e.matMulT1_gridZ(512, 512, 131072, 148) == 16
    # small output, moderate K: limited by K >> 8
    assert e.matMul_gridZ(128, 128, 1024, 148) in (2, 4)
    gz = e.matMulT2_gridZ(256, 256, 4096, 148)
    assert gz == 1 or (2 <= gz <= 16 and (gz == 2 or gz % 4 == 0))
    for N, M, K in [(64, 64, 2048), (256, 128, 8192), (512, 2048, 8192), (4, 4, 512)]:
        for f in (e.matMul_gridZ, e.matMulT1_gridZ, e.matMulT2_gridZ):
            g = f(N, M, K, 148)
            assert g == 1 or (2 <= g <= 16)


def test_pad4_and_conv_dims(pkg):
    e = pkg.engine
    assert [e.pad4(x) for x in (1, 4, 5, 4097, 8191)] == [4, 4, 8, 4100, 8192]
    assert e.conv_out_dim(28, 3, 1, 1) == 28
    assert e.conv_out_dim(32, 3, 2, 1) == 16
    assert e.conv_out_dim(224, 7, 2, 3) == 112


def test_gm_slice(pkg):
    cv = pkg.cu32.Cuda_conv3D
    assert cv.GEMM_GM_slice(256, 200704, 2304) == -1
    assert cv.GEMM_GM_slice(256, 128 * 65536 + 128, 2304) == 32768 << 7
    assert cv.GEMM_GM_slice(64, 64 * 65536 + 64, 2304) == 32768 << 6


def test_shard_ranges(pkg):
    s = pkg.shard
    for total, world, mult in [(1024, 8, 1), (8192, 8, 4), (8191, 4, 4), (10, 4, 4), (1048576, 8, 32), (7, 8, 1)]:
        spans = [s.split_range(total, world, r, mult) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == total
        for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
            assert a1 == b0 and a0 <= a1
        for a0, a1 in spans[:-1]:
            assert a0 % mult == 0 and (a1 % mult == 0 or a1 == total)
    assert s.shard_k(1048576, 8, 3) == (3 * 131072, 4 * 131072)
    with pytest.raises(ValueError):
        s.split_range(10, 2, 2)


def _header_symbols():
    text = (ROOT / "include" / "dragon_cu32.h").read_text()
    return sorted(set(re.findall(r"CU32_API\s+[\w\s\*]+?\b(cu32_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol(pkg):
    lib = pkg.cu32.load()
    names = _header_symbols()
    assert len(names) >= 83
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/dragon_cu32.h but not exported"
    # the ctypes table covers the same surface
    assert set(pkg.cu32.SIGNATURES) | {"cu32_version"} == set(names)
    assert pkg.cu32.version().startswith("dragon_cu32")


def test_jni_symbols_exported(pkg):
    out = subprocess.run(["nm", "-D", "--defined-only", str(pkg.cu32.LIB_PATH)], capture_output=True, text=True).stdout
    syms = set(re.findall(r"\bJava_z_dragon_engine_cuda_impl_math_Cuda_1(\w+)", out))
    want_matmul = {"matMul_matMul", "matMul_matMulT1", "matMul_matMulT2", "matMul_matMulSK", "matMul_matMulT1SK",
                   "matMul_matMulT2SK", "matMul_SKbuf_1summary", "matMul_matMul_1mma", "matMul_matMulT1_1mma",
                   "matMul_matMulT2_1mma"}
    want_bmm = {"batchMatMul_batchMatMul", "batchMatMul_batchMatMul_1texture", "batchMatMul_batchMatMulT1",
                "batchMatMul_batchMatMulT2", "batchMatMul_batchMatMulT2_1texture", "batchMatMul_batchMatMul_1mma",
                "batchMatMul_batchMatMulT1_1mma", "batchMatMul_batchMatMulT2_1mma"}
    want_conv = {"conv3D_kernel_1remode", "conv3D_conv3D", "conv3D_conv3D_1texture", "conv3D_conv3D_1np",
                 "conv3D_conv3D_1W1", "conv3D_conv3D_1GemmR", "conv3D_conv3D_1GemmR_1texture",
                 "conv3D_conv3D_1GemmR_1SGM", "conv3D_conv3D_1GemmR_1texture_1SGM", "conv3D_conv3D_1GemmR_1W1",
                 "conv3D_conv3D_1GemmR_1W1_1SGM", "conv3D_conv3DV2", "conv3D_conv3D_1GemmV2R",
                 "conv3D_conv3D_1Im2col_1Winograd_1s8_1R_1texture", "conv3D_conv3D_1Im2col_1WinogradR_1s8_1texture_1SGM",
                 "conv3D_conv3D_1Im2col_1Winograd_1s16_1R_1texture",
                 "conv3D_conv3D_1Im2col_1WinogradR_1s16_1texture_1SGM"}
    want_fused = {"matMul_matMul_1biased", "matMul_matMul_1mma_1biased", "matMul_SKbuf_1summary_1biased",
                  "conv3D_conv3D_1GemmR_1biased", "batchMatMul_batchMatMul_1scaled", "batchMatMul_batchMatMulT1_1scaled",
                  "batchMatMul_batchMatMulT2_1scaled", "dconv3D_1deltaX_dconv3D_1deltaX_1s1_1biased",
                  "dconv3D_1deltaX_dconv3D_1deltaX_1ksImsR_1biased"}   # no counterpart in the reference's Java classes
    want_dx = {"dconv3D_1deltaX_dconv3D_1deltaX_1s1", "dconv3D_1deltaX_dconv3D_1deltaX_1s1_1SGM",
               "dconv3D_1deltaX_dconv3D_1deltaX_1s1_1texture", "dconv3D_1deltaX_dconv3D_1deltaX_1s1_1texture_1SGM",
               "dconv3D_1deltaX_dconv3D_1deltaX_1W1", "dconv3D_1deltaX_dconv3D_1deltaX_1W1_1SGM",
               "dconv3D_1deltaX_dconv3D_1deltaX_1V2_1s1", "dconv3D_1deltaX_Im2col_1Winograd_1s8_1texture",
               "dconv3D_1deltaX_Im2col_1Winograd_1s8_1texture_1SGM", "dconv3D_1deltaX_Im2col_1Winograd_1s16_1texture",
               "dconv3D_1deltaX_Im2col_1Winograd_1s16_1texture_1SGM"}
    want_dx |= {"dconv3D_1deltaX_" + n for n in (
        "ks_1remode", "ks_1remodev2", "dconv3D_1deltaX_1kernelSplit", "dconv3D_1deltaX_1kernelSplit_1SGM",
        "dconv3D_1deltaX_1ksImsR", "dconv3D_1deltaX_1ksImsR_1SGM", "dconv3D_1deltaX_1ksImsR_1texture",
        "dconv3D_1deltaX_1ksImsR_1texture_1SGM", "dconv3D_1deltaX_1ksIms2R", "dconv3D_1deltaX_1ksIms2R_1SGM",
        "dconv3D_1deltaX_1ksIms2R_1texture", "dconv3D_1deltaX_1ksIms2R_1texture_1SGM", "dconv3D_1deltaX_1ksV2_1Ims2R",
        "dconv3D_1deltaX_1crossAdd", "dconv3D_1deltaX_1crossAdd_1SGM")}   # all 26 natives of the Java class
    assert len(want_dx) == 26
    want_dw = {"dconv3D_1deltaW_" + n for n in (
        "dconv3D_1deltaW", "dconv3D_1deltaW_1W1", "buf_1summary", "dconv3D_1deltaW_1GemmSK", "dconv3D_1deltaW_1GemmV2SK",
        "dconv3D_1deltaW_1GemmSK_1W1", "Im2col_1WinogradV2_1SHW_1s4_1texture", "Im2col_1WinogradV2_1SHW_1s8_1texture",
        "Im2col_1WinogradV2_1SHW_1s16_1texture")}   # all 9 natives of the Java class
    want_dx |= want_dw
    missing = (want_matmul | want_bmm | want_conv | want_fused | want_dx) - syms
    assert not missing, missing


def test_argument_errors_without_gpu(pkg):
    """Validation runs before any CUDA call, so it is testable here."""
    lib = pkg.cu32.load()
    fp = ctypes.POINTER(ctypes.c_float)
    null = ctypes.cast(None, fp)
    fake = ctypes.cast(ctypes.c_void_p(0x10000), fp)      # never dereferenced on these paths
    odd = ctypes.cast(ctypes.c_void_p(0x10004), fp)
    s = (ctypes.c_int64 * 10)()
    assert lib.cu32_matMul(None, 1, fake, fake, fake, 4, 4, 4) == -3
    assert lib.cu32_matMul(s, 0, fake, fake, fake, 4, 4, 4) == -3
    assert lib.cu32_matMul(s, 11, fake, fake, fake, 4, 4, 4) == -3
    assert lib.cu32_matMul(s, 1, null, fake, fake, 4, 4, 4) == -1
    assert lib.cu32_matMul(s, 1, fake, fake, fake, 0, 4, 4) == -2
    assert lib.cu32_matMul(s, 1, fake, fake, fake, 4, 4, -8) == -2
    assert lib.cu32_matMul(s, 1, odd, fake, fake, 4, 4, 4) == -4
    assert lib.cu32_matMul(s, 1, fake, fake, fake, 4, 6, 4) == -4      # pitch M=6 not a multiple of 4
    assert lib.cu32_matMulSK(s, 1, 0, fake, fake, fake, fake, 4, 4, 512) == -8
    assert lib.cu32_matMulSK(s, 1, 4, fake, fake, fake, null, 4, 4, 512) == -1
    assert lib.cu32_SKbuf_summary(0, fake, fake, 3, 6) == -4
    assert lib.cu32_SKbuf_summary(0, fake, null, 3, 8) == -1
    assert lib.cu32_SKbuf_summary(0, fake, fake, -1, 8) == -2
    assert lib.cu32_batchMatMul(s, 1, fake, fake, fake, 2, 8, 8, 8, 4) == -2  # AK < BK
    assert lib.cu32_batchMatMulT2(s, 1, fake, fake, fake, 2, 8, 4, 8, 8) == -2  # CM < BM
    assert lib.cu32_kernel_remode(0, null, fake, 3, 3, 8, 8) == -1
    assert lib.cu32_conv3D_GemmR(s, 1, fake, 8, 8, fake, fake, 3, 3, fake, 8, 8, 4, 6, 8, 1, 1, 1, 1) == -4  # IC % 4
    assert lib.cu32_conv3D_GemmR(s, 1, fake, 8, 8, fake, fake, 3, 3, fake, 8, 8, 4, 8, 8, 0, 1, 1, 1) == -2  # stride 0
    assert lib.cu32_conv3D_GemmR_SGM(s, 1, fake, 8, 8, fake, fake, 3, 3, fake, 8, 8, 4, 8, 8, 1, 1, 1, 1, 0) == -8
    # output extents that do not follow from the geometry (8x8, 3x3, pad 1, stride 1 gives 8x8, not 7x8)
    assert lib.cu32_conv3D_GemmR(s, 1, fake, 8, 8, fake, fake, 3, 3, fake, 7, 8, 4, 8, 8, 1, 1, 1, 1) == -2
    assert lib.cu32_conv3D(s, 1, fake, 8, 8, fake, 3, 3, fake, 8, 8, 4, 8, 8, 2, 2, 1, 1) == -2
    # the allocation-free split-K refuses everything its two launches would refuse before the first one
    assert lib.cu32_matMulT1SK_noalloc(s, 1, 4, fake, fake, odd, 8, 8, 512) == -4
    assert lib.cu32_matMulT1SK_noalloc(s, 1, 4, null, fake, fake, 8, 8, 512) == -1
    assert lib.cu32_matMulT1SK_noalloc(s, 1, 4, fake, fake, fake, 8, 6, 512) == -4
    assert lib.cu32_matMulT1SK_noalloc(s, 1, 100, fake, fake, fake, 512, 512, 512) == -9
    assert lib.cu32_selftest_wait_giveup(0, 0) == -8
    assert lib.cu32_tune(b"ring_raw", 9) == -8 and lib.cu32_tune(b"store_bufs", 3) == -8
    assert lib.cu32_tune(b"nonsense", 1) == -8
    assert lib.cu32_tune(b"tile", 6) == -8
    assert lib.cu32_tune(b"kc", 0) == -8
    v = ctypes.c_int(-5)
    assert lib.cu32_get_tune(b"kc", ctypes.byref(v)) == 0 and v.value >= 1
    with pytest.raises(pkg.cu32.CudaException) as ei:
        pkg.cu32.Cuda_matMul.matMul([0], 1, 0, 0x10000, 0x10000, 4, 4, 4)
    assert ei.value.code == -1


def test_missing_library_fails_loudly(pkg, tmp_path, monkeypatch):
    monkeypatch.setattr(pkg.cu32, "_lib", None)
    monkeypatch.setattr(pkg.cu32, "LIB_PATH", tmp_path / "libdragon_cu32.so")
    with pytest.raises(FileNotFoundError):
        pkg.cu32.load()


def test_status_decoding(pkg):
    assert pkg.cu32.decode_status(0) == "ok"
    assert "drainer" in pkg.cu32.decode_status((5 << 24) | (1 << 16) | 7)


def test_conv3D_deltaW_gridZ_rule(pkg):
    """The Java engine's split decision for the weight gradient, on hand-computed cases."""
    gz = pkg.engine.conv3D_deltaW_gridZ
    # config 4: b2 = blockNum(256, 2304) = 2*18 = 36 < 148*1.5; (3136 + 3136) / 72 = 87, capped by 148*4/36 = 16
    assert gz(28, 28, 28, 28, 3, 3, 256, 256, 256, 148) == 16
    # fewer than 512 output pixels: never split
    assert gz(7, 7, 7, 7, 3, 3, 4, 512, 512, 148) == 1
    # the output alone fills the SMs: blockNum(1024, 9*1024) = 8*72 = 576 >= 148 * 1.5 * GK/(GK+1024)
    assert gz(14, 14, 14, 14, 3, 3, 64, 1024, 1024, 148) == 1
    # small layer, 784 pixels: b2 = blockNum(64, 288) = 1*3; b0 = blockNum(64, 784) = 7, b1 = blockNum(32, 784) = 7;
    # 14 / 6 = 2, below the caps 784 >> 8 = 3 and 148*4/3; rounded up to a multiple of 4
    assert gz(14, 14, 14, 14, 3, 3, 4, 32, 64, 148) == 4
