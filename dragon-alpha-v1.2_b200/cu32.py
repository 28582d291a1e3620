"""ctypes binding of libdragon_cu32.so.

The three classes mirror the Java classes of the reference that declare the natives
(``z/dragon/engine/cuda/impl/math/Cuda_matMul.java``, ``Cuda_batchMatMul.java``,
``Cuda_conv3D.java``): same static-method names, same argument order, device memory and
streams passed as integers exactly as the Java side passes ``long`` addresses.  A non-zero
return code raises :class:`CudaException`, the analogue of
``z.dragon.engine.cuda.impl.CudaException``.

There is no fallback: if the shared library is missing, loading fails with an error that
says how to build it.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_int64, POINTER
from pathlib import Path

_HERE = Path(__file__).resolve().parent
LIB_PATH = _HERE / "libdragon_cu32.so"

ERROR_NAMES = {
    -1: "CU32_E_NULL", -2: "CU32_E_DIM", -3: "CU32_E_STREAMS", -4: "CU32_E_ALIGN",
    -5: "CU32_E_GEOMETRY", -6: "CU32_E_DRIVER", -7: "CU32_E_TENSORMAP", -8: "CU32_E_ARG",
    -9: "CU32_E_SCRATCH",
}

TILE_NAMES = {0: "128x64", 1: "128x128", 2: "128x256", 3: "256x128 pair", 4: "256x256 pair",
              5: "256x192 pair, A via TMEM", 6: "128x64, A via TMEM", 7: "128x128, A via TMEM",
              8: "256x64 pair"}


class CudaException(RuntimeError):
    """Raised for a non-zero return code (positive: cudaError_t, negative: CU32_E_*)."""

    def __init__(self, code: int, where: str = ""):
        self.code = code
        name = ERROR_NAMES.get(code, f"cudaError {code}" if code > 0 else f"error {code}")
        super().__init__(f"{where}: {name}" if where else name)


_lib = None
_fp = POINTER(c_float)
_sp = POINTER(c_int64)


def _sig(lib, name, argtypes):
    fn = getattr(lib, name)
    fn.argtypes = argtypes
    fn.restype = c_int
    return fn


# name -> ctypes argument types; also the list of symbols include/dragon_cu32.h declares.
_I = c_int
SIGNATURES = {
    "cu32_matMul": [_sp, _I, _fp, _fp, _fp, _I, _I, _I],
    "cu32_matMulT1": [_sp, _I, _fp, _fp, _fp, _I, _I, _I],
    "cu32_matMulT2": [_sp, _I, _fp, _fp, _fp, _I, _I, _I],
    "cu32_matMulSK": [_sp, _I, _I, _fp, _fp, _fp, _fp, _I, _I, _I],
    "cu32_matMulT1SK": [_sp, _I, _I, _fp, _fp, _fp, _fp, _I, _I, _I],
    "cu32_matMulT2SK": [_sp, _I, _I, _fp, _fp, _fp, _fp, _I, _I, _I],
    "cu32_SKbuf_summary": [c_int64, _fp, _fp, _I, _I],
    "cu32_matMul_replicated": [_sp, _I, _fp, _fp, _fp, POINTER(_fp), _I, _I, _I, _I],
    "cu32_matMulT2_replicated": [_sp, _I, _fp, _fp, _fp, POINTER(_fp), _I, _I, _I, _I],
    "cu32_matMulT1SK_noalloc": [_sp, _I, _I, _fp, _fp, _fp, _I, _I, _I],
    "cu32_matMul_mma": [_sp, _I, _fp, _fp, _fp, _I, _I, _I],
    "cu32_matMulT1_mma": [_sp, _I, _fp, _fp, _fp, _I, _I, _I],
    "cu32_matMulT2_mma": [_sp, _I, _fp, _fp, _fp, _I, _I, _I],
    "cu32_batchMatMul": [_sp, _I, _fp, _fp, _fp, _I, _I, _I, _I, _I],
    "cu32_batchMatMul_texture": [_sp, _I, _fp, _fp, _fp, _I, _I, _I, _I, _I],
    "cu32_batchMatMulT1": [_sp, _I, _fp, _fp, _fp, _I, _I, _I, _I, _I],
    "cu32_batchMatMulT2": [_sp, _I, _fp, _fp, _fp, _I, _I, _I, _I, _I],
    "cu32_batchMatMulT2_texture": [_sp, _I, _fp, _fp, _fp, _I, _I, _I, _I, _I],
    "cu32_batchMatMul_mma": [_I, _sp, _I, _fp, _fp, _fp, _I, _I, _I, _I, _I],
    "cu32_batchMatMulT1_mma": [_sp, _I, _fp, _fp, _fp, _I, _I, _I, _I, _I],
    "cu32_batchMatMulT2_mma": [_I, _sp, _I, _fp, _fp, _fp, _I, _I, _I, _I, _I],
    "cu32_kernel_remode": [c_int64, _fp, _fp, _I, _I, _I, _I],
    "cu32_conv3D_GemmR": [_sp, _I, _fp, _I, _I, _fp, _fp, _I, _I, _fp] + [_I] * 9,
    "cu32_conv3D_GemmR_texture": [_sp, _I, _fp, _I, _I, _fp, _fp, _I, _I, _fp] + [_I] * 9,
    "cu32_conv3D_GemmR_SGM": [_sp, _I, _fp, _I, _I, _fp, _fp, _I, _I, _fp] + [_I] * 10,
    "cu32_conv3D_GemmR_texture_SGM": [_sp, _I, _fp, _I, _I, _fp, _fp, _I, _I, _fp] + [_I] * 10,
    "cu32_conv3D_GemmR_W1": [_sp, _I, _fp, _I, _I, _fp, _fp, _fp, _I, _I, _I],
    "cu32_conv3D_GemmR_W1_SGM": [_sp, _I, _fp, _I, _I, _fp, _fp, _fp, _I, _I, _I, _I],
    "cu32_dconv3D_deltaX_s1": [_sp, _I, _fp, _I, _I, _fp, _I, _I, _fp] + [_I] * 7,
    "cu32_dconv3D_deltaX_s1_texture": [_sp, _I, _fp, _I, _I, _fp, _I, _I, _fp] + [_I] * 7,
    "cu32_dconv3D_deltaX_s1_SGM": [_sp, _I, _fp, _I, _I, _fp, _I, _I, _fp] + [_I] * 8,
    "cu32_dconv3D_deltaX_s1_texture_SGM": [_sp, _I, _fp, _I, _I, _fp, _I, _I, _fp] + [_I] * 8,
    "cu32_dconv3D_deltaX_V2_s1": [_I, _sp, _I, _fp, _I, _I, _fp, _I, _I, _fp] + [_I] * 7,
    "cu32_dconv3D_deltaX_W1": [_sp, _I, _fp, _fp, _fp] + [_I] * 5,
    "cu32_dconv3D_deltaX_W1_SGM": [_sp, _I, _fp, _fp, _fp] + [_I] * 6,
    "cu32_dconv3D_deltaX_Im2col_Winograd_s8_texture": [_I, _sp, _I, _fp, _I, _I, _fp, _I, _I, _fp] + [_I] * 7,
    "cu32_dconv3D_deltaX_Im2col_Winograd_s8_texture_SGM": [_I, _sp, _I, _fp, _I, _I, _fp, _I, _I, _fp] + [_I] * 8,
    "cu32_dconv3D_deltaX_Im2col_Winograd_s16_texture": [_I, _sp, _I, _fp, _I, _I, _fp, _I, _I, _fp] + [_I] * 7,
    "cu32_dconv3D_deltaX_Im2col_Winograd_s16_texture_SGM": [_I, _sp, _I, _fp, _I, _I, _fp, _I, _I, _fp] + [_I] * 8,
    "cu32_ks_remode": [c_int64, _fp, _I, _I, _fp] + [_I] * 6,
    "cu32_ks_remodev2": [c_int64, _fp, _I, _I, _fp] + [_I] * 6,
    "cu32_dconv3D_deltaX_kernelSplit": [_sp, _I, _fp, _I, _I, _fp, _I, _I, _fp] + [_I] * 9,
    "cu32_dconv3D_deltaX_kernelSplit_SGM": [_sp, _I, _fp, _I, _I, _fp, _I, _I, _fp] + [_I] * 10,
    "cu32_dconv3D_deltaX_ksImsR": [_sp, _I, _fp, _I, _I, _fp, _I, _I, _fp] + [_I] * 9,
    "cu32_dconv3D_deltaX_ksImsR_SGM": [_sp, _I, _fp, _I, _I, _fp, _I, _I, _fp] + [_I] * 10,
    "cu32_dconv3D_deltaX_ksImsR_texture": [_sp, _I, _fp, _I, _I, _fp, _I, _I, _fp] + [_I] * 9,
    "cu32_dconv3D_deltaX_ksImsR_texture_SGM": [_sp, _I, _fp, _I, _I, _fp, _I, _I, _fp] + [_I] * 10,
    "cu32_dconv3D_deltaX_ksIms2R": [_sp, _I, _fp, _I, _I, _fp, _I, _I, _fp] + [_I] * 7,
    "cu32_dconv3D_deltaX_ksIms2R_SGM": [_sp, _I, _fp, _I, _I, _fp, _I, _I, _fp] + [_I] * 8,
    "cu32_dconv3D_deltaX_ksIms2R_texture": [_sp, _I, _fp, _I, _I, _fp, _I, _I, _fp] + [_I] * 7,
    "cu32_dconv3D_deltaX_ksIms2R_texture_SGM": [_sp, _I, _fp, _I, _I, _fp, _I, _I, _fp] + [_I] * 8,
    "cu32_dconv3D_deltaX_ksV2_Ims2R": [_I, _sp, _I, _fp, _I, _I, _fp, _I, _I, _fp] + [_I] * 7,
    "cu32_dconv3D_deltaX_crossAdd": [_sp, _I, _fp, _I, _I, _fp, _I, _I, _fp] + [_I] * 9,
    "cu32_dconv3D_deltaX_crossAdd_SGM": [_sp, _I, _fp, _I, _I, _fp, _I, _I, _fp] + [_I] * 10,
    "cu32_dconv3D_deltaW": [_sp, _I, _fp, _I, _I, _fp, _I, _I, _fp] + [_I] * 9,
    "cu32_dconv3D_deltaW_W1": [_sp, _I, _fp, _I, _I, _fp, _fp, _I, _I, _I],
    "cu32_dconv3D_deltaW_buf_summary": [c_int64, _fp, _fp, _I, _I],
    "cu32_dconv3D_deltaW_GemmSK": [_sp, _I, _I, _fp, _I, _I, _fp, _I, _I, _fp, _fp] + [_I] * 9,
    "cu32_dconv3D_deltaW_GemmV2SK": [_sp, _I, _I, _fp, _I, _I, _fp, _I, _I, _fp, _fp] + [_I] * 9,
    "cu32_dconv3D_deltaW_GemmSK_W1": [_sp, _I, _I, _fp, _I, _I, _fp, _fp, _fp, _I, _I, _I],
    "cu32_dconv3D_deltaW_Im2col_WinogradV2_SHW_s4_texture": [_sp, _I, _I, _I, _I, _fp, _I, _I, _fp, _I, _I, _fp, _fp] + [_I] * 8,
    "cu32_dconv3D_deltaW_Im2col_WinogradV2_SHW_s8_texture": [_sp, _I, _I, _I, _I, _fp, _I, _I, _fp, _I, _I, _fp, _fp] + [_I] * 8,
    "cu32_dconv3D_deltaW_Im2col_WinogradV2_SHW_s16_texture": [_sp, _I, _I, _I, _I, _I, _fp, _I, _I, _fp, _I, _I, _fp, _fp] + [_I] * 8,
    "cu32_batchMatMul_scaled": [_sp, _I, _fp, _fp, _fp, _I, _I, _I, _I, _I, ctypes.c_float],
    "cu32_batchMatMulT1_scaled": [_sp, _I, _fp, _fp, _fp, _I, _I, _I, _I, _I, ctypes.c_float],
    "cu32_batchMatMulT2_scaled": [_sp, _I, _fp, _fp, _fp, _I, _I, _I, _I, _I, ctypes.c_float],
    "cu32_batchMatMulT2_softmax": [_sp, _I, _fp, _fp, _fp, _I, _I, _I, _I, _I, ctypes.c_float],
    "cu32_dconv3D_deltaX_s1_biased": [_sp, _I, _fp, _I, _I, _fp, _I, _I, _fp] + [_I] * 7 + [_fp, _I],
    "cu32_dconv3D_deltaX_ksImsR_biased": [_sp, _I, _fp, _I, _I, _fp, _I, _I, _fp] + [_I] * 9 + [_fp, _I],
    "cu32_matMul_biased": [_sp, _I, _fp, _fp, _fp, _fp, _I, _I, _I, _I],
    "cu32_matMul_mma_biased": [_sp, _I, _fp, _fp, _fp, _fp, _I, _I, _I, _I],
    "cu32_SKbuf_summary_biased": [c_int64, _fp, _fp, _fp, _I, _I, _I, _I],
    "cu32_conv3D_GemmR_biased": [_sp, _I, _fp, _I, _I, _fp, _fp, _I, _I, _fp] + [_I] * 9 + [_fp, _I],
    "cu32_conv3DV2": [_I, _sp, _I, _fp, _I, _I, _fp, _I, _I, _fp] + [_I] * 9,
    "cu32_conv3D_GemmV2R": [_I, _sp, _I, _fp, _I, _I, _fp, _fp, _I, _I, _fp] + [_I] * 9,
    "cu32_conv3D_Im2col_Winograd_s8_R_texture": [_I, _sp, _I, _fp, _I, _I, _fp, _fp, _I, _I, _fp] + [_I] * 7,
    "cu32_conv3D_Im2col_WinogradR_s8_texture_SGM": [_I, _sp, _I, _fp, _I, _I, _fp, _fp, _I, _I, _fp] + [_I] * 8,
    "cu32_conv3D_Im2col_Winograd_s16_R_texture": [_I, _sp, _I, _fp, _I, _I, _fp, _fp, _I, _I, _fp] + [_I] * 7,
    "cu32_conv3D_Im2col_WinogradR_s16_texture_SGM": [_I, _sp, _I, _fp, _I, _I, _fp, _fp, _I, _I, _fp] + [_I] * 8,
    "cu32_conv3D": [_sp, _I, _fp, _I, _I, _fp, _I, _I, _fp] + [_I] * 9,
    "cu32_conv3D_texture": [_sp, _I, _fp, _I, _I, _fp, _I, _I, _fp] + [_I] * 9,
    "cu32_conv3D_np": [_sp, _I, _fp, _I, _I, _fp, _I, _I, _fp] + [_I] * 7,
    "cu32_conv3D_W1": [_sp, _I, _fp, _I, _I, _fp, _fp, _I, _I, _I],
    "cu32_tune": [c_char_p, _I],
    "cu32_get_tune": [c_char_p, POINTER(c_int)],
    "cu32_read_status": [POINTER(c_int)],
    "cu32_selftest_wait_giveup": [c_int64, ctypes.c_longlong],
    "cu32_read_clock": [POINTER(ctypes.c_ulonglong)],
}


def load():
    """Load libdragon_cu32.so (once) and declare every entry point's signature."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise FileNotFoundError(
            f"{LIB_PATH} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
            "(needs nvcc); there is no CPU or PyTorch fallback for this library")
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, args in SIGNATURES.items():
        _sig(lib, name, args)
    lib.cu32_version.argtypes = []
    lib.cu32_version.restype = c_char_p
    _lib = lib
    return lib


def _p(addr):
    return ctypes.cast(ctypes.c_void_p(int(addr)), _fp)


def _streams(streamArray, length):
    arr = (c_int64 * 10)(*([int(s) for s in streamArray[:10]] + [0] * (10 - min(len(streamArray), 10))))
    return arr, int(length)


def _check(rc, where):
    if rc != 0:
        raise CudaException(rc, where)


def tune(key: str, value: int) -> None:
    _check(load().cu32_tune(key.encode(), int(value)), f"cu32_tune({key})")


def get_tune(key: str) -> int:
    v = c_int(0)
    _check(load().cu32_get_tune(key.encode(), ctypes.byref(v)), f"cu32_get_tune({key})")
    return v.value


def read_status() -> int:
    """Device give-up word (0 = every bounded wait completed).  Synchronises the device."""
    v = c_int(0)
    _check(load().cu32_read_status(ctypes.byref(v)), "cu32_read_status")
    return v.value


def decode_status(word: int) -> str:
    if word == 0:
        return "ok"
    roles = {1: "tma-producer", 2: "splitter", 3: "mma(operands)", 4: "mma(tmem-buffer)", 5: "drainer",
             7: "self-test"}
    return f"{roles.get(word >> 24, word >> 24)} gave up at stage/buffer {(word >> 16) & 0xFF}, iteration {word & 0xFFFF}"


def read_clock():
    """(SM cycles, nanoseconds, launches) accumulated by the contraction kernels since the last read, while the
    "clock" tuning key is on; cycles / nanoseconds is the SM clock in GHz the kernels ran at."""
    v = (ctypes.c_ulonglong * 3)()
    _check(load().cu32_read_clock(v), "cu32_read_clock")
    return int(v[0]), int(v[1]), int(v[2])


def selftest_wait_giveup(stream: int, limit_cycles: int) -> None:
    """Launch the one-warp kernel whose bounded wait runs out after `limit_cycles` (see the header)."""
    _check(load().cu32_selftest_wait_giveup(int(stream), int(limit_cycles)), "cu32_selftest_wait_giveup")


def version() -> str:
    return load().cu32_version().decode()


class Cuda_matMul:
    """Mirror of z.dragon.engine.cuda.impl.math.Cuda_matMul (natives + host helpers)."""

    @staticmethod
    def blockNum(N: int, M: int) -> int:
        """Number of 128/64/.../4-wide blocks the reference's tiling cuts [N, M] into
        (Cuda_matMul.java:18-38); input to the split-K decision."""
        def count(x):
            b = 0
            if x > 127:
                b += x >> 7
            x &= 127
            for w in (64, 32, 16, 8, 4):
                if x == 0:
                    break
                if x >= w:
                    b += 1
                x &= w - 1
            return b
        return count(N) * count(M)

    @staticmethod
    def nstream(N: int, M: int) -> int:
        """Streams the Java engine requests for an [N, M] output (Cuda_matMul.java:41-65)."""
        def count(x):
            if x & (x - 1) == 0:
                return 1
            s = 0
            for w in (128, 64, 32, 16, 8, 4):
                if x == 0:
                    break
                if x >= w:
                    s += 1
                x &= w - 1
            return s
        size = count(N) * count(M)
        return size if size < 10 else 10

    @staticmethod
    def matMul(streamArray, length, dA, dB, dC, N, M, K):
        s, n = _streams(streamArray, length)
        _check(load().cu32_matMul(s, n, _p(dA), _p(dB), _p(dC), N, M, K), "matMul")

    @staticmethod
    def matMulT1(streamArray, length, dA, dB, dC, N, M, K):
        s, n = _streams(streamArray, length)
        _check(load().cu32_matMulT1(s, n, _p(dA), _p(dB), _p(dC), N, M, K), "matMulT1")

    @staticmethod
    def matMulT2(streamArray, length, dA, dB, dC, N, M, K):
        s, n = _streams(streamArray, length)
        _check(load().cu32_matMulT2(s, n, _p(dA), _p(dB), _p(dC), N, M, K), "matMulT2")

    @staticmethod
    def matMul_mma(streamArray, length, dA, dB, dC, N, M, K):
        s, n = _streams(streamArray, length)
        _check(load().cu32_matMul_mma(s, n, _p(dA), _p(dB), _p(dC), N, M, K), "matMul_mma")

    @staticmethod
    def matMulT1_mma(streamArray, length, dA, dB, dC, N, M, K):
        s, n = _streams(streamArray, length)
        _check(load().cu32_matMulT1_mma(s, n, _p(dA), _p(dB), _p(dC), N, M, K), "matMulT1_mma")

    @staticmethod
    def matMulT2_mma(streamArray, length, dA, dB, dC, N, M, K):
        s, n = _streams(streamArray, length)
        _check(load().cu32_matMulT2_mma(s, n, _p(dA), _p(dB), _p(dC), N, M, K), "matMulT2_mma")

    @staticmethod
    def matMulSK(streamArray, length, GridZ, dA, dB, dC, dCbuf, N, M, K):
        s, n = _streams(streamArray, length)
        _check(load().cu32_matMulSK(s, n, GridZ, _p(dA), _p(dB), _p(dC), _p(dCbuf), N, M, K), "matMulSK")

    @staticmethod
    def matMulT1SK(streamArray, length, GridZ, dA, dB, dC, dCbuf, N, M, K):
        s, n = _streams(streamArray, length)
        _check(load().cu32_matMulT1SK(s, n, GridZ, _p(dA), _p(dB), _p(dC), _p(dCbuf), N, M, K), "matMulT1SK")

    @staticmethod
    def matMulT2SK(streamArray, length, GridZ, dA, dB, dC, dCbuf, N, M, K):
        s, n = _streams(streamArray, length)
        _check(load().cu32_matMulT2SK(s, n, GridZ, _p(dA), _p(dB), _p(dC), _p(dCbuf), N, M, K), "matMulT2SK")

    @staticmethod
    def SKbuf_summary(stream, dCbuf, dC, part, sizeC):
        _check(load().cu32_SKbuf_summary(int(stream), _p(dCbuf), _p(dC), part, sizeC), "SKbuf_summary")

    # ---- contraction + bias row in one pass: what the engine's matMul_biased does with two kernels
    # (CudaFloat32EngineBase.java:1594-1688); these natives do not exist in the reference
    @staticmethod
    def matMul_biased(streamArray, length, dA, dB, dC, dBias, N, M, K, width):
        s, n = _streams(streamArray, length)
        _check(load().cu32_matMul_biased(s, n, _p(dA), _p(dB), _p(dC), _p(dBias), N, M, K, width), "matMul_biased")

    # the product stored to several buffers at once (no counterpart in the reference): `replicas` are device
    # addresses of further [N, M] outputs, typically this rank's rows inside the peers' copies of a gathered output
    @staticmethod
    def _replicated(name, streamArray, length, dA, dB, dC, replicas, N, M, K):
        s, n = _streams(streamArray, length)
        arr = (_fp * max(len(replicas), 1))(*[_p(r) for r in replicas])
        _check(getattr(load(), "cu32_" + name)(s, n, _p(dA), _p(dB), _p(dC), arr, len(replicas), N, M, K), name)

    @staticmethod
    def matMul_replicated(streamArray, length, dA, dB, dC, replicas, N, M, K):
        Cuda_matMul._replicated("matMul_replicated", streamArray, length, dA, dB, dC, replicas, N, M, K)

    @staticmethod
    def matMulT2_replicated(streamArray, length, dA, dB, dC, replicas, N, M, K):
        Cuda_matMul._replicated("matMulT2_replicated", streamArray, length, dA, dB, dC, replicas, N, M, K)

    @staticmethod
    def matMul_mma_biased(streamArray, length, dA, dB, dC, dBias, N, M, K, width):
        s, n = _streams(streamArray, length)
        _check(load().cu32_matMul_mma_biased(s, n, _p(dA), _p(dB), _p(dC), _p(dBias), N, M, K, width),
               "matMul_mma_biased")

    @staticmethod
    def SKbuf_summary_biased(stream, dCbuf, dC, dBias, part, sizeC, M, width):
        _check(load().cu32_SKbuf_summary_biased(int(stream), _p(dCbuf), _p(dC), _p(dBias), part, sizeC, M, width),
               "SKbuf_summary_biased")


class Cuda_batchMatMul:
    """Mirror of z.dragon.engine.cuda.impl.math.Cuda_batchMatMul."""

    @staticmethod
    def batchMatMul(streamArray, length, dA, dB, dC, Batch, N, M, BK, AK):
        s, n = _streams(streamArray, length)
        _check(load().cu32_batchMatMul(s, n, _p(dA), _p(dB), _p(dC), Batch, N, M, BK, AK), "batchMatMul")

    @staticmethod
    def batchMatMul_texture(streamArray, length, dA, dB, dC, Batch, N, M, BK, AK):
        s, n = _streams(streamArray, length)
        _check(load().cu32_batchMatMul_texture(s, n, _p(dA), _p(dB), _p(dC), Batch, N, M, BK, AK),
               "batchMatMul_texture")

    @staticmethod
    def batchMatMul_mma(useTexture, streamArray, length, dA, dB, dC, Batch, N, M, BK, AK):
        s, n = _streams(streamArray, length)
        _check(load().cu32_batchMatMul_mma(int(bool(useTexture)), s, n, _p(dA), _p(dB), _p(dC), Batch, N, M, BK, AK),
               "batchMatMul_mma")

    @staticmethod
    def batchMatMulT1(streamArray, length, dA, dB, dC, Batch, CN, AN, M, K):
        s, n = _streams(streamArray, length)
        _check(load().cu32_batchMatMulT1(s, n, _p(dA), _p(dB), _p(dC), Batch, CN, AN, M, K), "batchMatMulT1")

    @staticmethod
    def batchMatMulT1_mma(streamArray, length, dA, dB, dC, Batch, CN, AN, M, K):
        s, n = _streams(streamArray, length)
        _check(load().cu32_batchMatMulT1_mma(s, n, _p(dA), _p(dB), _p(dC), Batch, CN, AN, M, K), "batchMatMulT1_mma")

    @staticmethod
    def batchMatMulT2(streamArray, length, dA, dB, dC, Batch, N, CM, BM, K):
        s, n = _streams(streamArray, length)
        _check(load().cu32_batchMatMulT2(s, n, _p(dA), _p(dB), _p(dC), Batch, N, CM, BM, K), "batchMatMulT2")

    @staticmethod
    def batchMatMulT2_texture(streamArray, length, dA, dB, dC, Batch, N, CM, BM, K):
        s, n = _streams(streamArray, length)
        _check(load().cu32_batchMatMulT2_texture(s, n, _p(dA), _p(dB), _p(dC), Batch, N, CM, BM, K),
               "batchMatMulT2_texture")

    @staticmethod
    def batchMatMulT2_mma(useTexture, streamArray, length, dA, dB, dC, Batch, N, CM, BM, K):
        s, n = _streams(streamArray, length)
        _check(load().cu32_batchMatMulT2_mma(int(bool(useTexture)), s, n, _p(dA), _p(dB), _p(dC), Batch, N, CM, BM, K),
               "batchMatMulT2_mma")

    # scale fused into the store (no counterpart in the Java class): arguments of the unscaled native, then alpha
    @staticmethod
    def _scaled(name, streamArray, length, dA, dB, dC, Batch, d0, d1, d2, d3, alpha):
        s, n = _streams(streamArray, length)
        _check(getattr(load(), "cu32_" + name)(s, n, _p(dA), _p(dB), _p(dC), Batch, d0, d1, d2, d3, float(alpha)), name)

    @staticmethod
    def batchMatMul_scaled(streamArray, length, dA, dB, dC, Batch, N, M, BK, AK, alpha):
        Cuda_batchMatMul._scaled("batchMatMul_scaled", streamArray, length, dA, dB, dC, Batch, N, M, BK, AK, alpha)

    @staticmethod
    def batchMatMulT1_scaled(streamArray, length, dA, dB, dC, Batch, CN, AN, M, K, alpha):
        Cuda_batchMatMul._scaled("batchMatMulT1_scaled", streamArray, length, dA, dB, dC, Batch, CN, AN, M, K, alpha)

    @staticmethod
    def batchMatMulT2_scaled(streamArray, length, dA, dB, dC, Batch, N, CM, BM, K, alpha):
        Cuda_batchMatMul._scaled("batchMatMulT2_scaled", streamArray, length, dA, dB, dC, Batch, N, CM, BM, K, alpha)

    @staticmethod
    def batchMatMulT2_softmax(streamArray, length, dA, dB, dP, Batch, N, CM, BM, K, alpha):
        """P = softmax over rows of alpha * A * B^T in one pass (scores never stored unnormalised)."""
        Cuda_batchMatMul._scaled("batchMatMulT2_softmax", streamArray, length, dA, dB, dP, Batch, N, CM, BM, K, alpha)


class Cuda_conv3D:
    """Mirror of the GEMM / GEMMR natives of z.dragon.engine.cuda.impl.math.Cuda_conv3D."""

    @staticmethod
    def kernel_remode(stream, dW, dCW, FH, FW, OC, IC):
        _check(load().cu32_kernel_remode(int(stream), _p(dW), _p(dCW), FH, FW, OC, IC), "kernel_remode")

    @staticmethod
    def conv3D_GemmR(streamArray, length, dX, IH, IW, dW, dCW, FH, FW, dY, OH, OW, N, IC, OC, sh, sw, ph, pw):
        s, n = _streams(streamArray, length)
        _check(load().cu32_conv3D_GemmR(s, n, _p(dX), IH, IW, _p(dW), _p(dCW), FH, FW, _p(dY), OH, OW, N, IC, OC,
                                        sh, sw, ph, pw), "conv3D_GemmR")

    @staticmethod
    def conv3D_GemmR_texture(streamArray, length, dX, IH, IW, dW, dCW, FH, FW, dY, OH, OW, N, IC, OC, sh, sw, ph, pw):
        s, n = _streams(streamArray, length)
        _check(load().cu32_conv3D_GemmR_texture(s, n, _p(dX), IH, IW, _p(dW), _p(dCW), FH, FW, _p(dY), OH, OW, N, IC,
                                                OC, sh, sw, ph, pw), "conv3D_GemmR_texture")

    @staticmethod
    def conv3D_GemmR_SGM(streamArray, length, dX, IH, IW, dW, dCW, FH, FW, dY, OH, OW, N, IC, OC, sh, sw, ph, pw,
                         GM_slice):
        s, n = _streams(streamArray, length)
        _check(load().cu32_conv3D_GemmR_SGM(s, n, _p(dX), IH, IW, _p(dW), _p(dCW), FH, FW, _p(dY), OH, OW, N, IC, OC,
                                            sh, sw, ph, pw, GM_slice), "conv3D_GemmR_SGM")

    @staticmethod
    def conv3D_GemmR_texture_SGM(streamArray, length, dX, IH, IW, dW, dCW, FH, FW, dY, OH, OW, N, IC, OC, sh, sw, ph,
                                 pw, GM_slice):
        s, n = _streams(streamArray, length)
        _check(load().cu32_conv3D_GemmR_texture_SGM(s, n, _p(dX), IH, IW, _p(dW), _p(dCW), FH, FW, _p(dY), OH, OW, N,
                                                    IC, OC, sh, sw, ph, pw, GM_slice), "conv3D_GemmR_texture_SGM")

    @staticmethod
    def conv3D_GemmR_W1(streamArray, length, dX, IH, IW, dW, dCW, dY, N, IC, OC):
        s, n = _streams(streamArray, length)
        _check(load().cu32_conv3D_GemmR_W1(s, n, _p(dX), IH, IW, _p(dW), _p(dCW), _p(dY), N, IC, OC), "conv3D_GemmR_W1")

    @staticmethod
    def conv3D_GemmR_W1_SGM(streamArray, length, dX, IH, IW, dW, dCW, dY, N, IC, OC, GM_slice):
        s, n = _streams(streamArray, length)
        _check(load().cu32_conv3D_GemmR_W1_SGM(s, n, _p(dX), IH, IW, _p(dW), _p(dCW), _p(dY), N, IC, OC, GM_slice),
               "conv3D_GemmR_W1_SGM")

    @staticmethod
    def conv3D(streamArray, length, dX, IH, IW, dW, FH, FW, dY, OH, OW, N, IC, OC, sh, sw, ph, pw):
        s, n = _streams(streamArray, length)
        _check(load().cu32_conv3D(s, n, _p(dX), IH, IW, _p(dW), FH, FW, _p(dY), OH, OW, N, IC, OC, sh, sw, ph, pw),
               "conv3D")

    @staticmethod
    def conv3D_texture(streamArray, length, dX, IH, IW, dW, FH, FW, dY, OH, OW, N, IC, OC, sh, sw, ph, pw):
        s, n = _streams(streamArray, length)
        _check(load().cu32_conv3D_texture(s, n, _p(dX), IH, IW, _p(dW), FH, FW, _p(dY), OH, OW, N, IC, OC, sh, sw, ph,
                                          pw), "conv3D_texture")

    @staticmethod
    def conv3D_np(streamArray, length, dX, IH, IW, dW, FH, FW, dY, OH, OW, N, IC, OC, sh, sw):
        s, n = _streams(streamArray, length)
        _check(load().cu32_conv3D_np(s, n, _p(dX), IH, IW, _p(dW), FH, FW, _p(dY), OH, OW, N, IC, OC, sh, sw),
               "conv3D_np")

    @staticmethod
    def conv3D_W1(streamArray, length, dX, IH, IW, dW, dY, N, IC, OC):
        s, n = _streams(streamArray, length)
        _check(load().cu32_conv3D_W1(s, n, _p(dX), IH, IW, _p(dW), _p(dY), N, IC, OC), "conv3D_W1")

    @staticmethod
    def conv3D_GemmR_biased(streamArray, length, dX, IH, IW, dW, dCW, FH, FW, dY, OH, OW, N, IC, OC, sh, sw, ph, pw,
                            dBias, width):
        """conv3D_GemmR plus the bias row of conv3D_biased (CudaFloat32EngineBase.java:2389-2542) in one
        pass; not a native of the reference."""
        s, n = _streams(streamArray, length)
        _check(load().cu32_conv3D_GemmR_biased(s, n, _p(dX), IH, IW, _p(dW), _p(dCW), FH, FW, _p(dY), OH, OW, N, IC,
                                               OC, sh, sw, ph, pw, _p(dBias), width), "conv3D_GemmR_biased")

    # ---- the V2 / Im2col-Winograd natives (Cuda_conv3D.java; Cuda_conv3D/A.cu:89-111, :390-637): same
    # contraction under the names the Java engine prefers with its default flags
    @staticmethod
    def conv3DV2(useTexture, streamArray, length, dX, IH, IW, dW, FH, FW, dY, OH, OW, N, IC, OC, sh, sw, ph, pw):
        s, n = _streams(streamArray, length)
        _check(load().cu32_conv3DV2(int(bool(useTexture)), s, n, _p(dX), IH, IW, _p(dW), FH, FW, _p(dY), OH, OW, N,
                                    IC, OC, sh, sw, ph, pw), "conv3DV2")

    @staticmethod
    def conv3D_GemmV2R(useTexture, streamArray, length, dX, IH, IW, dW, dCW, FH, FW, dY, OH, OW, N, IC, OC, sh, sw,
                       ph, pw):
        s, n = _streams(streamArray, length)
        _check(load().cu32_conv3D_GemmV2R(int(bool(useTexture)), s, n, _p(dX), IH, IW, _p(dW), _p(dCW), FH, FW,
                                          _p(dY), OH, OW, N, IC, OC, sh, sw, ph, pw), "conv3D_GemmV2R")

    @staticmethod
    def _winograd(name, useTexture, streamArray, length, dX, IH, IW, dW, dCW, FH, FW, dY, OH, OW, N, IC, OC, ph, pw,
                  *gm_slice) -> bool:
        s, n = _streams(streamArray, length)
        _check(getattr(load(), "cu32_" + name)(int(bool(useTexture)), s, n, _p(dX), IH, IW, _p(dW), _p(dCW), FH, FW,
                                               _p(dY), OH, OW, N, IC, OC, ph, pw, *gm_slice), name)
        return True   # the Java native returns "handled"; every shape is

    @staticmethod
    def conv3D_Im2col_Winograd_s8_R_texture(useTexture, streamArray, length, dX, IH, IW, dW, dCW, FH, FW, dY, OH,
                                            OW, N, IC, OC, ph, pw) -> bool:
        return Cuda_conv3D._winograd("conv3D_Im2col_Winograd_s8_R_texture", useTexture, streamArray, length, dX, IH,
                                     IW, dW, dCW, FH, FW, dY, OH, OW, N, IC, OC, ph, pw)

    @staticmethod
    def conv3D_Im2col_WinogradR_s8_texture_SGM(useTexture, streamArray, length, dX, IH, IW, dW, dCW, FH, FW, dY, OH,
                                               OW, N, IC, OC, ph, pw, GM_slice) -> bool:
        return Cuda_conv3D._winograd("conv3D_Im2col_WinogradR_s8_texture_SGM", useTexture, streamArray, length, dX,
                                     IH, IW, dW, dCW, FH, FW, dY, OH, OW, N, IC, OC, ph, pw, GM_slice)

    @staticmethod
    def conv3D_Im2col_Winograd_s16_R_texture(useTexture, streamArray, length, dX, IH, IW, dW, dCW, FH, FW, dY, OH,
                                             OW, N, IC, OC, ph, pw) -> bool:
        return Cuda_conv3D._winograd("conv3D_Im2col_Winograd_s16_R_texture", useTexture, streamArray, length, dX, IH,
                                     IW, dW, dCW, FH, FW, dY, OH, OW, N, IC, OC, ph, pw)

    @staticmethod
    def conv3D_Im2col_WinogradR_s16_texture_SGM(useTexture, streamArray, length, dX, IH, IW, dW, dCW, FH, FW, dY, OH,
                                                OW, N, IC, OC, ph, pw, GM_slice) -> bool:
        return Cuda_conv3D._winograd("conv3D_Im2col_WinogradR_s16_texture_SGM", useTexture, streamArray, length, dX,
                                     IH, IW, dW, dCW, FH, FW, dY, OH, OW, N, IC, OC, ph, pw, GM_slice)

    max_grid = 65535
    grid_slice = 32768

    @staticmethod
    def GEMM_GM_slice(GN: int, GM: int, GK: int) -> int:
        """Slice of GM the Java side passes to the _SGM natives when the reference's grid
        would exceed 65535 blocks along GM (Cuda_conv3D.java:346-356); -1 = no slicing.
        This library accepts the slice and ignores it (the result does not depend on it)."""
        max_GM = (Cuda_conv3D.max_grid + 1) << 6
        if GM < max_GM:
            return -1
        flag = GN > 127 and (GK & 7) == 0
        bm = GM >> 7 if flag else GM >> 6
        if bm <= Cuda_conv3D.max_grid:
            return -1
        return Cuda_conv3D.grid_slice << (7 if flag else 6)


def _dx_native(name):
    """A strided data-gradient native of Cuda_dconv3D_deltaX: every one takes the same leading arguments, followed by
    its own tail of geometry integers, and forwards them unchanged."""
    def f(streamArray, length, d_deltaY, OH, OW, dF, FH, FW, d_deltaX, IH, IW, N, IC, OC, *tail):
        s, n = _streams(streamArray, length)
        _check(getattr(load(), "cu32_dconv3D_deltaX_" + name)(s, n, _p(d_deltaY), OH, OW, _p(dF), FH, FW, _p(d_deltaX),
                                                              IH, IW, N, IC, OC, *tail), name)
    f.__name__ = "dconv3D_deltaX_" + name
    return staticmethod(f)


class Cuda_dconv3D_deltaX:
    """Mirror of the stride-1 natives of z.dragon.engine.cuda.impl.math.Cuda_dconv3D_deltaX (the data gradient
    of the forward convolution; reference: Cuda_dconv3D_deltaX/A.cu:21-277, :837-1040) and, further down, of the
    natives for strides > 1 (ks_remode*, kernelSplit, ksIms*, crossAdd; A.cu:280-834)."""

    @staticmethod
    def _s1(name, lead, streamArray, length, d_deltaY, OH, OW, dW, FH, FW, d_deltaX, IH, IW, N, IC, OC, ph, pw, *tail):
        s, n = _streams(streamArray, length)
        _check(getattr(load(), "cu32_" + name)(*lead, s, n, _p(d_deltaY), OH, OW, _p(dW), FH, FW, _p(d_deltaX), IH, IW,
                                               N, IC, OC, ph, pw, *tail), name)

    @staticmethod
    def dconv3D_deltaX_s1(streamArray, length, d_deltaY, OH, OW, dW, FH, FW, d_deltaX, IH, IW, N, IC, OC, ph, pw):
        Cuda_dconv3D_deltaX._s1("dconv3D_deltaX_s1", (), streamArray, length, d_deltaY, OH, OW, dW, FH, FW, d_deltaX, IH,
                                IW, N, IC, OC, ph, pw)

    @staticmethod
    def dconv3D_deltaX_s1_texture(streamArray, length, d_deltaY, OH, OW, dW, FH, FW, d_deltaX, IH, IW, N, IC, OC, ph,
                                  pw):
        Cuda_dconv3D_deltaX._s1("dconv3D_deltaX_s1_texture", (), streamArray, length, d_deltaY, OH, OW, dW, FH, FW,
                                d_deltaX, IH, IW, N, IC, OC, ph, pw)

    @staticmethod
    def dconv3D_deltaX_s1_SGM(streamArray, length, d_deltaY, OH, OW, dW, FH, FW, d_deltaX, IH, IW, N, IC, OC, ph, pw,
                              GM_slice):
        Cuda_dconv3D_deltaX._s1("dconv3D_deltaX_s1_SGM", (), streamArray, length, d_deltaY, OH, OW, dW, FH, FW, d_deltaX,
                                IH, IW, N, IC, OC, ph, pw, GM_slice)

    @staticmethod
    def dconv3D_deltaX_s1_texture_SGM(streamArray, length, d_deltaY, OH, OW, dW, FH, FW, d_deltaX, IH, IW, N, IC, OC,
                                      ph, pw, GM_slice):
        Cuda_dconv3D_deltaX._s1("dconv3D_deltaX_s1_texture_SGM", (), streamArray, length, d_deltaY, OH, OW, dW, FH, FW,
                                d_deltaX, IH, IW, N, IC, OC, ph, pw, GM_slice)

    @staticmethod
    def dconv3D_deltaX_V2_s1(useTexture, streamArray, length, d_deltaY, OH, OW, dW, FH, FW, d_deltaX, IH, IW, N, IC,
                             OC, ph, pw):
        Cuda_dconv3D_deltaX._s1("dconv3D_deltaX_V2_s1", (int(bool(useTexture)),), streamArray, length, d_deltaY, OH, OW,
                                dW, FH, FW, d_deltaX, IH, IW, N, IC, OC, ph, pw)

    @staticmethod
    def dconv3D_deltaX_W1(streamArray, length, d_deltaY, dW, d_deltaX, IH, IW, N, IC, OC):
        s, n = _streams(streamArray, length)
        _check(load().cu32_dconv3D_deltaX_W1(s, n, _p(d_deltaY), _p(dW), _p(d_deltaX), IH, IW, N, IC, OC),
               "dconv3D_deltaX_W1")

    @staticmethod
    def dconv3D_deltaX_W1_SGM(streamArray, length, d_deltaY, dW, d_deltaX, IH, IW, N, IC, OC, GM_slice):
        s, n = _streams(streamArray, length)
        _check(load().cu32_dconv3D_deltaX_W1_SGM(s, n, _p(d_deltaY), _p(dW), _p(d_deltaX), IH, IW, N, IC, OC, GM_slice),
               "dconv3D_deltaX_W1_SGM")

    @staticmethod
    def Im2col_Winograd_s8_texture(useTexture, streamArray, length, d_deltaY, OH, OW, dW, FH, FW, d_deltaX, IH, IW, N,
                                   IC, OC, ph, pw) -> bool:
        Cuda_dconv3D_deltaX._s1("dconv3D_deltaX_Im2col_Winograd_s8_texture", (int(bool(useTexture)),), streamArray,
                                length, d_deltaY, OH, OW, dW, FH, FW, d_deltaX, IH, IW, N, IC, OC, ph, pw)
        return True

    @staticmethod
    def Im2col_Winograd_s8_texture_SGM(useTexture, streamArray, length, d_deltaY, OH, OW, dW, FH, FW, d_deltaX, IH, IW,
                                       N, IC, OC, ph, pw, GM_slice) -> bool:
        Cuda_dconv3D_deltaX._s1("dconv3D_deltaX_Im2col_Winograd_s8_texture_SGM", (int(bool(useTexture)),), streamArray,
                                length, d_deltaY, OH, OW, dW, FH, FW, d_deltaX, IH, IW, N, IC, OC, ph, pw, GM_slice)
        return True

    @staticmethod
    def Im2col_Winograd_s16_texture(useTexture, streamArray, length, d_deltaY, OH, OW, dW, FH, FW, d_deltaX, IH, IW, N,
                                    IC, OC, ph, pw) -> bool:
        Cuda_dconv3D_deltaX._s1("dconv3D_deltaX_Im2col_Winograd_s16_texture", (int(bool(useTexture)),), streamArray,
                                length, d_deltaY, OH, OW, dW, FH, FW, d_deltaX, IH, IW, N, IC, OC, ph, pw)
        return True

    @staticmethod
    def Im2col_Winograd_s16_texture_SGM(useTexture, streamArray, length, d_deltaY, OH, OW, dW, FH, FW, d_deltaX, IH,
                                        IW, N, IC, OC, ph, pw, GM_slice) -> bool:
        Cuda_dconv3D_deltaX._s1("dconv3D_deltaX_Im2col_Winograd_s16_texture_SGM", (int(bool(useTexture)),), streamArray,
                                length, d_deltaY, OH, OW, dW, FH, FW, d_deltaX, IH, IW, N, IC, OC, ph, pw, GM_slice)
        return True

    # ---- strides > 1: the kernel-split natives take the ks_remodev2 workspace, crossAdd the filter itself
    @staticmethod
    def ks_remode(stream, dW, FH, FW, dCW, CFH, CFW, OC, IC, sh, sw):
        _check(load().cu32_ks_remode(int(stream), _p(dW), FH, FW, _p(dCW), CFH, CFW, OC, IC, sh, sw), "ks_remode")

    @staticmethod
    def ks_remodev2(stream, dW, FH, FW, dCW, CFH, CFW, OC, IC, sh, sw):
        _check(load().cu32_ks_remodev2(int(stream), _p(dW), FH, FW, _p(dCW), CFH, CFW, OC, IC, sh, sw), "ks_remodev2")

    @staticmethod
    def _ks(name, lead, streamArray, length, d_deltaY, OH, OW, dF, FH, FW, d_deltaX, IH, IW, N, IC, OC, *tail):
        s, n = _streams(streamArray, length)
        _check(getattr(load(), "cu32_dconv3D_deltaX_" + name)(*lead, s, n, _p(d_deltaY), OH, OW, _p(dF), FH, FW,
                                                              _p(d_deltaX), IH, IW, N, IC, OC, *tail), name)


    @staticmethod
    def dconv3D_deltaX_ksV2_Ims2R(useTexture, streamArray, length, d_deltaY, OH, OW, dCW, FH, FW, d_deltaX, IH, IW, N, IC,
                                  OC, ph, pw):
        Cuda_dconv3D_deltaX._ks("ksV2_Ims2R", (int(bool(useTexture)),), streamArray, length, d_deltaY, OH, OW, dCW, FH, FW,
                                d_deltaX, IH, IW, N, IC, OC, ph, pw)

    # (…, sh, sw, ph, pw[, GM_slice]) for any stride; (…, ph, pw[, GM_slice]) for the stride-2 "Ims2" natives
    dconv3D_deltaX_kernelSplit = _dx_native("kernelSplit")
    dconv3D_deltaX_kernelSplit_SGM = _dx_native("kernelSplit_SGM")
    dconv3D_deltaX_ksImsR = _dx_native("ksImsR")
    dconv3D_deltaX_ksImsR_SGM = _dx_native("ksImsR_SGM")
    dconv3D_deltaX_ksImsR_texture = _dx_native("ksImsR_texture")
    dconv3D_deltaX_ksImsR_texture_SGM = _dx_native("ksImsR_texture_SGM")
    dconv3D_deltaX_ksIms2R = _dx_native("ksIms2R")
    dconv3D_deltaX_ksIms2R_SGM = _dx_native("ksIms2R_SGM")
    dconv3D_deltaX_ksIms2R_texture = _dx_native("ksIms2R_texture")
    dconv3D_deltaX_ksIms2R_texture_SGM = _dx_native("ksIms2R_texture_SGM")
    dconv3D_deltaX_crossAdd = _dx_native("crossAdd")
    dconv3D_deltaX_crossAdd_SGM = _dx_native("crossAdd_SGM")

    # bias row fused (no counterpart in the Java class): (…unbiased arguments…, dBias, width)
    @staticmethod
    def dconv3D_deltaX_s1_biased(streamArray, length, d_deltaY, OH, OW, dW, FH, FW, d_deltaX, IH, IW, N, IC, OC, ph, pw,
                                 dBias, width):
        s, n = _streams(streamArray, length)
        _check(load().cu32_dconv3D_deltaX_s1_biased(s, n, _p(d_deltaY), OH, OW, _p(dW), FH, FW, _p(d_deltaX), IH, IW, N, IC,
                                                    OC, ph, pw, _p(dBias), width), "dconv3D_deltaX_s1_biased")

    @staticmethod
    def dconv3D_deltaX_ksImsR_biased(streamArray, length, d_deltaY, OH, OW, dCW, FH, FW, d_deltaX, IH, IW, N, IC, OC, sh, sw,
                                     ph, pw, dBias, width):
        s, n = _streams(streamArray, length)
        _check(load().cu32_dconv3D_deltaX_ksImsR_biased(s, n, _p(d_deltaY), OH, OW, _p(dCW), FH, FW, _p(d_deltaX), IH, IW, N,
                                                        IC, OC, sh, sw, ph, pw, _p(dBias), width), "dconv3D_deltaX_ksImsR_biased")


class Cuda_dconv3D_deltaW:
    """Mirror of z.dragon.engine.cuda.impl.math.Cuda_dconv3D_deltaW (Cuda_dconv3D_deltaW.java:288-640): the weight
    gradient of the convolution, deltaW[OC, FH, FW, IC] from X[N, IH, IW, IC] and deltaY[N, OH, OW, OC]."""

    @staticmethod
    def dconv3D_deltaW(streamArray, length, dX, IH, IW, d_deltaY, OH, OW, d_deltaW, FH, FW, N, IC, OC, sh, sw, ph, pw):
        s, n = _streams(streamArray, length)
        _check(load().cu32_dconv3D_deltaW(s, n, _p(dX), IH, IW, _p(d_deltaY), OH, OW, _p(d_deltaW), FH, FW, N, IC, OC,
                                          sh, sw, ph, pw), "dconv3D_deltaW")

    @staticmethod
    def dconv3D_deltaW_W1(streamArray, length, dX, IH, IW, d_deltaY, d_deltaW, N, IC, OC):
        s, n = _streams(streamArray, length)
        _check(load().cu32_dconv3D_deltaW_W1(s, n, _p(dX), IH, IW, _p(d_deltaY), _p(d_deltaW), N, IC, OC), "dconv3D_deltaW_W1")

    @staticmethod
    def buf_summary(stream, d_deltaW_buf, d_deltaW, part, sizeW):
        _check(load().cu32_dconv3D_deltaW_buf_summary(int(stream), _p(d_deltaW_buf), _p(d_deltaW), part, sizeW), "buf_summary")

    @staticmethod
    def _sk(name, streamArray, length, GridZ, dX, IH, IW, d_deltaY, OH, OW, d_deltaW, d_buf, FH, FW, N, IC, OC, sh, sw, ph, pw):
        s, n = _streams(streamArray, length)
        _check(getattr(load(), "cu32_dconv3D_deltaW_" + name)(s, n, GridZ, _p(dX), IH, IW, _p(d_deltaY), OH, OW, _p(d_deltaW),
                                                              _p(d_buf), FH, FW, N, IC, OC, sh, sw, ph, pw), name)

    @staticmethod
    def dconv3D_deltaW_GemmSK(*a):
        Cuda_dconv3D_deltaW._sk("GemmSK", *a)

    @staticmethod
    def dconv3D_deltaW_GemmV2SK(*a):
        Cuda_dconv3D_deltaW._sk("GemmV2SK", *a)

    @staticmethod
    def dconv3D_deltaW_GemmSK_W1(streamArray, length, GridZ, dX, IH, IW, d_deltaY, d_deltaW, d_buf, N, IC, OC):
        s, n = _streams(streamArray, length)
        _check(load().cu32_dconv3D_deltaW_GemmSK_W1(s, n, GridZ, _p(dX), IH, IW, _p(d_deltaY), _p(d_deltaW), _p(d_buf),
                                                    N, IC, OC), "dconv3D_deltaW_GemmSK_W1")

    @staticmethod
    def _wino(name, lead, streamArray, length, GridZ, OH_slice, OW_slice, dX, IH, IW, d_deltaY, OH, OW, d_deltaW, d_buf,
              FH, FW, N, IC, OC, ph, pw, n_):
        s, n = _streams(streamArray, length)
        _check(getattr(load(), "cu32_dconv3D_deltaW_Im2col_WinogradV2_SHW_" + name)(
            s, n, GridZ, OH_slice, OW_slice, *lead, _p(dX), IH, IW, _p(d_deltaY), OH, OW, _p(d_deltaW), _p(d_buf), FH, FW,
            N, IC, OC, ph, pw, n_), name)
        return True

    @staticmethod
    def Im2col_WinogradV2_SHW_s4_texture(streamArray, length, GridZ, OH_slice, OW_slice, *a):
        return Cuda_dconv3D_deltaW._wino("s4_texture", (), streamArray, length, GridZ, OH_slice, OW_slice, *a)

    @staticmethod
    def Im2col_WinogradV2_SHW_s8_texture(streamArray, length, GridZ, OH_slice, OW_slice, *a):
        return Cuda_dconv3D_deltaW._wino("s8_texture", (), streamArray, length, GridZ, OH_slice, OW_slice, *a)

    @staticmethod
    def Im2col_WinogradV2_SHW_s16_texture(streamArray, length, GridZ, OH_slice, OW_slice, c64, *a):
        return Cuda_dconv3D_deltaW._wino("s16_texture", (c64,), streamArray, length, GridZ, OH_slice, OW_slice, *a)
