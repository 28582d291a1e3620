"""Host-side mirror of the caller of the Cu32 natives.

``CudaFloat32EngineBase`` (z/dragon/engine/cuda/CudaFloat32EngineBase.java) decides, for
every matMul / matMulT1 / matMulT2, whether to split the reduction axis, sizes the partial
buffer, calls the natives and then the buffer summation; ``EngineCore`` pads dimensions to
multiples of 4 before that.  This module restates that integer logic so that tests and the
benchmark drive the natives the way the Java engine does, and provides a small engine
object working on device addresses.

Only integers and device addresses are handled here; device memory comes from a
caller-supplied ``malloc(nfloats) -> (address, keepalive)`` (the Java engine's
``core.malloc``), so this module does not depend on any array library.
"""
from __future__ import annotations

from dataclasses import dataclass

from .cu32 import Cuda_batchMatMul, Cuda_conv3D, Cuda_matMul


def pad4(x: int) -> int:
    """EngineCore pads every matrix dimension to a multiple of 4 (EngineCore.java:708-717)."""
    return (x + 3) >> 2 << 2


@dataclass
class SplitKConfig:
    """Per-form split-K constants (CudaFloat32EngineBase.java:1474-1477, :1691-1695, :1810-1814)."""
    threshold: int = 512
    maxPart: int = 16
    minBlock_perSM: float = 1.2
    maxBlock_perSM: float = 4.0


MATMUL_SK = SplitKConfig(512, 16, 1.2, 4.0)
MATMUL_T1_SK = SplitKConfig(512, 16, 1.14, 4.0)
MATMUL_T2_SK = SplitKConfig(512, 16, 1.14, 4.0)


def _clamp_gridz(fGridZ: float, K: int, sm_count: int, maxBlock_perSM: float, b: int, maxPart: int) -> int:
    GridZ = int(fGridZ)
    GridZ2 = K >> 8
    if GridZ > GridZ2:
        GridZ = GridZ2
    coef = K / (K + 4096.0)
    GridZ3 = int(sm_count * maxBlock_perSM * coef / b)
    if GridZ > GridZ3:
        GridZ = GridZ3
    GridZ = 2 if GridZ < 2 else (GridZ + 3) >> 2 << 2
    if GridZ > maxPart:
        GridZ = maxPart
    return GridZ


def matMul_gridZ(N: int, M: int, K: int, sm_count: int, cfg: SplitKConfig = MATMUL_SK) -> int:
    """GridZ the Java engine uses for C[N,M] = A[N,K] B[K,M]; 1 = no split
    (CudaFloat32EngineBase.java:1523-1562)."""
    fGridZ, b0 = 1.0, 1
    if K >= cfg.threshold:
        b0 = Cuda_matMul.blockNum(N, M)
        expect = cfg.minBlock_perSM + 0.4 * K / (K + 1024.0)
        if b0 < sm_count * expect:
            b1 = Cuda_matMul.blockNum(K, M)
            b2 = Cuda_matMul.blockNum(N, K)
            fGridZ = (b1 + b2) / (b0 * 2.0)
    if fGridZ < 1.8:
        return 1
    return _clamp_gridz(fGridZ, K, sm_count, cfg.maxBlock_perSM, b0, cfg.maxPart)


def matMulT1_gridZ(N: int, M: int, K: int, sm_count: int, cfg: SplitKConfig = MATMUL_T1_SK) -> int:
    """GridZ for C[N,M] = A[K,N]^T B[K,M] (CudaFloat32EngineBase.java:1740-1779)."""
    fGridZ, b1 = 1.0, 1
    if K >= cfg.threshold:
        b1 = Cuda_matMul.blockNum(N, M)
        expect = cfg.minBlock_perSM + K / (K + 1024.0)
        if b1 < sm_count * expect:
            b0 = Cuda_matMul.blockNum(K, N)
            b2 = Cuda_matMul.blockNum(K, M)
            fGridZ = (b0 + b2) / (b1 * 2.0)
    if fGridZ < 1.8:
        return 1
    return _clamp_gridz(fGridZ, K, sm_count, cfg.maxBlock_perSM, b1, cfg.maxPart)


def matMulT2_gridZ(N: int, M: int, K: int, sm_count: int, cfg: SplitKConfig = MATMUL_T2_SK,
                   matMul_cfg: SplitKConfig = MATMUL_SK) -> int:
    """GridZ for C[N,M] = A[N,K] B[M,K]^T (CudaFloat32EngineBase.java:1859-1898).  The Java
    code compares blockNum(N, K) against the *matMul* constants and divides by blockNum(N, M);
    that is reproduced as written."""
    fGridZ, b2 = 1.0, 1
    if K >= cfg.threshold:
        b2 = Cuda_matMul.blockNum(N, K)
        expect = matMul_cfg.minBlock_perSM + K / (K + 1024.0)
        if b2 < sm_count * expect:
            b0 = Cuda_matMul.blockNum(N, M)
            b1 = Cuda_matMul.blockNum(K, M)
            fGridZ = (b1 + b2) / (b0 * 2.0)
    if fGridZ < 1.8:
        return 1
    return _clamp_gridz(fGridZ, K, sm_count, matMul_cfg.maxBlock_perSM, b2, cfg.maxPart)


def conv_out_dim(I: int, F: int, s: int, p: int) -> int:
    """Output extent of the forward convolution (Cuda_conv3D micro_Gemm.cuh:11 GET_OUT_DIM)."""
    return (I + 2 * p - F) // s + 1


CONV3D_DW_SK = SplitKConfig(512, 16, 1.5, 4.0)


def conv3D_deltaW_gridZ(OH: int, OW: int, IH: int, IW: int, FH: int, FW: int, N: int, IC: int, OC: int, sm_count: int,
                        cfg: SplitKConfig = CONV3D_DW_SK) -> int:
    """GridZ of the convolution's weight gradient (CudaFloat32EngineBase.java:3519-3522 threshold, :3166-3187 rule):
    no split below `threshold` output pixels or when the [OC x FH*FW*IC] output alone gives every SM enough thread
    blocks; else the ratio of the forward and data-gradient block counts to the weight gradient's, capped by 256
    pixels per slice, by maxBlock_perSM and by maxPart, and rounded up to a multiple of 4."""
    GK = N * OH * OW
    if GK < cfg.threshold:
        return 1
    expect = cfg.minBlock_perSM * (GK / (GK + 1024.0))
    b2 = Cuda_matMul.blockNum(OC, FH * FW * IC)         # Cuda_dconv3D_deltaW.GEMM_nblock
    if b2 >= sm_count * expect:
        return 1
    b0 = Cuda_matMul.blockNum(OC, N * OH * OW)          # Cuda_conv3D.GEMM_nblock
    b1 = Cuda_matMul.blockNum(IC, N * IH * IW)          # Cuda_dconv3D_deltaX.GEMM_nblock
    GZ = (b0 + b1) // (b2 << 1)
    GZ = min(GZ, GK >> 8, int(sm_count * cfg.maxBlock_perSM / b2))
    GZ = 2 if GZ < 2 else (GZ + 3) >> 2 << 2
    return min(GZ, cfg.maxPart)


class Cu32Engine:
    """The hot-path methods of CudaFloat32EngineBase on raw device addresses.

    ``malloc(nfloats)`` must return ``(address, keepalive)`` for a device buffer of that many
    floats; ``streams`` is a list of stream handles (integers), at least one.
    """

    def __init__(self, sm_count: int, malloc, streams, tf32: bool = False):
        self.sm_count = sm_count
        self.malloc = malloc
        self.streams = list(streams)
        self.tf32 = tf32
        self._keep = []

    def _stream_array(self, N, M):
        n = min(Cuda_matMul.nstream(N, M), len(self.streams))
        return self.streams[:n], n

    def _run(self, plain, mma, sk, gz, C, A, B, N, M, K):
        sa, n = self._stream_array(N, M)
        if gz == 1:
            if self.tf32 and N > 127 and M > 127 and K % 8 == 0:
                mma(sa, n, A, B, C, N, M, K)
            else:
                plain(sa, n, A, B, C, N, M, K)
            return 1
        part, sizeC = gz - 1, N * M
        Cbuf, keep = self.malloc(sizeC * part)
        self._keep.append(keep)
        sk(sa, n, gz, A, B, C, Cbuf, N, M, K)
        Cuda_matMul.SKbuf_summary(sa[0], Cbuf, C, part, sizeC)
        return gz

    def matMul(self, C, A, B, N, M, K):
        gz = matMul_gridZ(N, M, K, self.sm_count)
        return self._run(Cuda_matMul.matMul, Cuda_matMul.matMul_mma, Cuda_matMul.matMulSK, gz, C, A, B, N, M, K)

    def matMul_biased(self, C, A, B, N, M, K, Bias, width):
        """CudaFloat32EngineBase.matMul_biased (:1594-1688) with the bias row fused: one native instead of
        product + linear_dual2D_row when K is not split, matMulSK + SKbuf_summary_biased when it is.
        The split decision is the engine's own (same as matMul)."""
        gz = matMul_gridZ(N, M, K, self.sm_count)
        sa, n = self._stream_array(N, M)
        if gz == 1:
            fn = Cuda_matMul.matMul_mma_biased if (self.tf32 and N > 127 and M > 127 and K % 8 == 0) \
                else Cuda_matMul.matMul_biased
            fn(sa, n, A, B, C, Bias, N, M, K, width)
            return 1
        part, sizeC = gz - 1, N * M
        Cbuf, keep = self.malloc(sizeC * part)
        self._keep.append(keep)
        Cuda_matMul.matMulSK(sa, n, gz, A, B, C, Cbuf, N, M, K)
        Cuda_matMul.SKbuf_summary_biased(sa[0], Cbuf, C, Bias, part, sizeC, M, width)
        return gz

    def matMulT1(self, C, A, B, N, M, K):
        gz = matMulT1_gridZ(N, M, K, self.sm_count)
        return self._run(Cuda_matMul.matMulT1, Cuda_matMul.matMulT1_mma, Cuda_matMul.matMulT1SK, gz, C, A, B, N, M, K)

    def matMulT2(self, C, A, B, N, M, K):
        gz = matMulT2_gridZ(N, M, K, self.sm_count)
        return self._run(Cuda_matMul.matMulT2, Cuda_matMul.matMulT2_mma, Cuda_matMul.matMulT2SK, gz, C, A, B, N, M, K)

    def batchMatMul(self, C, A, B, Batch, N, M, BK, AK):
        sa, n = self._stream_array(N, M)
        Cuda_batchMatMul.batchMatMul_texture(sa, n, A, B, C, Batch, N, M, BK, AK)

    def batchMatMulT1(self, C, A, B, Batch, CN, AN, M, K):
        sa, n = self._stream_array(CN, M)
        Cuda_batchMatMul.batchMatMulT1(sa, n, A, B, C, Batch, CN, AN, M, K)

    def batchMatMulT2(self, C, A, B, Batch, N, CM, BM, K):
        sa, n = self._stream_array(N, CM)
        Cuda_batchMatMul.batchMatMulT2_texture(sa, n, A, B, C, Batch, N, CM, BM, K)

    def batchMatMulT1_sdiv(self, C, A, B, Batch, CN, AN, M, K, divisor):
        """sdiv(divisor, batchMatMulT1(A, B)) - the attention block's scaled scores (ImageMHA.java:67-68) - in one
        kernel; alpha is formed as the Java engine forms it, 1.0f / divisor in FP32 (Engine.java:4002)."""
        import numpy as np
        sa, n = self._stream_array(CN, M)
        alpha = float(np.float32(1.0) / np.float32(divisor))
        Cuda_batchMatMul.batchMatMulT1_scaled(sa, n, A, B, C, Batch, CN, AN, M, K, alpha)

    def batchMatMulT2_sdiv(self, C, A, B, Batch, N, CM, BM, K, divisor):
        import numpy as np
        sa, n = self._stream_array(N, CM)
        alpha = float(np.float32(1.0) / np.float32(divisor))
        Cuda_batchMatMul.batchMatMulT2_scaled(sa, n, A, B, C, Batch, N, CM, BM, K, alpha)

    def conv3D(self, Y, OH, OW, X, IH, IW, W, FH, FW, N, IC, OC, sh, sw, ph, pw):
        """Forward convolution the way the Java engine runs its GEMMR branch: remode the
        filter on streams[0], then the implicit GEMM (CudaFloat32EngineBase.java:2268-2332)."""
        CW, keep = self.malloc(FH * FW * IC * OC)
        self._keep.append(keep)
        Cuda_conv3D.kernel_remode(self.streams[0], W, CW, FH, FW, OC, IC)
        GM, GK = N * OH * OW, FH * FW * IC
        sl = Cuda_conv3D.GEMM_GM_slice(OC, GM, GK)
        sa = self.streams[:1]
        if FH == 1 and FW == 1 and sh == 1 and sw == 1 and ph == 0 and pw == 0:
            Cuda_conv3D.conv3D_GemmR_W1(sa, 1, X, IH, IW, W, CW, Y, N, IC, OC)
        elif sl < 0:
            Cuda_conv3D.conv3D_GemmR(sa, 1, X, IH, IW, W, CW, FH, FW, Y, OH, OW, N, IC, OC, sh, sw, ph, pw)
        else:
            Cuda_conv3D.conv3D_GemmR_SGM(sa, 1, X, IH, IW, W, CW, FH, FW, Y, OH, OW, N, IC, OC, sh, sw, ph, pw, sl)

    def conv3D_deltaX(self, deltaX, IH, IW, deltaY, OH, OW, W, FH, FW, N, IC, OC, sh, sw, ph, pw):
        """Data gradient the way the Java engine runs it (CudaFloat32EngineBase.java:3773-3900).  Stride 1: 1x1
        filters take the W1 native, everything else the zero-padding s1 native.  Strides > 1: rearrange the filter
        into the kernel-split workspace CW[sh][sw][CFH][CFW][OC][IC] with ks_remodev2 on streams[0], then the
        Ims2R native for stride 2 x 2 and the ImsR native otherwise."""
        from .cu32 import Cuda_dconv3D_deltaX as dx
        sa = self.streams[:1]
        if sh != 1 or sw != 1:
            CFH, CFW = (FH + sh - 1) // sh, (FW + sw - 1) // sw
            CW, keep = self.malloc(OC * CFH * CFW * IC * sh * sw)
            self._keep.append(keep)
            dx.ks_remodev2(self.streams[0], W, FH, FW, CW, CFH, CFW, OC, IC, sh, sw)
            if sh == 2 and sw == 2:
                dx.dconv3D_deltaX_ksIms2R(sa, 1, deltaY, OH, OW, CW, FH, FW, deltaX, IH, IW, N, IC, OC, ph, pw)
            else:
                dx.dconv3D_deltaX_ksImsR(sa, 1, deltaY, OH, OW, CW, FH, FW, deltaX, IH, IW, N, IC, OC, sh, sw, ph, pw)
        elif FH == 1 and FW == 1 and ph == 0 and pw == 0:
            dx.dconv3D_deltaX_W1(sa, 1, deltaY, W, deltaX, IH, IW, N, IC, OC)
        else:
            dx.dconv3D_deltaX_s1(sa, 1, deltaY, OH, OW, W, FH, FW, deltaX, IH, IW, N, IC, OC, ph, pw)

    def conv3D_deltaW(self, deltaW, FH, FW, X, IH, IW, deltaY, OH, OW, N, IC, OC, sh, sw, ph, pw, GridZ=None):
        """Weight gradient the way the Java engine runs its split-K branch (CudaFloat32EngineBase.java:3541-3640):
        partial buffers for GridZ - 1 slices from the pool, the GemmSK native (W1 form for 1x1 filters), then
        buf_summary on streams[0].  GridZ: the caller's, else the Java engine's own rule (conv3D_deltaW_gridZ)."""
        from .cu32 import Cuda_dconv3D_deltaW as dw
        sa = self.streams[:1]
        if GridZ is None:
            GridZ = conv3D_deltaW_gridZ(OH, OW, IH, IW, FH, FW, N, IC, OC, self.sm_count)
        size = OC * FH * FW * IC
        buf = 0
        if GridZ > 1:
            buf, keep = self.malloc((GridZ - 1) * size)
            self._keep.append(keep)
        if FH == 1 and FW == 1 and sh == 1 and sw == 1 and ph == 0 and pw == 0:
            if GridZ > 1:
                dw.dconv3D_deltaW_GemmSK_W1(sa, 1, GridZ, X, IH, IW, deltaY, deltaW, buf, N, IC, OC)
            else:
                dw.dconv3D_deltaW_W1(sa, 1, X, IH, IW, deltaY, deltaW, N, IC, OC)
        elif GridZ > 1:
            dw.dconv3D_deltaW_GemmSK(sa, 1, GridZ, X, IH, IW, deltaY, OH, OW, deltaW, buf, FH, FW, N, IC, OC, sh, sw, ph, pw)
        else:
            dw.dconv3D_deltaW(sa, 1, X, IH, IW, deltaY, OH, OW, deltaW, FH, FW, N, IC, OC, sh, sw, ph, pw)
        if GridZ > 1:
            dw.buf_summary(self.streams[0], buf, deltaW, GridZ - 1, size)
        return GridZ

    def release(self):
        """Drop the workspaces (the Java Syncer frees them after the streams complete)."""
        self._keep.clear()
