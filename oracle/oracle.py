"""CPU oracle for the Cu32 dense-contraction path (TEST INFRASTRUCTURE ONLY).

Only tests/, ``__graft_entry__.smoke()`` and the CPU-baseline / reference legs of
``bench.py`` import this module, and only as the checker or the timed CPU baseline; the
product library never does.

Three layers:
  * ``ref_loops``  the reference's CPU check loops restated in C (oracle/cu32_oracle.c),
                   FP32 accumulation in the reference's loop order;
  * ``f64``        FP64 contractions (numpy) — the accuracy oracle;
  * ``ref_native`` the reference's own routines compiled from the reference tree into
                   oracle/_ref/ by oracle/build_ref.py, when that build exists.
Error metrics follow the definitions used throughout the reports:
  frob  = ||C - C64||_F / ||C64||_F
  elem  = max_i |C_i - C64_i| / max(|C64_i|, rms(C64))
          A contraction's outputs are sums of signed products, so some of them land
          arbitrarily close to zero; an unfloored elementwise relative error is then unbounded
          for every finite-precision implementation (the reference's FP32 kernels and cuBLAS
          FP32 included).  The floor at the output's RMS magnitude makes the criterion "no
          element is off by more than 1e-4 of the typical output magnitude, and large elements
          are relatively accurate to 1e-4".  `report` also returns the same quantity with the
          floor at 1e-3 * rms and the unfloored 99.9th-percentile relative error, for reference.
  same% = share of elements with |a-b|/|a+b| < thr  (the reference's own gate; meaningful for
          the non-negative inputs the reference's tests use, where no output is near zero)
"""
from __future__ import annotations

import ctypes
import subprocess
from ctypes import POINTER, c_double, c_float, c_int
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
SRC = HERE / "cu32_oracle.c"
LIB = HERE / "libcu32_oracle.so"
REF_DIR = HERE / "_ref"

_lib = None
_fp = POINTER(c_float)
_dp = POINTER(c_double)


def build(force: bool = False) -> Path:
    """Compile cu32_oracle.c with gcc -O2 (no vectorisation flags, like the reference's loops)."""
    if force or not LIB.exists() or LIB.stat().st_mtime < SRC.stat().st_mtime:
        subprocess.run(["gcc", "-O2", "-shared", "-fPIC", "-o", str(LIB), str(SRC), "-lm"], check=True)
    return LIB


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(str(LIB))
        _lib.oracle_samePercent_relative.restype = c_float
        _lib.oracle_samePercent_absolute.restype = c_float
        _lib.oracle_zeroPercent.restype = c_float
    return _lib


def _f(a: np.ndarray):
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_fp)


def _d(a: np.ndarray):
    assert a.dtype == np.float64 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_dp)


def _c32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


# ------------------------------------------------------------------ reference loops (FP32)
class ref_loops:
    """The reference's CPU check loops (restated).  Letters as in the reference."""

    @staticmethod
    def multiply(A, B, N, M, K):
        A, B = _c32(A), _c32(B)
        C = np.zeros((N, M), np.float32)
        lib().oracle_multiply(_f(A), _f(B), _f(C), N, M, K)
        return C

    @staticmethod
    def multiplyT1(A, B, N, M, K):
        A, B = _c32(A), _c32(B)
        C = np.zeros((N, M), np.float32)
        lib().oracle_multiplyT1(_f(A), _f(B), _f(C), N, M, K)
        return C

    @staticmethod
    def multiplyT2(A, B, N, M, K):
        A, B = _c32(A), _c32(B)
        C = np.zeros((N, M), np.float32)
        lib().oracle_multiplyT2(_f(A), _f(B), _f(C), N, M, K)
        return C

    @staticmethod
    def bmm(A, B, Batch, N, CM, BK, AK):
        A, B = _c32(A), _c32(B)
        C = np.zeros((Batch, N, CM), np.float32)
        lib().oracle_bmm(_f(A), _f(B), _f(C), Batch, N, CM, BK, AK)
        return C

    @staticmethod
    def bmmT1(A, B, Batch, CN, AN, CM, K):
        A, B = _c32(A), _c32(B)
        C = np.zeros((Batch, CN, CM), np.float32)
        lib().oracle_bmmT1(_f(A), _f(B), _f(C), Batch, CN, AN, CM, K)
        return C

    @staticmethod
    def bmmT2(A, B, Batch, N, CM, BM, K):
        A, B = _c32(A), _c32(B)
        C = np.zeros((Batch, N, CM), np.float32)
        lib().oracle_bmmT2(_f(A), _f(B), _f(C), Batch, N, CM, BM, K)
        return C

    @staticmethod
    def conv3D_naive(X, W, OH, OW, sh, sw, ph, pw):
        X, W = _c32(X), _c32(W)
        N, IH, IW, IC = X.shape
        OC, FH, FW, _ = W.shape
        Y = np.zeros((N, OH, OW, OC), np.float32)
        lib().oracle_conv3D_naive(_f(X), IH, IW, _f(W), FH, FW, _f(Y), OH, OW, N, IC, OC, sh, sw, ph, pw)
        return Y

    @staticmethod
    def conv3D_img2col(X, W, OH, OW, sh, sw, ph, pw):
        X, W = _c32(X), _c32(W)
        N, IH, IW, IC = X.shape
        OC, FH, FW, _ = W.shape
        Y = np.zeros((N, OH, OW, OC), np.float32)
        lib().oracle_conv3D_img2col(_f(X), IH, IW, _f(W), FH, FW, _f(Y), OH, OW, N, IC, OC, sh, sw, ph, pw)
        return Y

    @staticmethod
    def buf_summary(Cbuf, C, part, sizeC):
        Cbuf, C = _c32(Cbuf), _c32(C).copy()
        lib().oracle_buf_summary(_f(Cbuf), _f(C), part, sizeC)
        return C

    @staticmethod
    def deconv3D_deltaX_img2col_s1(deltaY, W, IH, IW, ph, pw):
        """deltaY [N, OH, OW, OC], W [OC, FH, FW, IC] -> deltaX [N, IH, IW, IC], the reference's float-accumulator
        check loop for the stride-1 data gradient (Cuda_dconv3D_deltaX/test.cuh:154-196)."""
        deltaY, W = _c32(deltaY), _c32(W)
        N, OH, OW, OC = deltaY.shape
        _, FH, FW, IC = W.shape
        dX = np.zeros((N, IH, IW, IC), np.float32)
        lib().oracle_deconv3D_deltaX_img2col_s1(_f(deltaY), OH, OW, _f(W), FH, FW, _f(dX), IH, IW, N, IC, OC, ph, pw)
        return dX

    @staticmethod
    def deconv3D_deltaX_img2col(deltaY, W, IH, IW, sh, sw, ph, pw):
        """Any stride: the reference's float-accumulator check loop (Cuda_dconv3D_deltaX/test.cuh:109-152)."""
        deltaY, W = _c32(deltaY), _c32(W)
        N, OH, OW, OC = deltaY.shape
        _, FH, FW, IC = W.shape
        dX = np.zeros((N, IH, IW, IC), np.float32)
        lib().oracle_deconv3D_deltaX_img2col(_f(deltaY), OH, OW, _f(W), FH, FW, _f(dX), IH, IW, N, IC, OC, sh, sw, ph, pw)
        return dX

    @staticmethod
    def deconv3D_deltaW_naive(X, deltaY, FH, FW, sh, sw, ph, pw):
        """X [N, IH, IW, IC], deltaY [N, OH, OW, OC] -> deltaW [OC, FH, FW, IC]: the Java check loop the reference's
        own weight-gradient test uses (ZUTIL-STD-1.2 Tense.java:1276-1318: float products, double accumulator)."""
        X, deltaY = _c32(X), _c32(deltaY)
        N, IH, IW, IC = X.shape
        _, OH, OW, OC = deltaY.shape
        dW = np.zeros((OC, FH, FW, IC), np.float32)
        lib().oracle_deconv3D_deltaW_naive(_f(X), IH, IW, _f(deltaY), OH, OW, _f(dW), FH, FW, N, IC, OC, sh, sw, ph, pw)
        return dW

    @staticmethod
    def linear2D(alpha, X, beta):
        """Y = alpha * X + beta as the reference's linear2D kernel computes it (type1_linear2D.cuh:40-58): one FMA."""
        X = _c32(X)
        Y = np.empty_like(X)
        lib().oracle_linear2D(c_float(alpha), _f(X), c_float(beta), _f(Y), ctypes.c_longlong(X.size))
        return Y

    @staticmethod
    def softmax2D(X, width=None):
        """Row softmax of X[..., stride] over the first `width` columns as the engine's three-kernel softmax2D
        computes it (see oracle_softmax2D); padding columns come out 0."""
        X = _c32(X)
        stride = X.shape[-1]
        width = stride if width is None else width
        Y = np.empty_like(X)
        lib().oracle_softmax2D(_f(X), _f(Y), ctypes.c_longlong(X.size // stride), stride, width)
        return Y

    @staticmethod
    def ks_remode(W, sh, sw, v2=True, fill=np.nan):
        """W [OC, FH, FW, IC] -> the kernel-split workspace as a flat array of sh*sw*OC*mCFH*mCFW*IC floats
        (dconv3D_dX_kernelSplit_remode_v1.cuh:28-66 / _v2.cuh:31-66); untouched elements keep `fill`."""
        W = _c32(W)
        OC, FH, FW, IC = W.shape
        mCFH, mCFW = (FH + sh - 1) // sh, (FW + sw - 1) // sw
        CW = np.full(sh * sw * OC * mCFH * mCFW * IC, fill, np.float32)
        lib().oracle_ks_remode(1 if v2 else 0, _f(W), FH, FW, _f(CW), mCFH, mCFW, OC, IC, sh, sw)
        return CW

    @staticmethod
    def linear_dual2D_row(X1, X2, alpha, beta, gamma, width):
        """X1 [height, stride] (stride = padded row length), X2 [stride]: Y = alpha*X1 + beta*X2 + gamma per
        row, columns >= width zeroed (Cuda_function/type1_linear_dual2D_row.cuh:41-70)."""
        X1, X2 = _c32(X1), _c32(X2)
        height, stride = X1.shape
        Y = np.empty_like(X1)
        lib().oracle_linear_dual2D_row(_f(X1), _f(X2), int(X2.size), c_float(alpha), c_float(beta), c_float(gamma),
                                       _f(Y), height * stride, int(width), stride)
        return Y

    @staticmethod
    def kernel_remode(W):
        W = _c32(W)
        OC, FH, FW, IC = W.shape
        CW = np.zeros((FH, FW, IC, OC), np.float32)
        lib().oracle_kernel_remode(_f(W), _f(CW), FH, FW, OC, IC)
        return CW


def same_percent(a, b, threshold=1e-5, absolute=False) -> float:
    a, b = _c32(a).ravel(), _c32(b).ravel()
    fn = lib().oracle_samePercent_absolute if absolute else lib().oracle_samePercent_relative
    return float(fn(_f(a), _f(b), a.size, c_float(threshold)))


def zero_percent(a) -> float:
    a = _c32(a).ravel()
    return float(lib().oracle_zeroPercent(_f(a), a.size))


# ------------------------------------------------------------------ FP64 oracle
class f64:
    """FP64 contractions of FP32 inputs; results are float64 arrays."""

    @staticmethod
    def matMul(A, B):
        return np.asarray(A, np.float64) @ np.asarray(B, np.float64)

    @staticmethod
    def matMulT1(A, B):
        return np.asarray(A, np.float64).T @ np.asarray(B, np.float64)

    @staticmethod
    def matMulT2(A, B):
        return np.asarray(A, np.float64) @ np.asarray(B, np.float64).T

    @staticmethod
    def batchMatMul(A, B, BK=None):
        A, B = np.asarray(A, np.float64), np.asarray(B, np.float64)
        if BK is not None:
            A = A[:, :, :BK]
        return np.matmul(A, B)

    @staticmethod
    def batchMatMulT1(A, B, CN=None):
        A, B = np.asarray(A, np.float64), np.asarray(B, np.float64)
        if CN is not None:
            A = A[:, :, :CN]
        return np.matmul(A.transpose(0, 2, 1), B)

    @staticmethod
    def batchMatMulT2(A, B, CM=None):
        A, B = np.asarray(A, np.float64), np.asarray(B, np.float64)
        C = np.matmul(A, B.transpose(0, 2, 1))
        if CM is not None and CM > C.shape[2]:
            C = np.concatenate([C, np.zeros(C.shape[:2] + (CM - C.shape[2],))], axis=2)
        return C

    @staticmethod
    def softmax_rows(S, alpha=1.0, width=None):
        """softmax over the last axis of alpha * S in FP64 (S float64 scores); columns >= width are padding: 0."""
        S = np.asarray(S, np.float64) * np.float64(np.float32(alpha))
        width = S.shape[-1] if width is None else width
        Z = S[..., :width]
        Z = np.exp(Z - Z.max(axis=-1, keepdims=True))
        Z /= Z.sum(axis=-1, keepdims=True)
        out = np.zeros(S.shape, np.float64)
        out[..., :width] = Z
        return out

    @staticmethod
    def conv3D(X, W, OH, OW, sh, sw, ph, pw, n_begin=0, n_end=None):
        """Forward convolution, NHWC / OCxFHxFWxIC, zero padding, via im2col in FP64."""
        X, W = np.asarray(X, np.float64), np.asarray(W, np.float64)
        N, IH, IW, IC = X.shape
        OC, FH, FW, _ = W.shape
        n_end = N if n_end is None else n_end
        Xs = X[n_begin:n_end]
        # pad so that every tap of every output position exists
        need_h = (OH - 1) * sh + FH
        need_w = (OW - 1) * sw + FW
        Xp = np.zeros((Xs.shape[0], max(need_h, IH + 2 * ph), max(need_w, IW + 2 * pw), IC))
        Xp[:, ph:ph + IH, pw:pw + IW, :] = Xs
        Y = np.zeros((Xs.shape[0], OH, OW, OC))
        for fh in range(FH):
            for fw in range(FW):
                patch = Xp[:, fh:fh + (OH - 1) * sh + 1:sh, fw:fw + (OW - 1) * sw + 1:sw, :]
                Y += patch @ W[:, fh, fw, :].T
        return Y


# ------------------------------------------------------------------ metrics
def f64_deconv3D_deltaX_s1(deltaY, W, IH, IW, ph, pw):
    """FP64 data gradient of the stride-1 convolution (accuracy oracle for the deltaX entry points)."""
    deltaY, W = _c32(deltaY), _c32(W)
    N, OH, OW, OC = deltaY.shape
    _, FH, FW, IC = W.shape
    dX = np.zeros((N, IH, IW, IC), np.float64)
    lib().oracle_deconv3D_deltaX_s1_f64(_f(deltaY), OH, OW, _f(W), FH, FW, _d(dX), IH, IW, N, IC, OC, ph, pw)
    return dX


f64.deconv3D_deltaX_s1 = staticmethod(f64_deconv3D_deltaX_s1)


def f64_deconv3D_deltaX(deltaY, W, IH, IW, sh, sw, ph, pw):
    """FP64 data gradient of the convolution for any stride."""
    deltaY, W = _c32(deltaY), _c32(W)
    N, OH, OW, OC = deltaY.shape
    _, FH, FW, IC = W.shape
    dX = np.zeros((N, IH, IW, IC), np.float64)
    lib().oracle_deconv3D_deltaX_f64(_f(deltaY), OH, OW, _f(W), FH, FW, _d(dX), IH, IW, N, IC, OC, sh, sw, ph, pw)
    return dX


f64.deconv3D_deltaX = staticmethod(f64_deconv3D_deltaX)


def frob_rel(C, C64) -> float:
    C64 = np.asarray(C64, np.float64)
    d = np.asarray(C, np.float64) - C64
    return float(np.linalg.norm(d.ravel()) / max(np.linalg.norm(C64.ravel()), 1e-300))


def elem_rel(C, C64, tau_factor: float = 1.0) -> float:
    C64 = np.asarray(C64, np.float64)
    d = np.abs(np.asarray(C, np.float64) - C64)
    rms = float(np.sqrt(np.mean(C64 * C64)))
    tau = tau_factor * rms if rms > 0 else 1.0
    return float(np.max(d / np.maximum(np.abs(C64), tau)))


def report(C, C64) -> dict:
    C64 = np.asarray(C64, np.float64)
    d = np.abs(np.asarray(C, np.float64) - C64)
    nz = np.abs(C64) > 0
    rel = d[nz] / np.abs(C64[nz]) if nz.any() else np.zeros(1)
    return {"frob": frob_rel(C, C64), "elem": elem_rel(C, C64), "elem_floor1e-3": elem_rel(C, C64, 1e-3),
            "rel_p999": float(np.quantile(rel, 0.999)) if rel.size else 0.0}


# ------------------------------------------------------------------ reference's own routines
def ref_native(name: str):
    """ctypes handle on oracle/_ref/libref_<name>.so ('matmul', 'bmm', 'conv', 'function'), or None if
    that build is absent (it needs the reference tree; see oracle/build_ref.py)."""
    p = REF_DIR / f"libref_{name}.so"
    if not p.exists():
        return None
    try:
        l = ctypes.CDLL(str(p))
    except OSError:
        return None
    if hasattr(l, "ref_cpu_samePercent"):
        l.ref_cpu_samePercent.restype = c_float
    return l


def f64_deconv3D_deltaW(X, deltaY, FH, FW, sh, sw, ph, pw):
    """Weight gradient in FP64: deltaW [OC, FH, FW, IC] (float64)."""
    X, deltaY = _c32(X), _c32(deltaY)
    N, IH, IW, IC = X.shape
    _, OH, OW, OC = deltaY.shape
    dW = np.zeros((OC, FH, FW, IC), np.float64)
    lib().oracle_deconv3D_deltaW_f64(_f(X), IH, IW, _f(deltaY), OH, OW, _d(dW), FH, FW, N, IC, OC, sh, sw, ph, pw)
    return dW


f64.deconv3D_deltaW = staticmethod(f64_deconv3D_deltaW)
