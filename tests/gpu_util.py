"""Helpers for the GPU parity tests: run an entry point of the C ABI on torch device buffers
the way the Java engine would (dimensions already padded to multiples of 4, stream handles as
integers) and hand back host arrays.  Outputs are surrounded by canary floats so that a store
outside the output is caught."""
from __future__ import annotations

import numpy as np
import torch

CANARY = 12345.678
PAD = 64


class Out:
    """Device output buffer of `n` floats with PAD canary floats on both sides, NaN-filled."""

    def __init__(self, n: int):
        self.n = n
        self.buf = torch.full((n + 2 * PAD,), CANARY, device="cuda", dtype=torch.float32)
        self.view = self.buf[PAD:PAD + n]
        self.view.fill_(float("nan"))

    @property
    def ptr(self) -> int:
        return self.view.data_ptr()

    def host(self, shape) -> np.ndarray:
        torch.cuda.synchronize()
        h = self.buf.cpu().numpy()
        assert np.all(h[:PAD] == np.float32(CANARY)) and np.all(h[PAD + self.n:] == np.float32(CANARY)), \
            "store outside the output buffer"
        return h[PAD:PAD + self.n].reshape(shape).copy()


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def dev(a) -> torch.Tensor:
    t = torch.as_tensor(np.ascontiguousarray(a, dtype=np.float32)) if not isinstance(a, torch.Tensor) else a
    return t.contiguous().cuda()


def check_status(pkg):
    st = pkg.cu32.read_status()
    assert st == 0, "kernel gave up: " + pkg.cu32.decode_status(st)


def matmul(pkg, form, A, B, N, M, K, mma=False):
    mm = pkg.cu32.Cuda_matMul
    fn = {("AB", False): mm.matMul, ("T1", False): mm.matMulT1, ("T2", False): mm.matMulT2,
          ("AB", True): mm.matMul_mma, ("T1", True): mm.matMulT1_mma, ("T2", True): mm.matMulT2_mma}[(form, mma)]
    dA, dB = dev(A), dev(B)
    out = Out(N * M)
    fn([stream()], 1, dA.data_ptr(), dB.data_ptr(), out.ptr, N, M, K)
    C = out.host((N, M))
    check_status(pkg)
    return C


def matmul_sk(pkg, form, A, B, N, M, K, GZ, summary=True):
    mm = pkg.cu32.Cuda_matMul
    fn = {"AB": mm.matMulSK, "T1": mm.matMulT1SK, "T2": mm.matMulT2SK}[form]
    dA, dB = dev(A), dev(B)
    out = Out(N * M)
    buf = Out(N * M * (GZ - 1))
    fn([stream()], 1, GZ, dA.data_ptr(), dB.data_ptr(), out.ptr, buf.ptr, N, M, K)
    C0 = out.host((N, M))
    Cbuf = buf.host((GZ - 1, N, M))
    if summary:
        mm.SKbuf_summary(stream(), buf.ptr, out.ptr, GZ - 1, N * M)
    C = out.host((N, M))
    check_status(pkg)
    return C, C0, Cbuf


def bmm_t2(pkg, Q, Kt):
    """C[b] = Q[b] * Kt[b]^T through batchMatMulT2 (Q [Batch, N, K], Kt [Batch, M, K])."""
    Batch, N, K = Q.shape
    M = Kt.shape[1]
    dQ, dK = dev(Q), dev(Kt)
    out = Out(Batch * N * M)
    pkg.cu32.Cuda_batchMatMul.batchMatMulT2([stream()], 1, dQ.data_ptr(), dK.data_ptr(), out.ptr, Batch, N, M, M, K)
    C = out.host((Batch, N, M))
    check_status(pkg)
    return C


def f64_matmul(O, form, A, B):
    return {"AB": O.f64.matMul, "T1": O.f64.matMulT1, "T2": O.f64.matMulT2}[form](A, B)


def ref_matmul(O, form, A, B, N, M, K):
    return {"AB": O.ref_loops.multiply, "T1": O.ref_loops.multiplyT1, "T2": O.ref_loops.multiplyT2}[form](A, B, N, M, K)


def mm_shapes(form, N, M, K):
    return {"AB": ((N, K), (K, M)), "T1": ((K, N), (K, M)), "T2": ((N, K), (M, K))}[form]


def rand_pm1(shape, seed):
    g = torch.Generator().manual_seed(seed)
    return (torch.rand(shape, generator=g, dtype=torch.float32) * 2 - 1).numpy()


def conv(pkg, entry, X, W, sh, sw, ph, pw, OH=None, OW=None, GM_slice=None):
    cv = pkg.cu32.Cuda_conv3D
    N, IH, IW, IC = X.shape
    OC, FH, FW, _ = W.shape
    OH = (IH + 2 * ph - FH) // sh + 1 if OH is None else OH
    OW = (IW + 2 * pw - FW) // sw + 1 if OW is None else OW
    dX, dW = dev(X), dev(W)
    out = Out(N * OH * OW * OC)
    s = [stream()]
    if entry in ("conv3D_GemmR", "conv3D_GemmR_texture", "conv3D_GemmR_SGM", "conv3D_GemmR_texture_SGM"):
        dCW = torch.empty(FH * FW * IC * OC, device="cuda")
        cv.kernel_remode(s[0], dW.data_ptr(), dCW.data_ptr(), FH, FW, OC, IC)
        args = [s, 1, dX.data_ptr(), IH, IW, dW.data_ptr(), dCW.data_ptr(), FH, FW, out.ptr, OH, OW, N, IC, OC,
                sh, sw, ph, pw]
        if entry.endswith("SGM"):
            args.append(GM_slice or 128)
        getattr(cv, entry)(*args)
    elif entry in ("conv3D_GemmV2R", "conv3D_Im2col_Winograd_s8_R_texture", "conv3D_Im2col_WinogradR_s8_texture_SGM",
                   "conv3D_Im2col_Winograd_s16_R_texture", "conv3D_Im2col_WinogradR_s16_texture_SGM"):
        dCW = torch.empty(FH * FW * IC * OC, device="cuda")
        cv.kernel_remode(s[0], dW.data_ptr(), dCW.data_ptr(), FH, FW, OC, IC)
        args = [True, s, 1, dX.data_ptr(), IH, IW, dW.data_ptr(), dCW.data_ptr(), FH, FW, out.ptr, OH, OW, N, IC, OC]
        if entry == "conv3D_GemmV2R":
            args += [sh, sw]
        else:
            assert sh == 1 and sw == 1, "the Winograd natives are stride-1 only"
        args += [ph, pw]
        if entry.endswith("SGM"):
            args.append(GM_slice or 128)
        handled = getattr(cv, entry)(*args)
        assert entry == "conv3D_GemmV2R" or handled is True
    elif entry == "conv3DV2":
        cv.conv3DV2(False, s, 1, dX.data_ptr(), IH, IW, dW.data_ptr(), FH, FW, out.ptr, OH, OW, N, IC, OC, sh, sw, ph, pw)
    elif entry in ("conv3D", "conv3D_texture"):
        getattr(cv, entry)(s, 1, dX.data_ptr(), IH, IW, dW.data_ptr(), FH, FW, out.ptr, OH, OW, N, IC, OC, sh, sw, ph, pw)
    elif entry == "conv3D_np":
        cv.conv3D_np(s, 1, dX.data_ptr(), IH, IW, dW.data_ptr(), FH, FW, out.ptr, OH, OW, N, IC, OC, sh, sw)
    elif entry == "conv3D_W1":
        cv.conv3D_W1(s, 1, dX.data_ptr(), IH, IW, dW.data_ptr(), out.ptr, N, IC, OC)
    elif entry in ("conv3D_GemmR_W1", "conv3D_GemmR_W1_SGM"):
        dCW = torch.empty(IC * OC, device="cuda")
        cv.kernel_remode(s[0], dW.data_ptr(), dCW.data_ptr(), 1, 1, OC, IC)
        args = [s, 1, dX.data_ptr(), IH, IW, dW.data_ptr(), dCW.data_ptr(), out.ptr, N, IC, OC]
        if entry.endswith("SGM"):
            args.append(GM_slice or 128)
        getattr(cv, entry)(*args)
    else:
        raise ValueError(entry)
    Y = out.host((N, OH, OW, OC))
    check_status(pkg)
    return Y
