"""Generate the golden fixtures in this directory from the REFERENCE'S OWN CPU routines.

Run in a container that has the reference tree: ``python oracle/build_ref.py [--conv]`` builds
the reference's test.cuh loops (multiply*, bmm*, CONV_3D_NAIVE, CONV_3D_img2col, and with --deltax
deconv3D_deltaX_img2col_s1) into
oracle/_ref/, and this script runs them on small seeded inputs and stores inputs' seeds,
shapes and the outputs as .npz.  The fixtures then travel with the repository, so the CPU
oracle (tests/test_oracle.py) and the GPU kernels (tests/test_parity_gpu.py) can be checked
against the reference's results where the reference tree does not exist.

Inputs are regenerated from the seed by ``golden_inputs`` below (numpy PCG64, FP32), so only
the outputs are stored.
"""
from __future__ import annotations

import ctypes
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))

FP = ctypes.POINTER(ctypes.c_float)

# name -> (kind, dims...)
MATMUL_CASES = {
    "mm_ab_52x36x40": ("AB", 52, 36, 40),
    "mm_ab_128x128x64": ("AB", 128, 128, 64),
    "mm_ab_200x260x132": ("AB", 200, 260, 132),
    "mm_t1_68x44x516": ("T1", 68, 44, 516),
    "mm_t1_132x256x96": ("T1", 132, 256, 96),
    "mm_t2_36x300x128": ("T2", 36, 300, 128),
    "mm_t2_256x132x200": ("T2", 256, 132, 200),
}
BMM_CASES = {
    # kind, Batch, then the native's four dims
    "bmm_ab_3x37x20x30": ("AB", 3, 37, 20, 30, 32),     # N, M(CM), BK, AK
    "bmm_t1_2x50x52x24x40": ("T1", 2, 50, 52, 24, 40),  # CN, AN, M, K
    "bmm_t2_4x33x68x66x16": ("T2", 4, 33, 68, 66, 16),  # N, CM, BM, K
}
CONV_CASES = {
    # N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw
    "conv_3x3_s1p1": (4, 9, 9, 8, 12, 3, 3, 1, 1, 1, 1),
    "conv_5x3_s2p2": (4, 11, 10, 4, 8, 5, 3, 2, 2, 2, 1),
    "conv_1x1": (4, 6, 6, 16, 20, 1, 1, 1, 1, 0, 0),
    "conv_3x3_np": (4, 8, 8, 36, 8, 3, 3, 1, 1, 0, 0),
}


DELTAX_CASES = {
    # stride-1 data gradient: N, IH, IW, IC, OC, FH, FW, ph, pw
    "dx_3x3_p1": (3, 9, 8, 8, 12, 3, 3, 1, 1),
    "dx_5x3_p2p0": (2, 10, 11, 4, 8, 5, 3, 2, 0),
    "dx_1x1": (4, 6, 6, 16, 20, 1, 1, 0, 0),
    "dx_2x4_p1p3": (2, 7, 9, 12, 4, 2, 4, 1, 3),
}
DELTAX_STRIDED_CASES = {
    # any-stride data gradient: N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw
    "dxs_3x3_s2_p1": (3, 9, 8, 8, 12, 3, 3, 2, 2, 1, 1),
    "dxs_5x3_s2_p2p1": (2, 11, 10, 4, 8, 5, 3, 2, 2, 2, 1),
    "dxs_3x3_s3_p1": (2, 10, 11, 8, 4, 3, 3, 3, 3, 1, 1),
    "dxs_1x1_s2": (2, 8, 8, 8, 8, 1, 1, 2, 2, 0, 0),
    "dxs_4x4_s2s1_p1p2": (2, 10, 13, 4, 8, 4, 4, 2, 1, 1, 2),
}


def golden_inputs(name: str, shapes):
    """FP32 inputs in [0,1) (the reference tests' distribution), seeded by the case name."""
    seed = int.from_bytes(name.encode(), "little") % (2 ** 32)
    rng = np.random.default_rng(seed)
    return [rng.random(s, dtype=np.float32) for s in shapes]


def matmul_shapes(kind, N, M, K):
    return {"AB": [(N, K), (K, M)], "T1": [(K, N), (K, M)], "T2": [(N, K), (M, K)]}[kind]


def bmm_shapes(kind, Batch, d0, d1, d2, d3):
    if kind == "AB":
        N, M, BK, AK = d0, d1, d2, d3
        return [(Batch, N, AK), (Batch, BK, M)], (Batch, N, M)
    if kind == "T1":
        CN, AN, M, K = d0, d1, d2, d3
        return [(Batch, K, AN), (Batch, K, M)], (Batch, CN, M)
    N, CM, BM, K = d0, d1, d2, d3
    return [(Batch, N, K), (Batch, BM, K)], (Batch, N, CM)


def conv_out(I, F, s, p):
    return (I + 2 * p - F) // s + 1


def _p(a):
    return a.ctypes.data_as(FP)


def main():
    from oracle import oracle as O
    mm, bm, cv = O.ref_native("matmul"), O.ref_native("bmm"), O.ref_native("conv")
    if mm is None or bm is None:
        raise SystemExit("oracle/_ref is not built: run `python oracle/build_ref.py` first")
    out = {}
    for name, (kind, N, M, K) in MATMUL_CASES.items():
        A, B = golden_inputs(name, matmul_shapes(kind, N, M, K))
        C = np.zeros((N, M), np.float32)
        {"AB": mm.ref_cpu_multiply, "T1": mm.ref_cpu_multiplyT1, "T2": mm.ref_cpu_multiplyT2}[kind](
            _p(A), _p(B), _p(C), N, M, K)
        out[name] = C
    for name, (kind, Batch, d0, d1, d2, d3) in BMM_CASES.items():
        shapes, cshape = bmm_shapes(kind, Batch, d0, d1, d2, d3)
        A, B = golden_inputs(name, shapes)
        C = np.zeros(cshape, np.float32)
        if kind == "AB":
            bm.ref_cpu_bmm(_p(A), _p(B), _p(C), Batch, d0, d1, d2, d3)
        elif kind == "T1":
            bm.ref_cpu_bmmT1(_p(A), _p(B), _p(C), Batch, d0, d1, d2, d3)
        else:
            bm.ref_cpu_bmmT2(_p(A), _p(B), _p(C), Batch, d0, d1, d2, d3)
        out[name] = C
    np.savez_compressed(HERE / "golden_matmul_bmm.npz", **out)
    print("wrote golden_matmul_bmm.npz:", len(out), "cases")
    if cv is None:
        print("libref_conv.so absent: conv fixtures not regenerated (python oracle/build_ref.py --conv)")
        return
    out = {}
    for name, (N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw) in CONV_CASES.items():
        X, W = golden_inputs(name, [(N, IH, IW, IC), (OC, FH, FW, IC)])
        OH, OW = conv_out(IH, FH, sh, ph), conv_out(IW, FW, sw, pw)
        Y1 = np.zeros((N, OH, OW, OC), np.float32)
        Y2 = np.zeros((N, OH, OW, OC), np.float32)
        cv.ref_cpu_conv3D_naive(_p(X), IH, IW, _p(W), FH, FW, _p(Y1), OH, OW, N, IC, OC, sh, sw, ph, pw)
        cv.ref_cpu_conv3D_img2col(_p(X), IH, IW, _p(W), FH, FW, _p(Y2), OH, OW, N, IC, OC, sh, sw, ph, pw)
        out[name + "/naive"] = Y1
        out[name + "/img2col"] = Y2
    np.savez_compressed(HERE / "golden_conv.npz", **out)
    print("wrote golden_conv.npz:", len(out), "arrays")
    make_deltax(O)


def make_deltax(O):
    """Stride-1 data gradient from the reference's deconv3D_deltaX_img2col_s1 (oracle/_ref/libref_deltax.so)."""
    dx = O.ref_native("deltax")
    if dx is None:
        print("libref_deltax.so absent: deltaX fixtures not regenerated (python oracle/build_ref.py --deltax)")
        return
    out = {}
    for name, (N, IH, IW, IC, OC, FH, FW, ph, pw) in DELTAX_CASES.items():
        OH, OW = IH + 2 * ph - FH + 1, IW + 2 * pw - FW + 1
        dY, W = golden_inputs(name, [(N, OH, OW, OC), (OC, FH, FW, IC)])
        dX = np.zeros((N, IH, IW, IC), np.float32)
        dx.ref_cpu_deconv3D_deltaX_img2col_s1(_p(dY), OH, OW, _p(W), FH, FW, _p(dX), IH, IW, N, IC, OC, ph, pw)
        out[name] = dX
    np.savez_compressed(HERE / "golden_deltax.npz", **out)
    print("wrote golden_deltax.npz:", len(out), "cases")
    if not hasattr(dx, "ref_cpu_deconv3D_deltaX_img2col"):
        print("libref_deltax.so lacks the any-stride routine: rebuild it (python oracle/build_ref.py --deltax --force)")
        return
    out = {}
    for name, (N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw) in DELTAX_STRIDED_CASES.items():
        OH, OW = (IH + 2 * ph - FH) // sh + 1, (IW + 2 * pw - FW) // sw + 1
        dY, W = golden_inputs(name, [(N, OH, OW, OC), (OC, FH, FW, IC)])
        dX = np.zeros((N, IH, IW, IC), np.float32)
        dx.ref_cpu_deconv3D_deltaX_img2col(_p(dY), OH, OW, _p(W), FH, FW, _p(dX), IH, IW, N, IC, OC, sh, sw, ph, pw)
        out[name] = dX
    np.savez_compressed(HERE / "golden_deltax_strided.npz", **out)
    print("wrote golden_deltax_strided.npz:", len(out), "cases")


if __name__ == "__main__":
    main()
