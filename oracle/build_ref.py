"""Compile the reference's own sources for this path into oracle/_ref/ (test infrastructure).

What is built, from the read-only reference tree given by --reference (sources are compiled
where they lie; nothing is copied into this repository):

  libref_matmul.so   Cuda_matMul:      CPU check loops (test.cuh) + SIMT kernels/dispatchers
  libref_bmm.so      Cuda_batchMatMul: same
  libref_conv.so     Cuda_conv3D:      same (about 25 minutes; only with --conv)
  libref_deltax.so   Cuda_dconv3D_deltaX: CPU check loop + stride-1 dispatcher (long build; only with --deltax)
  libref_function.so Cuda_function:    linear_dual2D_row, the bias-row add that follows the
                                       contractions in matMul_biased / conv3D_biased (seconds)

The CPU loops pin oracle/cu32_oracle.c (tests/test_oracle.py compares them bit for bit) and
serve as the timed CPU baseline of the benchmark; the GPU dispatchers give the reference's
own FP32 output on the same inputs as a second witness.  The reference's Visual-Studio
build system is not used: each project is a single translation unit, compiled by one nvcc
command on a thin wrapper (ref_wrap_*.cu) that #includes the project's headers.
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")

PROJECTS = {
    "matmul": ("ref_wrap_matmul.cu", "Cuda_matMul/Cuda_matMul", "libref_matmul.so"),
    "bmm": ("ref_wrap_bmm.cu", "Cuda_batchMatMul/Cuda_batchMatMul", "libref_bmm.so"),
    "conv": ("ref_wrap_conv.cu", "Cuda_conv3D/Cuda_conv3D", "libref_conv.so"),
    "function": ("ref_wrap_function.cu", "Cuda_function/Cuda_function", "libref_function.so"),
    "reduce": ("ref_wrap_reduce.cu", "Cuda_reduce/Cuda_reduce", "libref_reduce.so"),
    "deltax": ("ref_wrap_deltax.cu", "Cuda_dconv3D_deltaX/Cuda_dconv3D_deltaX", "libref_deltax.so"),
}

# The conv project was written on a case-insensitive file system: these includes differ in
# case from the files on disk (conv3D.cuh:9, conv3D_tensor_remode.cuh:6-8).
CASE_FIX = {
    "conv3D_im2col_Winograd.cuh": "conv3D_Im2col_Winograd.cuh",
    "conv3D_kernel_remode_v1.cuh": "conv3D_kernel_remode_V1.cuh",
    "conv3D_kernel_remode_v2.cuh": "conv3D_kernel_remode_V2.cuh",
    "conv3D_kernel_remode_v3.cuh": "conv3D_kernel_remode_V3.cuh",
}


def auto_casefix(proj: Path, fix: Path) -> None:
    """The projects were written on a case-insensitive file system.  For every #include "name" in the
    project whose file does not exist under that spelling but does under another case, put an alias
    (symlink) with the spelled name into `fix`, which then goes on the include path."""
    import re
    fix.mkdir(parents=True, exist_ok=True)
    have = {f.name.lower(): f for f in proj.iterdir() if f.is_file()}
    for src in proj.iterdir():
        if src.suffix not in (".cuh", ".cu", ".h"):
            continue
        for name in re.findall(r'#include\s+"([^"]+)"', src.read_text(errors="ignore")):
            if (proj / name).exists() or "/" in name or "\\" in name:
                continue
            real = have.get(name.lower())
            if real is not None and not (fix / name).exists():
                (fix / name).symlink_to(real)


def build(reference: Path, names: list[str], force: bool = False) -> list[Path]:
    base = reference / "source" / "engine-cuda-base"
    if not base.is_dir():
        raise FileNotFoundError(f"{base} not found: the reference tree is needed to build oracle/_ref")
    OUT.mkdir(exist_ok=True)
    built = []
    for name in names:
        wrap, proj, lib = PROJECTS[name]
        out = OUT / lib
        if out.exists() and not force and out.stat().st_mtime > (HERE / wrap).stat().st_mtime:
            built.append(out)
            continue
        inc = ["-I", str(HERE / "jni_shim"), "-I", str(base / proj)]
        if name == "conv":
            fix = OUT / "casefix"
            fix.mkdir(exist_ok=True)
            for alias, real in CASE_FIX.items():
                link = fix / alias
                if not link.exists():
                    link.symlink_to(base / proj / real)
            inc += ["-I", str(fix)]
        if name == "deltax":
            fix = OUT / "casefix_deltax"
            auto_casefix(base / proj, fix)
            inc += ["-I", str(fix)]
        cmd = [NVCC, "-std=c++14", "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-shared",
               "-Xcompiler", "-fPIC", "-w", *inc, "-o", str(out), str(HERE / wrap)]
        print(" ".join(cmd), flush=True)
        subprocess.run(cmd, check=True)
        built.append(out)
    return built


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("DRAGON_REFERENCE_TREE"),
                    help="root of the reference tree (or set DRAGON_REFERENCE_TREE)")
    ap.add_argument("--conv", action="store_true", help="also build Cuda_conv3D (about 25 minutes)")
    ap.add_argument("--deltax", action="store_true", help="also build Cuda_dconv3D_deltaX (long)")
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    if not a.reference:
        ap.error("give --reference <tree> or set DRAGON_REFERENCE_TREE")
    names = ["matmul", "bmm", "function", "reduce"] + (["conv"] if a.conv else []) + (["deltax"] if a.deltax else [])
    for p in build(Path(a.reference), names, a.force):
        print(p)
