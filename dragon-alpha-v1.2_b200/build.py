"""Build recipe for libdragon_cu32.so (sm_100a only).

Compiles the CUDA translation units in parallel with nvcc and links them, together
with the JNI export shim, into one shared library placed next to this file.  nvcc
cross-compiles without a GPU, so this also serves as the "does it build" check.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OBJ = HERE / "build"
LIB = HERE / "libdragon_cu32.so"
BRIDGE_LIB = HERE / "libdragon_cuda.so"      # the Linux port of the reference's `Cuda` runtime-bridge natives
BRIDGE_SOURCE = "cuda_bridge.cu"

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
CUFLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]

CU_SOURCES = ["cu32_api.cu", "gemm_kk.cu", "gemm_kk_softmax.cu", "gemm_rep.cu", "gemm_kn.cu", "gemm_nn.cu", "gemm_nn_im2col.cu"]
CPP_SOURCES = ["jni_exports.cpp"]
HEADERS = ["sm100_ptx.cuh", "gemm_tf32.cuh", "gemm_launch.h", "jni_min.h", "../../include/dragon_cu32.h",
           "../../include/dragon_cuda.h"]


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps if d.exists())


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        raise RuntimeError(f"build step failed: {cmd[0]} ... {cmd[-1]}")


def build(force: bool = False, verbose: bool = False) -> Path:
    """Build (or reuse an up-to-date) libdragon_cu32.so and return its path."""
    OBJ.mkdir(exist_ok=True)
    hdrs = [CSRC / h for h in HEADERS] + [Path(__file__)]
    jobs = []
    objs = []
    for src in CU_SOURCES:
        o = OBJ / (src + ".o")
        objs.append(o)
        if force or _stale(o, [CSRC / src] + hdrs):
            extra = ["-Xptxas", "-v"] if verbose else []
            jobs.append([NVCC, *ARCH, *CUFLAGS, *extra, "-c", str(CSRC / src), "-o", str(o)])
    for src in CPP_SOURCES:
        o = OBJ / (src + ".o")
        objs.append(o)
        if force or _stale(o, [CSRC / src] + hdrs):
            jobs.append(["g++", "-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-c", str(CSRC / src), "-o", str(o)])
    bridge_obj = OBJ / (BRIDGE_SOURCE + ".o")
    if force or _stale(bridge_obj, [CSRC / BRIDGE_SOURCE] + hdrs):
        jobs.append([NVCC, *ARCH, *CUFLAGS, "-c", str(CSRC / BRIDGE_SOURCE), "-o", str(bridge_obj)])
    if jobs:
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as ex:
            list(ex.map(_run, jobs))
    if force or jobs or _stale(LIB, objs):
        _run([NVCC, *ARCH, "-shared", "-o", str(LIB), *map(str, objs), "-cudart", "shared"])
    if force or _stale(BRIDGE_LIB, [bridge_obj]):
        _run([NVCC, *ARCH, "-shared", "-o", str(BRIDGE_LIB), str(bridge_obj), "-cudart", "shared"])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
