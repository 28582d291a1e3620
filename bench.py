#!/usr/bin/env python
"""Benchmark of the Cu32 dense-contraction hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" is one pass of the hot path over one batch of synthetic input: by default the
configuration the headline metric is quoted on, FP32-accurate matMul C = A*B at 8192^3
(uniform[-1,1] inputs from a fixed seed).  With N GPUs every rank runs that same step on its
own row block of an N-times-taller problem (rows of A and C sharded, B replicated): weak
scaling, no data-path collective.  Rank 0 prints ONE JSON line.

value      whole-job TFLOP/s (2*N*M*K per launch), inputs resident in HBM, timed with CUDA
           events on the launching stream, max over ranks
e2e        the same metric through the C-ABI call with HOST buffers: pinned host -> device
           copies of A and B and the device -> host read of C are inside the timed region
roofline   tensor bound: achieved FP32-accurate TFLOP/s against (measured bf16 peak / 2 for
           TF32 / 3 products per term); `traffic` is the ncu DRAM-bytes figure recorded in
           profiles/ for this kernel and workload (null until captured)
cpu_baseline  the reference's CPU check loop timed on the host cores on a bounded row sample
--impl reference   times that CPU loop alone (the reference has no other CPU implementation of
           this path), all host threads, on the same configuration

configs    (default run on one GPU) every other benchmark configuration timed the same way in the same run:
           ms, TFLOP/s, GB/s, roofline fraction and the tile the library chose
gpu_reference  the reference's own SIMT kernels (built from the reference tree into oracle/_ref) on the same
           8192^3 operands on this GPU, in the same run
clock      SM clock the kernels really ran at, from cycle and nanosecond counts taken inside the kernel, next to
           the management library's samples; cycles per k-block against the tensor pipe's 1536
sustained  the headline launched back to back for >= 2 s (power-capped clocks), against the sustained peak

With N > 1 GPUs `value` includes the reassembly of the output shards (NCCL all-gather over NVLink, issued per row
block so that it overlaps the next block's compute); `compute_only` is the figure without it, `strong` the
8192^3 problem itself split over the ranks.

Other workloads (for profiling and the reports in profiles/): c1, c2_bias, c2_t1, c2_t2, c2_ragged, c4_dx, dx_s2, c4_dw, c3_qk_scaled,
c3_qk, c3_pv, c3_sm, c3_attn, c4, c5.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "FP32-accurate matMul TFLOPS"
UNIT = "TFLOP/s"

# DRAM bytes per launch of the dominant kernel (dram__bytes_read.sum + dram__bytes_write.sum from
# one ncu capture of the same workload; the captures are summarised in profiles/).
NCU_TRAFFIC_BYTES = {
    "c2_ab": 2.54e9,     # profiles/gemm_tf32_matMul_AB_8192_traffic.md (same file for the two below)
    "c3_qk": 1.291e9,
    "c3_sm": 1.283e9,
}


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16": d["bf16_tflops"], "bf16_sustained": d["bf16_tflops_sustained"],
                "basis": "measured"}
    return {"hbm_gbs": 6650.0, "bf16": 1590.0, "bf16_sustained": 1400.0, "basis": "fallback"}


# ------------------------------------------------------------------ clocks
class ClockSampler:
    """SM clock and clock-event reasons sampled DURING the timed region (read-only queries).  NVML is
    polled from a thread every few milliseconds, so that even a 50 ms region gets a dozen samples; if the
    NVML bindings are missing, `nvidia-smi -lms` is the fallback (about one sample per 100 ms)."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int, uuid: str | None = None):
        self.proc = None
        self.thread = None
        self.samples = []          # (sm_mhz, reasons bitmask)
        self.max_mhz = None
        self._stop = threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            h = None
            if uuid:
                try:
                    h = pynvml.nvmlDeviceGetHandleByUUID(uuid if uuid.startswith("GPU-") else "GPU-" + uuid)
                except Exception:
                    h = None
            if h is None:
                h = pynvml.nvmlDeviceGetHandleByIndex(gpu_index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
            reasons_fn = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                pynvml.nvmlDeviceGetCurrentClocksThrottleReasons
            self._nvml = pynvml

            def poll():
                while not self._stop.is_set():
                    try:
                        self.samples.append((float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)),
                                             int(reasons_fn(h))))
                    except Exception:
                        pass
                    self._stop.wait(0.004)
            self.thread = threading.Thread(target=poll, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.thread = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        if self.thread is not None:
            self._stop.set()
            self.thread.join(timeout=2)
            nv = self._nvml
            bits = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}
            for n, const in (("hw_slowdown", "nvmlClocksEventReasonHwSlowdown"),
                             ("hw_thermal_slowdown", "nvmlClocksEventReasonHwThermalSlowdown"),
                             ("sw_thermal_slowdown", "nvmlClocksEventReasonSwThermalSlowdown"),
                             ("sw_power_cap", "nvmlClocksEventReasonSwPowerCap")):
                bits[n] = int(getattr(nv, const, bits[n]))
            sm = [x[0] for x in self.samples]
            seen = 0
            for _, r in self.samples:
                seen |= r
            return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": self.max_mhz,
                    "reasons": sorted(n for n in names if seen & bits[n]), "samples": len(sm), "source": "nvml"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        for line in out.strip().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "source": "nvidia-smi"}


# ------------------------------------------------------------------ CPU baseline (reference loops)
CPU_BLOCK_ROWS = 128   # output rows per host thread and pass: the same block in every CPU leg


def cpu_reference_loop(form: str, N: int, M: int, K: int, A, B, passes: int = 1):
    """Time the reference's CPU check loop (multiply*, Cuda_matMul/test.cuh:60-82) on a bounded
    sample: every host thread runs the loop `passes` times on its own block of CPU_BLOCK_ROWS output
    rows.  Returns (TFLOP/s, cores, kind, sample description)."""
    import numpy as np
    from oracle import oracle as O
    ref = O.ref_native("matmul")
    kind = "reference" if ref is not None else "port"
    cores = os.cpu_count() or 1
    fp = ctypes.POINTER(ctypes.c_float)
    names = {"AB": ("ref_cpu_multiply", "oracle_multiply"), "T1": ("ref_cpu_multiplyT1", "oracle_multiplyT1"),
             "T2": ("ref_cpu_multiplyT2", "oracle_multiplyT2")}[form]
    fn = getattr(ref, names[0]) if ref is not None else getattr(O.lib(), names[1])
    rows = max(4, min(CPU_BLOCK_ROWS, (N // cores) // 4 * 4))
    A = np.ascontiguousarray(A, dtype=np.float32)
    B = np.ascontiguousarray(B, dtype=np.float32)
    work = []
    for t in range(cores):
        r0 = (t * rows) % max(N - rows + 1, 1)
        if form == "T1":   # A is [K, N]: a row block of C needs a column block of A
            a = np.ascontiguousarray(A[:, r0:r0 + rows])
        else:
            a = np.ascontiguousarray(A[r0:r0 + rows])
        c = np.zeros((rows, M), np.float32)
        work.append((a, c))

    def run(a, c):
        for _ in range(passes):
            c[:] = 0
            fn(a.ctypes.data_as(fp), B.ctypes.data_as(fp), c.ctypes.data_as(fp), rows, M, K)
    threads = [threading.Thread(target=run, args=w) for w in work]
    t0 = time.perf_counter()
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    dt = time.perf_counter() - t0
    flops = 2.0 * rows * M * K * cores * passes
    return (flops / dt / 1e12, cores, kind,
            f"{cores} threads x {passes} pass(es) over {rows} output rows each of the {N}x{M}x{K} problem ({dt:.1f} s)")


# ------------------------------------------------------------------ workloads on the device
class Workload:
    """Builds device operands and returns `launch()` (enqueue one step on the current stream),
    flops and algorithmic bytes per launch, plus host buffers for the end-to-end leg."""

    def __init__(self, name, pkg, torch, rank, size=8192, batch=1024, images=256, light=False):
        self.name, self.pkg, self.torch = name, pkg, torch
        self.light = light          # no end-to-end leg: the host copies need not be pinned
        pin = (lambda t: t) if light else (lambda t: t.pin_memory())
        W = pkg.workloads
        mm, bm, cv = pkg.cu32.Cuda_matMul, pkg.cu32.Cuda_batchMatMul, pkg.cu32.Cuda_conv3D
        st = lambda: [torch.cuda.current_stream().cuda_stream]
        self.kernels_per_step = 1
        self.cpu_case = None
        if name in ("c1", "c2_ab", "c2_bias", "c2_t1", "c2_t2", "c2_ragged", "c5"):
            if name == "c1":
                w = W.config1()
            elif name == "c2_ragged":
                w = W.config2_ragged("AB")
            elif name == "c5":
                w = W.config5(K=1048576 // 8)   # one GPU's K shard of the 8-GPU configuration
            else:
                w = W.config2({"c2_ab": "AB", "c2_bias": "AB", "c2_t1": "T1", "c2_t2": "T2"}[name], size)
            self.hosts = [pin(w.A), pin(w.B)]
            self.dev_in = [torch.empty_like(h, device="cuda") for h in self.hosts]
            for d, h in zip(self.dev_in, self.hosts):
                d.copy_(h)
            self.out = torch.empty((w.N, w.M), device="cuda")
            fn = {"AB": mm.matMul, "T1": mm.matMulT1, "T2": mm.matMulT2}[w.form]
            dA, dB, dC = self.dev_in[0], self.dev_in[1], self.out
            if name == "c5":
                gz = pkg.engine.matMulT1_gridZ(w.N, w.M, w.K, 148)
                self.gz = gz
                self.cbuf = torch.empty((gz - 1) * w.N * w.M, device="cuda")
                self.kernels_per_step = 2

                def launch():
                    s = st()
                    mm.matMulT1SK(s, 1, gz, dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), self.cbuf.data_ptr(), w.N, w.M, w.K)
                    mm.SKbuf_summary(s[0], self.cbuf.data_ptr(), dC.data_ptr(), gz - 1, w.N * w.M)
                self.launch = launch
            elif name == "c2_bias":
                # the engine's matMul_biased as one kernel: product, bias row and padding zeroing
                g = torch.Generator().manual_seed(2002)
                self.bias = torch.randn(w.M, generator=g).cuda()
                self.launch = lambda: mm.matMul_biased(st(), 1, dA.data_ptr(), dB.data_ptr(), dC.data_ptr(),
                                                       self.bias.data_ptr(), w.N, w.M, w.K, w.M)
            else:
                self.launch = lambda: fn(st(), 1, dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), w.N, w.M, w.K)
            lg = getattr(w, "logical", (w.N, w.M, w.K))
            self.flops = 2.0 * lg[0] * lg[1] * lg[2]
            self.bytes = 4.0 * (lg[0] * lg[2] + lg[2] * lg[1] + lg[0] * lg[1])
            self.desc = f"matMul {w.form} N={w.N} M={w.M} K={w.K}"
            self.cpu_case = (w.form, w.N, w.M, w.K, w.A, w.B)
            self.units = None
        elif name in ("c3_qk", "c3_qk_scaled", "c3_pv"):
            w = W.config3(Batch=batch)
            self.attn = (w.Batch, w.L, w.D)
            if name in ("c3_qk", "c3_qk_scaled"):
                self.hosts = [pin(w.Q), pin(w.K)]
                self.dev_in = [h.cuda() for h in self.hosts]
                self.out = torch.empty((w.Batch, w.L, w.L), device="cuda")
                dA, dB, dC = self.dev_in[0], self.dev_in[1], self.out
                self.launch = lambda: bm.batchMatMulT2(st(), 1, dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), w.Batch, w.L, w.L, w.L, w.D)
                self.desc = f"batchMatMulT2 Q*K^T Batch={w.Batch} {w.L}x{w.L}x{w.D}"
                if name == "c3_qk_scaled":   # the attention block's 1/sqrt(d) scale fused into the store
                    alpha = 1.0 / (w.D ** 0.5)
                    self.launch = lambda: bm.batchMatMulT2_scaled(st(), 1, dA.data_ptr(), dB.data_ptr(), dC.data_ptr(),
                                                                  w.Batch, w.L, w.L, w.L, w.D, alpha)
                    self.desc = f"batchMatMulT2_scaled Q*K^T/sqrt(d) Batch={w.Batch} {w.L}x{w.L}x{w.D}"
            else:
                if light:   # softmax-normalised rows made on the device
                    g = torch.Generator(device="cuda").manual_seed(3003)
                    P = torch.softmax(torch.randn((w.Batch, w.L, w.L), generator=g, device="cuda"), dim=-1)
                    self.hosts = [None, w.V]
                    self.dev_in = [P, w.V.cuda()]
                else:
                    g = torch.Generator().manual_seed(3003)
                    P = torch.softmax(torch.randn((w.Batch, w.L, w.L), generator=g), dim=-1)
                    self.hosts = [P.pin_memory(), w.V.pin_memory()]
                    self.dev_in = [h.cuda() for h in self.hosts]
                self.out = torch.empty((w.Batch, w.L, w.D), device="cuda")
                dA, dB, dC = self.dev_in[0], self.dev_in[1], self.out
                self.launch = lambda: bm.batchMatMul(st(), 1, dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), w.Batch, w.L, w.D, w.L, w.L)
                self.desc = f"batchMatMul P*V Batch={w.Batch} {w.L}x{w.D}x{w.L}"
            self.flops = w.flops_each
            self.bytes = w.algorithmic_bytes_each
        elif name in ("c3_sm", "c3_attn"):
            # the attention block's scores in one pass - P = softmax(Q K^T / sqrt(d)) - and, for c3_attn, O = P V after it
            w = W.config3(Batch=batch)
            self.attn = (w.Batch, w.L, w.D)
            self.hosts = [pin(w.Q), pin(w.K), pin(w.V)]
            self.dev_in = [h.cuda() for h in (w.Q, w.K, w.V)]
            self.P = torch.empty((w.Batch, w.L, w.L), device="cuda")
            dQ, dK, dV, dP = self.dev_in[0], self.dev_in[1], self.dev_in[2], self.P
            alpha = 1.0 / (w.D ** 0.5)
            score_bytes = 4.0 * w.Batch * w.L * w.L
            qkv_bytes = 4.0 * w.Batch * w.L * w.D
            if name == "c3_sm":
                self.out = self.P
                self.launch = lambda: bm.batchMatMulT2_softmax(st(), 1, dQ.data_ptr(), dK.data_ptr(), dP.data_ptr(), w.Batch,
                                                                w.L, w.L, w.L, w.D, alpha)
                self.flops = w.flops_each
                self.bytes = 2 * qkv_bytes + score_bytes
                self.desc = f"batchMatMulT2_softmax P=softmax(Q*K^T/sqrt(d)) Batch={w.Batch} {w.L}x{w.L}x{w.D}"
            else:
                self.out = torch.empty((w.Batch, w.L, w.D), device="cuda")
                dO = self.out
                self.kernels_per_step = 2

                def launch():
                    s = st()
                    bm.batchMatMulT2_softmax(s, 1, dQ.data_ptr(), dK.data_ptr(), dP.data_ptr(), w.Batch, w.L, w.L, w.L, w.D, alpha)
                    bm.batchMatMul(s, 1, dP.data_ptr(), dV.data_ptr(), dO.data_ptr(), w.Batch, w.L, w.D, w.L, w.L)
                self.launch = launch
                self.flops = 2 * w.flops_each
                self.bytes = 4 * qkv_bytes + 2 * score_bytes
                # the reference's block moves the score tensor nine times (product w, scale r+w, row_max r,
                # row_softmax r+w, div2D_field r+w, P*V r), this one twice
                self.reference_sequence_bytes = 4 * qkv_bytes + 9 * score_bytes
                self.desc = (f"attention block Batch={w.Batch} L={w.L} d={w.D}: batchMatMulT2_softmax + batchMatMul "
                             f"(score tensor written once, read once)")
        elif name == "c4":
            w = W.config4(N=images)
            d = w.dims
            self.hosts = [pin(w.X), pin(w.W)]
            self.dev_in = [h.cuda() for h in self.hosts]
            self.out = torch.empty((d["N"], d["OH"], d["OW"], d["OC"]), device="cuda")
            self.cw = torch.empty(w.W.numel(), device="cuda")
            self.conv = dict(d, sh=w.sh, sw=w.sw, ph=w.ph, pw=w.pw)
            dX, dW, dY = self.dev_in[0], self.dev_in[1], self.out
            self.kernels_per_step = 2

            def launch():
                s = st()
                cv.kernel_remode(s[0], dW.data_ptr(), self.cw.data_ptr(), d["FH"], d["FW"], d["OC"], d["IC"])
                cv.conv3D_GemmR(s, 1, dX.data_ptr(), d["IH"], d["IW"], dW.data_ptr(), self.cw.data_ptr(), d["FH"], d["FW"],
                                dY.data_ptr(), d["OH"], d["OW"], d["N"], d["IC"], d["OC"], w.sh, w.sw, w.ph, w.pw)
            self.launch = launch
            self.flops = w.flops
            self.bytes = w.algorithmic_bytes
            self.desc = f"conv3D_GemmR N={d['N']} {d['IH']}x{d['IW']}x{d['IC']} -> {d['OC']}, 3x3 s1 p1 (remode + GEMM)"
            self.images = d["N"]
        elif name == "c4_dx":
            # data gradient of config 4 (stride 1): same sizes and FLOPs, deltaY in, deltaX out, W read in place
            w = W.config4(N=images)
            d = w.dims
            g = torch.Generator().manual_seed(4004)
            dYh = torch.randn((d["N"], d["OH"], d["OW"], d["OC"]), generator=g)
            self.hosts = [pin(dYh), pin(w.W)]
            self.dev_in = [h.cuda() for h in self.hosts]
            self.out = torch.empty((d["N"], d["IH"], d["IW"], d["IC"]), device="cuda")
            ddY, dW, dDX = self.dev_in[0], self.dev_in[1], self.out
            dx = pkg.cu32.Cuda_dconv3D_deltaX
            self.launch = lambda: dx.dconv3D_deltaX_s1(st(), 1, ddY.data_ptr(), d["OH"], d["OW"], dW.data_ptr(), d["FH"],
                                                       d["FW"], dDX.data_ptr(), d["IH"], d["IW"], d["N"], d["IC"], d["OC"],
                                                       w.ph, w.pw)
            self.flops = w.flops
            self.bytes = w.algorithmic_bytes
            self.desc = f"dconv3D_deltaX_s1 N={d['N']} {d['OH']}x{d['OW']}x{d['OC']} -> {d['IC']}, 3x3 s1 p1"
            self.images = d["N"]
        elif name == "dx_s2":
            # data gradient of a residual network's down-sampling convolution, as the engine runs it for strides > 1:
            # ks_remodev2 (filter -> kernel-split workspace) + the Ims2R native.  Synthetic, seeded.
            N_, IH, IC, OC, F, sd, pd = images, 56, 128, 256, 3, 2, 1
            OH = (IH + 2 * pd - F) // sd + 1
            g = torch.Generator().manual_seed(4005)
            dYh = torch.randn((N_, OH, OH, OC), generator=g)
            Wh = torch.randn((OC, F, F, IC), generator=g) * 0.03
            self.hosts = [pin(dYh), pin(Wh)]
            self.dev_in = [h.cuda() for h in self.hosts]
            self.out = torch.empty((N_, IH, IH, IC), device="cuda")
            CF = (F + sd - 1) // sd
            self.cw = torch.zeros(sd * sd * OC * CF * CF * IC, device="cuda")
            ddY, dW, dDX = self.dev_in[0], self.dev_in[1], self.out
            dx = pkg.cu32.Cuda_dconv3D_deltaX
            # the filter rearrangement plus the gradient: its sd*sd phases run in one launch when there are at most four
            self.kernels_per_step = 1 + (1 if sd * sd <= 4 and pkg.cu32.get_tune("phase_fused") else sd * sd)

            def launch():
                s = st()
                dx.ks_remodev2(s[0], dW.data_ptr(), F, F, self.cw.data_ptr(), CF, CF, OC, IC, sd, sd)
                dx.dconv3D_deltaX_ksIms2R(s, 1, ddY.data_ptr(), OH, OH, self.cw.data_ptr(), F, F, dDX.data_ptr(), IH, IH,
                                          N_, IC, OC, pd, pd)
            self.launch = launch
            self.flops = 2.0 * N_ * OH * OH * OC * F * F * IC
            self.bytes = 4.0 * (dYh.numel() + Wh.numel() + self.out.numel())
            self.desc = f"ks_remodev2 + dconv3D_deltaX_ksIms2R N={N_} {OH}x{OH}x{OC} -> {IH}x{IH}x{IC}, 3x3 s2 p1"
            self.images = N_
        elif name == "c4_dw":
            # weight gradient of config 4: deltaW[256,3,3,256] from X and deltaY, split over the pixel axis
            w = W.config4(N=images)
            d = w.dims
            g = torch.Generator().manual_seed(4006)
            dYh = torch.randn((d["N"], d["OH"], d["OW"], d["OC"]), generator=g)
            self.hosts = [pin(w.X), pin(dYh)]
            self.dev_in = [h.cuda() for h in self.hosts]
            size = d["OC"] * d["FH"] * d["FW"] * d["IC"]
            self.out = torch.empty((d["OC"], d["FH"], d["FW"], d["IC"]), device="cuda")
            gz = int(os.environ.get("DRAGON_BENCH_DW_GRIDZ", "8"))
            self.cbuf = torch.empty(max(gz - 1, 1) * size, device="cuda")
            dX, ddY, dDW = self.dev_in[0], self.dev_in[1], self.out
            dwc = pkg.cu32.Cuda_dconv3D_deltaW
            self.kernels_per_step = 2 if gz > 1 else 1

            def launch():
                s = st()
                dwc.dconv3D_deltaW_GemmSK(s, 1, gz, dX.data_ptr(), d["IH"], d["IW"], ddY.data_ptr(), d["OH"], d["OW"],
                                          dDW.data_ptr(), self.cbuf.data_ptr(), d["FH"], d["FW"], d["N"], d["IC"], d["OC"],
                                          w.sh, w.sw, w.ph, w.pw)
                if gz > 1:
                    dwc.buf_summary(s[0], self.cbuf.data_ptr(), dDW.data_ptr(), gz - 1, size)
            self.launch = launch
            self.flops = w.flops
            self.bytes = 4.0 * (w.X.numel() + dYh.numel() + size)
            self.desc = (f"dconv3D_deltaW_GemmSK GridZ={gz} + buf_summary N={d['N']} {d['IH']}x{d['IW']}x{d['IC']}, "
                         f"deltaY {d['OC']} channels, 3x3 s1 p1")
            self.images = d["N"]
        else:
            raise SystemExit(f"unknown workload {name}")

    def e2e_step(self):
        """Host -> device copies of the inputs, the contraction, device -> host read of the result.
        For the row-shardable matMul forms the three are pipelined over row blocks of A and C on
        three streams (copy-in, compute, copy-out): B goes first, then block i is multiplied while
        block i+1 arrives and block i-1 leaves - what a host that owns the buffers would do."""
        torch = self.torch
        if getattr(self, "row_blocks", None) is None:
            for d, h in zip(self.dev_in, self.hosts):
                d.copy_(h, non_blocking=True)
            self.launch()
            self.host_out.copy_(self.out, non_blocking=True)
            return
        cur = torch.cuda.current_stream()
        s_in, s_out = self.s_in, self.s_out
        s_in.wait_stream(cur)
        s_out.wait_stream(cur)
        form, N, M, K = self.row_blocks
        mm = self.pkg.cu32.Cuda_matMul
        fn = mm.matMul if form == "AB" else mm.matMulT2
        dA, dB, dC = self.dev_in[0], self.dev_in[1], self.out
        hA, hB = self.hosts
        with torch.cuda.stream(s_in):
            dB.copy_(hB, non_blocking=True)
        nblk = self.nblk
        rows = N // nblk
        for b in range(nblk):
            r0, r1 = b * rows, (b + 1) * rows if b + 1 < nblk else N
            with torch.cuda.stream(s_in):
                dA[r0:r1].copy_(hA[r0:r1], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(s_in)
            cur.wait_event(ev)
            fn([cur.cuda_stream], 1, dA[r0:r1].data_ptr(), dB.data_ptr(), dC[r0:r1].data_ptr(), r1 - r0, M, K)
            ev2 = torch.cuda.Event()
            ev2.record(cur)
            s_out.wait_event(ev2)
            with torch.cuda.stream(s_out):
                self.host_out[r0:r1].copy_(dC[r0:r1], non_blocking=True)
        cur.wait_stream(s_out)

    def prepare_e2e(self):
        self.host_out = self.torch.empty(self.out.shape, dtype=self.out.dtype).pin_memory()
        c = self.cpu_case
        if c is not None and c[0] in ("AB", "T2") and c[1] >= 2048 and self.kernels_per_step == 1:
            self.row_blocks = (c[0], c[1], c[2], c[3])
            self.nblk = int(os.environ.get("DRAGON_BENCH_E2E_BLOCKS", "32"))   # row blocks of the copy/compute/copy pipeline
            self.s_in, self.s_out = self.torch.cuda.Stream(), self.torch.cuda.Stream()
        self.h2d = sum(h.numel() * 4 for h in self.hosts)
        self.d2h = self.out.numel() * 4


def time_steps(torch, dist, fn, steps, world, on_start=None, on_stop=None):
    """barrier + sync, `steps` launches bracketed by CUDA events on the current stream, sync +
    barrier; returns the max over ranks of the elapsed milliseconds.  `on_start` / `on_stop` run
    right around the timed launches (after the opening barrier, before the closing one) - the
    clock sampler hooks in there so that it sees the GPU under load only."""
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    if on_start:
        on_start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    if on_stop:
        on_stop()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        dist.barrier()
    return ms


TILE_NAMES = {0: "128x64", 1: "128x128", 2: "128x256", 3: "256x128 pair", 4: "256x256 pair", 5: "256x64 pair"}
HBM_BOUND = ("c3_qk", "c3_qk_scaled", "c3_pv", "c3_sm", "c3_attn")


def roofline_of(name, wl, ms_step, pk, sustained=False, traffic=None):
    """Roofline object for one launch: tensor bound (FP32-accurate = three TF32 products per term, TF32 at half
    the bf16 rate) or HBM bound for the attention-shaped batched products."""
    per_gpu = wl.flops / (ms_step * 1e-3) / 1e12
    if name in HBM_BOUND:
        gbs = wl.bytes / (ms_step * 1e-3) / 1e9
        return {"bound": "hbm", "achieved": gbs, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": gbs / pk["hbm_gbs"],
                "traffic": traffic, "peak_basis": f"{pk['basis']} copy bandwidth"}
    bf16 = pk["bf16_sustained"] if sustained else pk["bf16"]
    ceiling = bf16 / 2.0 / 3.0
    return {"bound": "tensor", "achieved": per_gpu, "peak": ceiling, "unit": "TFLOP/s", "frac": per_gpu / ceiling,
            "traffic": traffic,
            "peak_basis": f"{pk['basis']} bf16 {'sustained' if sustained else 'burst'} {bf16} TFLOP/s / 2 (TF32 rate) / 3 (hi*hi + hi*lo + lo*hi)"}


def check_status(pkg):
    st = pkg.cu32.read_status()
    if st != 0:
        raise SystemExit("kernel gave up: " + pkg.cu32.decode_status(st))


def device_clock(pkg):
    """Effective SM clock in MHz over the contraction launches since the last read (cycles and nanoseconds are
    counted inside the kernel by CTA 0), or None if nothing ran."""
    cyc, ns, launches = pkg.cu32.read_clock()
    return {"effective_sm_mhz": cyc / ns * 1e3 if ns else None, "kernel_cycles": cyc, "kernel_ns": ns, "launches": launches}


def other_configs(pkg, torch, pk, names, steps, warmup):
    """Every other benchmark configuration, timed like the headline (CUDA events on the launching stream, inputs
    resident, operands larger than L2 except config 1), one after the other on this GPU; where oracle/_ref holds the
    reference's own kernels for the configuration, those are timed on the same operands right after
    (`gpu_reference_ms`, `gpu_reference_ratio`)."""
    out = {}
    for name in names:
        wl = Workload(name, pkg, torch, 0, light=True)
        for _ in range(warmup):
            wl.launch()
        check_status(pkg)
        ms, clk = None, None
        for _ in range(2):   # the better of two averages over `steps` launches: these launches are short, and a
            pkg.cu32.read_clock()   # transient (an allocation being released, a clock step) can double one window
            t = time_steps(torch, None, wl.launch, steps, 1) / steps
            c = device_clock(pkg)
            if ms is None or t < ms:
                ms, clk = t, c
        check_status(pkg)
        roof = roofline_of(name, wl, ms, pk)
        tile = pkg.cu32.get_tune("last_tile")
        entry = {"workload": wl.desc, "ms_per_step": ms, "tflops": wl.flops / (ms * 1e-3) / 1e12,
                 "gbs": wl.bytes / (ms * 1e-3) / 1e9, "bound": roof["bound"], "frac": roof["frac"],
                 "peak": roof["peak"], "unit": roof["unit"], "tile": TILE_NAMES.get(tile, tile),
                 "launches_per_step": wl.kernels_per_step, "effective_sm_mhz": clk["effective_sm_mhz"],
                 "l2": "operands larger than L2" if wl.bytes > 126e6 else "operands fit in L2 (not flushed)"}
        if hasattr(wl, "images"):
            entry["images_per_s"] = wl.images / (ms * 1e-3)
        if hasattr(wl, "reference_sequence_bytes"):
            entry["algorithmic_bytes"] = wl.bytes
            entry["reference_sequence_bytes"] = wl.reference_sequence_bytes
        try:
            ref_ms = gpu_reference_config(torch, name, wl)
        except Exception:   # a reference library built from another tree: leave the comparison out
            ref_ms = None
        if ref_ms:
            entry["gpu_reference_ms"] = ref_ms
            entry["gpu_reference_ratio"] = ref_ms / ms
        out[name] = entry
        del wl
        torch.cuda.empty_cache()
    return out


def gpu_reference_config(torch, name, wl):
    """The reference's own kernels for one of the other configurations (compiled for sm_100a from the reference
    tree into oracle/_ref), on the device operands of `wl`, into a scratch output: best of 3 launches, CUDA events.
    Returns milliseconds, or None where the reference library is not built or has no kernel for the configuration.
    The attention block is the engine's sequence: product, scale (linear2D), row_max, row_softmax, div2D_field, P*V."""
    from oracle import oracle as O
    fp = ctypes.POINTER(ctypes.c_float)
    ptr = lambda t: ctypes.cast(ctypes.c_void_p(t.data_ptr()), fp)
    s0 = torch.cuda.current_stream().cuda_stream
    streams = (ctypes.c_longlong * 10)(*([s0] * 10))
    st = ctypes.c_longlong(s0)
    f32 = ctypes.c_float
    keep = []
    if name in ("c2_t1", "c2_t2", "c2_ragged", "c2_ab", "c1") and wl.cpu_case is not None:
        ref = O.ref_native("matmul")
        if ref is None:
            return None
        form, N, M, K = wl.cpu_case[:4]
        fn = {"AB": ref.ref_gpu_matMul, "T1": ref.ref_gpu_matMulT1, "T2": ref.ref_gpu_matMulT2}[form]
        C = torch.zeros((N, M), device="cuda")
        run = lambda: fn(streams, 10, ptr(wl.dev_in[0]), ptr(wl.dev_in[1]), ptr(C), N, M, K)
    elif name == "c5":
        ref = O.ref_native("matmul")
        if ref is None or not hasattr(ref, "ref_gpu_matMulT1SK"):
            return None
        _, N, M, K = wl.cpu_case[:4]
        C = torch.zeros((N, M), device="cuda")
        Cbuf = torch.zeros_like(wl.cbuf)

        def run():
            rc = ref.ref_gpu_matMulT1SK(streams, 10, wl.gz, ptr(wl.dev_in[0]), ptr(wl.dev_in[1]), ptr(C), ptr(Cbuf), N, M, K)
            return rc or ref.ref_gpu_SKbuf_summary(st, ptr(Cbuf), ptr(C), wl.gz - 1, N * M)
    elif name in ("c3_qk", "c3_pv"):
        ref = O.ref_native("bmm")
        if ref is None:
            return None
        Batch, L, D = wl.attn
        C = torch.zeros_like(wl.out)
        if name == "c3_qk":
            run = lambda: ref.ref_gpu_batchMatMulT2(streams, 10, ptr(wl.dev_in[0]), ptr(wl.dev_in[1]), ptr(C), Batch, L, L, L, D)
        else:
            run = lambda: ref.ref_gpu_batchMatMul(streams, 10, ptr(wl.dev_in[0]), ptr(wl.dev_in[1]), ptr(C), Batch, L, D, L, L)
    elif name == "c3_attn":
        ref, red, fun = O.ref_native("bmm"), O.ref_native("reduce"), O.ref_native("function")
        if ref is None or red is None or fun is None or not hasattr(fun, "ref_gpu_div2D_field"):
            return None
        Batch, L, D = wl.attn
        rows = Batch * L
        S = torch.empty((Batch, L, L), device="cuda")
        X = torch.empty_like(S)
        Y = torch.empty_like(S)
        Oo = torch.zeros_like(wl.out)
        V = torch.zeros(max(L >> 8, 1) * ((rows + 3) // 4 * 4) + 16, device="cuda")
        mx = torch.zeros(rows + 16, device="cuda")
        alpha = 1.0 / (D ** 0.5)
        dQ, dK, dV = wl.dev_in[0], wl.dev_in[1], wl.dev_in[2]

        def run():
            rc = ref.ref_gpu_batchMatMulT2(streams, 10, ptr(dQ), ptr(dK), ptr(S), Batch, L, L, L, D)
            rc = rc or fun.ref_gpu_linear2D(st, f32(alpha), ptr(S), f32(0.0), ptr(X), rows * L, L, L)
            rc = rc or red.ref_gpu_row_max(st, ptr(X), rows, L, ptr(V), ptr(mx), L, L)
            rc = rc or red.ref_gpu_row_softmax(st, ptr(X), ptr(mx), ptr(Y), rows, L, ptr(V), L, L)
            rc = rc or fun.ref_gpu_div2D_field(st, f32(1.0), ptr(Y), f32(0.0), f32(1.0), ptr(V), f32(0.0), f32(0.0), L,
                                               ptr(Y), rows * L, L, L)
            return rc or ref.ref_gpu_batchMatMul(streams, 10, ptr(Y), ptr(dV), ptr(Oo), Batch, L, D, L, L)
    elif name == "c4":
        ref = O.ref_native("conv")
        if ref is None:
            return None
        d = wl.conv
        Yr = torch.zeros_like(wl.out)
        CW = torch.empty_like(wl.cw)
        dX, dW = wl.dev_in[0], wl.dev_in[1]

        def run():
            rc = ref.ref_gpu_kernel_remode(st, ptr(dW), ptr(CW), d["FH"], d["FW"], d["OC"], d["IC"])
            return rc or ref.ref_gpu_conv3D_GemmR(streams, 10, ptr(dX), d["IH"], d["IW"], ptr(dW), ptr(CW), d["FH"], d["FW"],
                                                  ptr(Yr), d["OH"], d["OW"], d["N"], d["IC"], d["OC"], d["sh"], d["sw"],
                                                  d["ph"], d["pw"])
    else:
        return None
    if run() != 0:
        return None
    torch.cuda.synchronize()
    best = None
    for _ in range(3):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        rc = run()
        e1.record()
        torch.cuda.synchronize()
        if rc != 0:
            return None
        t = e0.elapsed_time(e1)
        best = t if best is None else min(best, t)
    return best


def gpu_reference_leg(torch, wl):
    """The reference's own SIMT FP32 kernels (matMul4x, Cuda_matMul/matMul.cuh:47-119, compiled for sm_100a from the
    reference tree into oracle/_ref) on the same device operands: best of 5 launches, CUDA events."""
    from oracle import oracle as O
    ref = O.ref_native("matmul")
    if ref is None or wl.cpu_case is None:
        return None
    form, N, M, K = wl.cpu_case[:4]
    fn = {"AB": ref.ref_gpu_matMul, "T1": ref.ref_gpu_matMulT1, "T2": ref.ref_gpu_matMulT2}[form]
    fp = ctypes.POINTER(ctypes.c_float)
    ptr = lambda t: ctypes.cast(ctypes.c_void_p(t.data_ptr()), fp)
    streams = (ctypes.c_longlong * 10)(*([torch.cuda.current_stream().cuda_stream] * 10))
    C = torch.zeros((N, M), device="cuda")
    run = lambda: fn(streams, 10, ptr(wl.dev_in[0]), ptr(wl.dev_in[1]), ptr(C), N, M, K)
    for _ in range(2):
        if run() != 0:
            return None
    torch.cuda.synchronize()
    best = None
    for _ in range(5):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); run(); e1.record()
        torch.cuda.synchronize()
        t = e0.elapsed_time(e1)
        best = t if best is None else min(best, t)
    return {"value": wl.flops / (best * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": best,
            "kind": "the reference's SIMT FP32 kernels built for sm_100a (oracle/_ref/libref_matmul.so), same operands"}


class FusedGatherStep:
    """One multi-GPU step of a row-shardable matMul with the reassembly inside the kernel: the epilogue stores each
    tile of this rank's rows into its own copy of the full output and into every peer's copy (peer memory mapped into
    this process), so no collective follows the launch and nothing is loaded over NVLink."""

    def __init__(self, torch, dist, pkg, wl, world, rank):
        form, N, M, K = wl.cpu_case[:4]
        assert form in ("AB", "T2")
        self.torch, self.wl = torch, wl
        mm = pkg.cu32.Cuda_matMul
        self.fn = mm.matMul_replicated if form == "AB" else mm.matMulT2_replicated
        self.N, self.M, self.K = N, M, K
        self.pg = pkg.shard.PeerGather(dist, world, rank, (N, M), torch.device("cuda", torch.cuda.current_device()))
        self.bytes_sent = (world - 1) * N * M * 4

    def __call__(self):
        wl, pg = self.wl, self.pg
        cur = self.torch.cuda.current_stream()
        self.fn([cur.cuda_stream], 1, wl.dev_in[0].data_ptr(), wl.dev_in[1].data_ptr(), pg.local.data_ptr(), pg.replicas,
                self.N, self.M, self.K)

    def check(self):
        """Every rank multiplies the same seeded operands here, so every block of the gathered output must equal
        this rank's own block bit for bit once all ranks have finished."""
        pg = self.pg
        pg.barrier()
        ok = all(bool(self.torch.equal(pg.block(r), pg.local)) for r in range(pg.world))
        pg.barrier()
        return ok


class ShardedStep:
    """One multi-GPU step of a row-shardable matMul: this rank's rows are cut into blocks; block b is multiplied
    on the current stream and then all-gathered (NCCL over NVLink, its own stream) while block b+1 is being
    multiplied.  Block b of every rank lands side by side in `gathered[b]`, i.e. the rows of the full output
    are dealt to the ranks block-cyclically and the reassembled output is in row order."""

    def __init__(self, torch, dist, pkg, wl, world, nblk):
        form, N, M, K = wl.cpu_case[:4]
        assert form in ("AB", "T2")
        self.torch, self.dist, self.wl = torch, dist, wl
        mm = pkg.cu32.Cuda_matMul
        self.fn = mm.matMul if form == "AB" else mm.matMulT2
        self.N, self.M, self.K, self.nblk = N, M, K, nblk
        self.rows = N // nblk
        self.gathered = torch.empty((nblk, world, self.rows * M), device="cuda")
        self.bytes_received = (world - 1) * N * M * 4

    def __call__(self):
        torch, dist, wl = self.torch, self.dist, self.wl
        dA, dB, dC = wl.dev_in[0], wl.dev_in[1], wl.out
        cur = torch.cuda.current_stream()
        works = []
        for b in range(self.nblk):
            r0, r1 = b * self.rows, (b + 1) * self.rows
            self.fn([cur.cuda_stream], 1, dA[r0:r1].data_ptr(), dB.data_ptr(), dC[r0:r1].data_ptr(), r1 - r0, self.M, self.K)
            works.append(dist.all_gather_into_tensor(self.gathered[b].view(-1), dC[r0:r1].reshape(-1), async_op=True))
        for w in works:
            w.wait()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2_ab")
    ap.add_argument("--size", type=int, default=8192, help="edge of the c2_* cubes (profiling on a smaller case)")
    ap.add_argument("--batch", type=int, default=1024, help="batch of the c3_* workloads (smaller for profiling)")
    ap.add_argument("--images", type=int, default=256, help="images of the c4 workload (smaller for profiling)")
    ap.add_argument("--tune", action="append", default=[], metavar="KEY=VALUE",
                    help="cu32_tune setting applied before anything runs (diagnostics), e.g. rep_lazy=0")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the other configurations, the reference-kernel leg and the sustained leg (profiling runs)")
    a = ap.parse_args()
    a.warmup = max(a.warmup, 3)
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:   # peer-mapped output copies use plain mappings, never an NVLink multicast object
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")

    import __graft_entry__ as entry
    pkg = entry.load_package()

    if a.impl == "reference":
        # The reference's own CPU implementation of this path: its check loops, all host threads.
        if rank != 0:
            return
        w = pkg.workloads.config2("AB")
        vals, cores, kind, sample = [], 1, "port", ""
        for i in range(a.warmup + a.steps):
            v, cores, kind, sample = cpu_reference_loop("AB", w.N, w.M, w.K, w.A.numpy(), w.B.numpy())
            if i >= a.warmup:
                vals.append(v)
        v = statistics.mean(vals)
        flops = 2.0 * w.N * w.M * w.K
        print(json.dumps({
            "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": a.gpus, "steps": a.steps,
            "warmup": a.warmup, "ms_per_step": flops / (v * 1e12) * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "matMul AB N=8192 M=8192 K=8192 (config 2); each step times a bounded row sample, "
                                   "ms_per_step extrapolates it to the full product"},
            "cpu_baseline": {"value": v, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample},
            "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}))
        return

    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    pkg.cu32.load()
    pkg.cu32.tune("clock", 1)
    for kv in a.tune:
        key, _, val = kv.partition("=")
        pkg.cu32.tune(key, int(val))
    pk = peaks()

    wl = Workload(a.workload, pkg, torch, rank, a.size, a.batch, a.images)
    for _ in range(a.warmup):
        wl.launch()
    check_status(pkg)

    gpu_uuid = None
    try:
        gpu_uuid = str(torch.cuda.get_device_properties(torch.cuda.current_device()).uuid)
    except Exception:
        pass
    box = {}

    def start_sampler():
        if rank == 0:
            box["sampler"] = ClockSampler(local_rank, gpu_uuid)

    def stop_sampler():
        if "sampler" in box:
            box["clocks"] = box.pop("sampler").stop()

    # ---- compute only (device-timed, inputs resident)
    pkg.cu32.read_clock()
    ms = time_steps(torch, dist, wl.launch, a.steps, world, start_sampler, stop_sampler)
    clocks = box.get("clocks")
    dev_clk = device_clock(pkg)
    check_status(pkg)
    ms_compute = ms / a.steps
    tile = pkg.cu32.get_tune("last_tile")

    # ---- N > 1: the step that counts includes the reassembly of the shards
    collective = None
    ms_step = ms_compute
    launches_per_step = wl.kernels_per_step
    if world > 1:
        if a.workload in ("c5", "c4_dw"):
            # K-sharded shapes: each rank reduces over its own rows (c5) or its own images (the convolution's
            # weight gradient, the data-parallel training pattern) and the partial outputs are summed
            def step_collective():
                wl.launch()
                dist.all_reduce(wl.out)
            kind, nblk = "all-reduce of the partial products", 1
            moved = 2.0 * wl.out.numel() * 4 * (world - 1) / world
        elif wl.cpu_case is not None and wl.cpu_case[0] in ("AB", "T2") and wl.kernels_per_step == 1 and wl.cpu_case[1] >= 2048:
            fused = None
            if os.environ.get("DRAGON_BENCH_GATHER", "fused") == "fused":
                try:
                    fused = FusedGatherStep(torch, dist, pkg, wl, world, rank)
                except Exception as ex:   # no peer-addressable memory on this box: fall back to the collective
                    if rank == 0:
                        print(f"peer-mapped output unavailable ({type(ex).__name__}: {ex}); using NCCL all-gather", file=sys.stderr)
            if fused is not None:
                step_collective = fused
                nblk = 1
                kind = ("output shards reassembled by the contraction kernel itself: every tile is stored into each rank's "
                        "copy of the full output over NVLink (stores only), no collective after the launch")
                moved = float(fused.bytes_sent)
            else:
                nblk = int(os.environ.get("DRAGON_BENCH_GATHER_BLOCKS", "2"))
                step_collective = ShardedStep(torch, dist, pkg, wl, world, nblk)
                kind = f"NCCL all-gather of the output shards in {nblk} row blocks, block b in flight while block b+1 is multiplied"
                moved = float(step_collective.bytes_received)
                launches_per_step = nblk
        else:
            gathered = torch.empty((world,) + tuple(wl.out.shape), device="cuda")

            def step_collective():
                wl.launch()
                dist.all_gather_into_tensor(gathered, wl.out)
            kind, nblk = "all-gather of the output shards after the launch", 1
            moved = float((world - 1) * wl.out.numel() * 4)
        # the collective's kernels need SMs of their own while the persistent contraction grid runs
        reserve = int(os.environ.get("DRAGON_BENCH_SM_RESERVE", "0")) if nblk > 1 else 0
        pkg.cu32.tune("sm_reserve", reserve)
        for _ in range(3):
            step_collective()
        ms_step = time_steps(torch, dist, step_collective, a.steps, world) / a.steps
        pkg.cu32.tune("sm_reserve", 0)
        check_status(pkg)
        gathered_ok = step_collective.check() if isinstance(step_collective, FusedGatherStep) else None
        exposed = max(ms_step - ms_compute, 1e-9)
        collective = {"kind": kind, "ms_per_step": ms_step, "compute_only_ms": ms_compute,
                      "bytes_over_nvlink_per_rank": moved, "sms_left_to_the_collective": reserve,
                      "gathered_output_verified": gathered_ok,
                      "exposed_ms": ms_step - ms_compute,
                      "nvlink_gbs_over_the_step": moved / (ms_step * 1e-3) / 1e9,
                      "note": "NVLink reference on this pool: 770 GB/s peer copy per direction"}
    value = wl.flops * world / (ms_step * 1e-3) / 1e12

    # ---- strong scaling: the 8192^3 problem itself, rows divided over the ranks, output reassembled
    strong = None
    if world > 1 and a.workload == "c2_ab" and a.size % (world * 4 * 128) == 0:
        rows = a.size // world
        dA, dB = wl.dev_in[0][:rows], wl.dev_in[1]
        mm = pkg.cu32.Cuda_matMul
        pg = None
        if isinstance(step_collective, FusedGatherStep):
            pg = pkg.shard.PeerGather(dist, world, rank, (rows, a.size), torch.device("cuda", torch.cuda.current_device()))

            def strong_step():
                mm.matMul_replicated([torch.cuda.current_stream().cuda_stream], 1, dA.data_ptr(), dB.data_ptr(),
                                     pg.local.data_ptr(), pg.replicas, rows, a.size, a.size)
            how = "C reassembled by the kernel's own stores into every rank's copy"
        else:
            dC = wl.out[:rows]
            full = torch.empty((world, rows * a.size), device="cuda")

            def strong_step():
                mm.matMul([torch.cuda.current_stream().cuda_stream], 1, dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), rows, a.size, a.size)
                dist.all_gather_into_tensor(full.view(-1), dC.reshape(-1))
            how = "C all-gathered (NCCL) after the launch"
        for _ in range(3):
            strong_step()
        ms_s = time_steps(torch, dist, strong_step, a.steps, world) / a.steps
        if pg is not None:
            pg.barrier()
        strong = {"value": 2.0 * a.size ** 3 / (ms_s * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": ms_s,
                  "workload": f"matMul AB 8192^3 in total: {rows} rows of A and C per rank, B replicated, {how}"}

    # ---- end to end with host buffers
    e2e = None
    if not a.no_e2e:
        wl.prepare_e2e()
        if getattr(wl, "row_blocks", None) is not None and "DRAGON_BENCH_E2E_BLOCKS" not in os.environ:
            # Warm-up doubles as the choice of the pipeline's row-block count: fewer, larger blocks keep the copy
            # engine at its best rate and fill the persistent grid; more, smaller ones shorten the tail after the
            # last copy.  Which wins depends on the host (PCIe rate with both directions busy), so each candidate
            # runs twice here and the fastest is kept for the timed steps.
            best = None
            for nblk in (16, 20, 32):
                wl.nblk = nblk
                wl.e2e_step()
                t = time_steps(torch, None, wl.e2e_step, 2, 1)
                if best is None or t < best[0]:
                    best = (t, nblk)
            wl.nblk = best[1]
        for _ in range(3):
            wl.e2e_step()
        e2e_steps = max(3, min(a.steps, 10))
        ms_e = time_steps(torch, dist, wl.e2e_step, e2e_steps, world) / e2e_steps
        e2e = {"value": wl.flops * world / (ms_e * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": ms_e,
               "h2d_bytes_per_step": wl.h2d, "d2h_bytes_per_step": wl.d2h}
        if getattr(wl, "row_blocks", None) is not None:
            e2e["row_blocks"] = wl.nblk

    # ---- sustained: the same launch back to back for >= 2 s, clocks sampled, against the sustained peak
    sustained = None
    extras = world == 1 and not a.no_extras and a.workload == "c2_ab" and a.size == 8192
    if extras:
        n_sus = max(a.steps, int(2200.0 / ms_compute))
        pkg.cu32.read_clock()
        ms_sus = time_steps(torch, dist, wl.launch, n_sus, world, start_sampler, stop_sampler) / n_sus
        clk_sus = device_clock(pkg)
        check_status(pkg)
        roof_s = roofline_of(a.workload, wl, ms_sus, pk, sustained=True)
        sustained = {"launches": n_sus, "seconds": n_sus * ms_sus * 1e-3, "ms_per_step": ms_sus,
                     "value": wl.flops / (ms_sus * 1e-3) / 1e12, "unit": UNIT, "frac": roof_s["frac"], "peak": roof_s["peak"],
                     "peak_basis": roof_s["peak_basis"], "effective_sm_mhz": clk_sus["effective_sm_mhz"],
                     "clocks": box.get("clocks")}

    gpu_ref = gpu_reference_leg(torch, wl) if extras else None
    if gpu_ref:
        gpu_ref["ratio"] = (wl.flops / (ms_compute * 1e-3) / 1e12) / gpu_ref["value"]

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    roof = roofline_of(a.workload, wl, ms_compute, pk, sustained=a.steps * ms_compute > 1500.0,
                       traffic=NCU_TRAFFIC_BYTES.get(a.workload) if (a.size == 8192 and a.batch == 1024) else None)

    # ---- where the fraction comes from: (tensor-pipe utilisation at the clock the kernel ran at) x (that clock / max)
    clock = dict(dev_clk)
    clock["nvml_median_mhz"] = clocks.get("sm_mhz") if clocks else None
    clock["sm_max_mhz"] = clocks.get("sm_max_mhz") if clocks else None
    if roof["bound"] == "tensor" and wl.cpu_case is not None and dev_clk["effective_sm_mhz"] and tile in (4,) \
            and wl.kernels_per_step == 1:
        form, N, M, K = wl.cpu_case[:4]
        sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
        tiles = -(-N // 256) * -(-M // 256)
        rounds = -(-tiles // (sms // 2))
        kblocks = -(-K // 32)
        cyc = ms_compute * 1e-3 * dev_clk["effective_sm_mhz"] * 1e6 / (rounds * kblocks)
        clock.update({"tile_rounds": rounds, "k_blocks": kblocks, "cycles_per_kblock": cyc, "ideal_cycles_per_kblock": 1536,
                      "pipe_utilisation": 1536.0 / cyc,
                      "explains": "frac = pipe_utilisation x (tiles / (rounds x CTA pairs)) x effective clock x 4096 TF32-flop/clk/SM x SMs / 3 / peak"})
        if clock["sm_max_mhz"]:
            clock["clock_ratio"] = dev_clk["effective_sm_mhz"] / clock["sm_max_mhz"]

    cpu = None
    if world == 1 and not a.no_cpu_baseline and wl.cpu_case is not None:
        form, N, M, K, A, B = wl.cpu_case
        v, cores, kind, sample = cpu_reference_loop(form, N, M, K, A.numpy(), B.numpy(), passes=3)
        cpu = {"value": v, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample}

    configs = None
    if extras:
        del wl.dev_in, wl.out
        torch.cuda.empty_cache()
        configs = other_configs(pkg, torch, pk, ["c1", "c2_t1", "c2_t2", "c2_ragged", "c3_qk", "c3_pv", "c3_attn", "c4", "c5"],
                                a.steps, a.warmup)

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": a.steps, "warmup": a.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "tf32x3",
        "data": "synthetic",
        "config": {"workload": wl.desc + (f"; {world} ranks, each its own shard of a {world}x larger problem, "
                                                    "output shards all-gathered inside the step" if world > 1 else ""),
                   "l2": "operands larger than L2 (no flush needed)" if wl.bytes > 126e6 else "L2 not flushed: operands fit in L2",
                   "kc": pkg.cu32.get_tune("kc"), "tile": TILE_NAMES.get(tile, tile)},
        "roofline": roof, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": a.steps * launches_per_step,
        "clocks": clocks, "clock": clock,
    }
    if world > 1:
        line["compute_only"] = {"value": wl.flops * world / (ms_compute * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": ms_compute}
        line["collective"] = collective
        if strong:
            line["strong"] = strong
    if sustained:
        line["sustained"] = sustained
    if gpu_ref:
        line["gpu_reference"] = gpu_ref
    if configs:
        line["configs"] = configs
    if hasattr(wl, "images"):
        line["images_per_s"] = wl.images * world / (ms_step * 1e-3)
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
