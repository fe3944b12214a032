#!/usr/bin/env python
"""Benchmark of the five hot-path kernels on B200: HBM GB/s and tensor TFLOP/s per GPU against the
measured roofline, next to the same computation on the host CPU.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workloads a,b,...]

One JSON line on stdout (rank 0).  The headline workload is the fp32 row softmax [16384, 4096]; the
other four workloads (vadd 2^28, fp16 GEMM 8192^3, int8 GEMM 8192^3 with dequant, attention forward
[4,32,4096,128] non-causal and causal) are reported under "workloads" with the same sub-keys, and once
more, compactly, under "summary" (the last key of the line).

value      device-resident throughput: the K timed launches are recorded into one CUDA graph and the
           graph is replayed once between two CUDA events on the launching stream (max over ranks);
           algorithmic bytes or FLOPs of the whole configuration / time per step.
e2e        the same metric through the public asc2 surface (`kernel[cores](host tensors)`): pinned host
           tensors in, host tensor out, H2D and D2H copies inside the timed region.
roofline   achieved (= value per GPU) over the measured peak from MEASURED_PEAKS.json.
cpu_baseline / --impl reference
           the reference's own CPU computation of the path (the torch expressions its tests assert
           against, oracle/golden.py) timed on a bounded sample with all host threads.

Multi-GPU (launched under torchrun, one rank per GPU): strong scaling.  The one fixed configuration of
every workload is split N ways along its independent axis (element ranges, softmax rows, row blocks of A
and C with B replicated, batch x heads; pyasc_b200/sharding.py), the inputs are resident before the timed
region, there is no data-path collective, and a step is one pass over the whole configuration: in step i
rank r processes shard (r + i) mod N, so every step covers each shard exactly once and no rank re-reads
data that is still in its L2.  Per workload the line also carries "allgather_ms" (the NCCL all-gather that
reassembles the output in place on every rank, alone), "compute_plus_allgather_ms" (kernel, then gather),
"speedup_vs_one_gpu" (the same run's single-GPU time of the whole configuration / the sharded time) and,
under "weak", the replica numbers (every rank runs the whole configuration on its own).
All inputs are seeded synthetic data with the workloads' shapes and distributions; every timed input
set is larger than the 126 MB L2.
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
from typing import Any, Callable, Dict, List, Optional

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

HEADLINE = "softmax"
ALL_WORKLOADS = ["softmax", "vadd", "gemm_f16", "gemm_i8", "gemm_i8_dequant", "attention", "attention_causal",
                 "gelu", "gelu_tanh", "leaky_relu_bf16", "mish", "row_sum", "rms_norm", "layer_norm"]

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks() -> Dict[str, Any]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            peaks = json.load(f)
        peaks["source"] = "measured"
        return peaks
    peaks = dict(FALLBACK_PEAKS)
    peaks["source"] = "fallback"
    return peaks


# ---------------------------------------------------------------------------------------------------
# clocks: nvidia-smi sampled while the timed regions run
# ---------------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.proc: Optional[subprocess.Popen] = None
        self.gpu_index = gpu_index

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu_index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> Dict[str, Any]:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, smax, power = [], [], []
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                smax.append(float(parts[1]))
                power.append(float(parts[2]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[3:7]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        busy = [s for s, p in zip(sm, power) if p > 300.0] or sm
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(smax) if smax else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


# ---------------------------------------------------------------------------------------------------
# seeded synthetic inputs with the workloads' shapes and distributions
# ---------------------------------------------------------------------------------------------------
SEED = 2026      # the reference's own asc2 seed (python/test/asc2/kernels/test_vadd.py:43)


def seeded(device="cpu", seed: int = SEED) -> torch.Generator:
    return torch.Generator(device=device).manual_seed(seed)


def softmax_input(rows: int, cols: int, device="cpu") -> torch.Tensor:
    return torch.randn(rows, cols, generator=seeded(device), device=device)


def vadd_inputs(n: int, device="cpu"):
    g = seeded(device)
    return torch.rand(n, generator=g, device=device), torch.rand(n, generator=g, device=device)


def gemm_f16_inputs(m: int, n: int, k: int, device="cpu"):
    g = seeded(device)
    a = (torch.randn(m, k, generator=g, device=device) * k ** -0.5).to(torch.float16)
    b = (torch.randn(k, n, generator=g, device=device) * k ** -0.5).to(torch.float16)
    return a, b


def gemm_i8_inputs(m: int, n: int, k: int, device="cpu"):
    g = seeded(device)
    a = torch.randint(-128, 128, (m, k), dtype=torch.int8, generator=g, device=device)
    b = torch.randint(-128, 128, (k, n), dtype=torch.int8, generator=g, device=device)
    a_scale = torch.rand(m, generator=g, device=device) * (1e-2 - 1e-3) + 1e-3
    b_scale = torch.rand(n, generator=g, device=device) * (1e-2 - 1e-3) + 1e-3
    return a, b, a_scale, b_scale


def attention_inputs(heads: int, seq: int, dim: int, device="cpu"):
    g = seeded(device)
    return tuple(torch.randn(heads, seq, dim, generator=g, device=device).to(torch.float16) for _ in range(3))


# ---------------------------------------------------------------------------------------------------
# workloads
# ---------------------------------------------------------------------------------------------------
def P(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


class Workload:
    """One benchmarked configuration.  `work` is the algorithmic bytes (HBM-bound) or FLOPs (tensor-bound) of the
    whole configuration; `units` is the length of the independent axis the configuration is sharded along
    (pyasc_b200.sharding.partition_for names the same axes) and `granule` the multiple shard boundaries keep."""
    name = ""
    label = ""
    unit = "GB/s"
    bound = "hbm"
    dtype = "f32"
    work = 0.0
    units = 0
    granule = 1
    axis = ""
    replicated: tuple = ()
    h2d_bytes = 0           # of the whole configuration; a shard moves its share (+ the replicated operands)
    d2h_bytes = 0
    replicated_h2d_bytes = 0

    def setup_device(self, dev: torch.device) -> None: ...            # the whole configuration, resident
    def launch_units(self, lib, stream, lo: int, hi: int) -> int: ...  # the C-ABI call(s) for units [lo, hi)
    def output(self) -> torch.Tensor: ...                             # the whole output; numel % units == 0
    def setup_host(self, lo: int, hi: int) -> None: ...               # pinned host tensors of units [lo, hi)
    def e2e_step(self) -> None: ...                                   # the public asc2 call on them
    def cpu_sample(self) -> float: ...          # runs the bounded CPU sample once, returns its work
    cpu_sample_desc = ""

    def throughput(self, work: float, seconds: float) -> float:
        return work / seconds / (1e9 if self.unit == "GB/s" else 1e12)

    def peak(self, peaks: Dict[str, Any]) -> float:
        return float(peaks["hbm_gbs"]) if self.bound == "hbm" else float(peaks["bf16_tflops"])


class Softmax(Workload):
    name, label, dtype = "softmax", "softmax_f32_16384x4096", "f32"
    R, C = 16384, 4096
    units, granule, axis = R, 1, "rows"
    work = 2.0 * 4 * R * C                      # one 4-byte read + one 4-byte write per element
    h2d_bytes, d2h_bytes = 4 * R * C, 4 * R * C
    cpu_sample_desc = "torch.softmax(x, -1) on the full [16384, 4096] input"

    def setup_device(self, dev):
        self.x = softmax_input(self.R, self.C, dev)
        self.out = torch.empty_like(self.x)

    def launch_units(self, lib, stream, lo, hi):
        return lib.asc_cuda_softmax_f32(P(self.x[lo:hi]), P(self.out[lo:hi]), hi - lo, self.C, self.C, stream)

    def output(self):
        return self.out

    def setup_host(self, lo, hi):
        self.hx = softmax_input(hi - lo, self.C).pin_memory()
        self.hout = torch.empty_like(self.hx).pin_memory()

    def e2e_step(self):
        from pyasc_b200 import tutorials as T
        T.softmax_launch(self.hx, self.hout, core_num=148)

    def cpu_sample(self):
        from oracle import golden as G
        if not hasattr(self, "cx"):
            self.cx = softmax_input(self.R, self.C)
        G.softmax(self.cx)
        return self.work


class VAdd(Workload):
    name, label, dtype = "vadd", "vadd_f32_2^28", "f32"
    N = 1 << 28
    units, granule, axis = N, 1 << 16, "elements"
    work = 3.0 * 4 * N
    h2d_bytes, d2h_bytes = 2 * 4 * N, 4 * N
    CPU_N = 1 << 26
    cpu_sample_desc = "x + y on 2^26 of the 2^28 elements"

    def setup_device(self, dev):
        self.x, self.y = vadd_inputs(self.N, dev)
        self.out = torch.empty_like(self.x)

    def launch_units(self, lib, stream, lo, hi):
        return lib.asc_cuda_vadd_f32(P(self.x[lo:hi]), P(self.y[lo:hi]), P(self.out[lo:hi]), hi - lo, stream)

    def output(self):
        return self.out

    def setup_host(self, lo, hi):
        x, y = vadd_inputs(hi - lo)
        self.hx, self.hy = x.pin_memory(), y.pin_memory()
        self.hout = torch.empty(hi - lo).pin_memory()

    def e2e_step(self):
        from pyasc_b200 import tutorials as T
        T.vadd_launch(self.hx, self.hy, self.hout, core_num=148, tile_size=1 << 16)

    def cpu_sample(self):
        from oracle import golden as G
        if not hasattr(self, "cx"):
            self.cx, self.cy = vadd_inputs(self.CPU_N)
        G.vadd(self.cx, self.cy)
        return 3.0 * 4 * self.CPU_N


class GemmF16(Workload):
    name, label, dtype, unit, bound = "gemm_f16", "gemm_f16_8192x8192x8192_f32acc_f16out", "f16", "TFLOP/s", "tensor"
    M = N = K = 8192
    units, granule, axis, replicated = M, 256, "rows of A and C", ("B", )
    work = 2.0 * M * N * K
    h2d_bytes, d2h_bytes, replicated_h2d_bytes = 2 * (M * K + K * N), 2 * M * N, 2 * K * N
    CPU_M = 1024
    cpu_sample_desc = "(A.float() @ B.float()).half() on 1024 of the 8192 rows of A"

    def setup_device(self, dev):
        self.a, self.b = gemm_f16_inputs(self.M, self.N, self.K, dev)
        self.c = torch.empty(self.M, self.N, dtype=torch.float16, device=dev)

    def launch_units(self, lib, stream, lo, hi):
        return lib.asc_cuda_gemm_f16(P(self.a[lo:hi]), P(self.b), P(self.c[lo:hi]), hi - lo, self.N, self.K, self.K,
                                     self.N, self.N, 0, 0, 0, stream)

    def output(self):
        return self.c

    def setup_host(self, lo, hi):
        a, b = gemm_f16_inputs(hi - lo, self.N, self.K)
        self.ha, self.hb = a.pin_memory(), b.pin_memory()
        self.hc = torch.empty(hi - lo, self.N, dtype=torch.float16).pin_memory()

    def e2e_step(self):
        from pyasc_b200 import tutorials as T
        T.matmul_fp16_launch(self.ha, self.hb, self.hc, core_num=148)

    def cpu_sample(self):
        from oracle import golden as G
        if not hasattr(self, "ca"):
            self.ca, self.cb = gemm_f16_inputs(self.CPU_M, self.N, self.K)
        G.gemm_f16(self.ca, self.cb)
        return 2.0 * self.CPU_M * self.N * self.K


class GemmI8(Workload):
    name, label, dtype, unit, bound = "gemm_i8", "gemm_i8_8192x8192x8192_int32out", "s8", "TFLOP/s", "tensor"
    M = N = K = 8192
    units, granule, axis, replicated = M, 256, "rows of A and C", ("B", )
    work = 2.0 * M * N * K
    h2d_bytes, d2h_bytes, replicated_h2d_bytes = M * K + K * N, 4 * M * N, K * N
    CPU_M = 256
    dequant = False
    cpu_sample_desc = "A.int32 @ B.int32 (evaluated exactly in fp64) on 256 of the 8192 rows of A"

    def peak(self, peaks):
        return 2.0 * float(peaks["bf16_tflops"])    # dense int8 runs at twice the 16-bit rate

    def setup_device(self, dev):
        self.a, self.b, self.sa, self.sb = gemm_i8_inputs(self.M, self.N, self.K, dev)
        self.acc = None if self.dequant else torch.empty(self.M, self.N, dtype=torch.int32, device=dev)
        self.deq = torch.empty(self.M, self.N, dtype=torch.float16, device=dev) if self.dequant else None

    def launch_units(self, lib, stream, lo, hi):
        return lib.asc_cuda_gemm_i8(P(self.a[lo:hi]), P(self.b), P(self.acc[lo:hi]) if self.acc is not None else None,
                                    P(self.deq[lo:hi]) if self.deq is not None else None,
                                    P(self.sa[lo:hi]) if self.dequant else None, P(self.sb) if self.dequant else None,
                                    hi - lo, self.N, self.K, self.K, self.N, self.N, stream)

    def output(self):
        return self.deq if self.dequant else self.acc

    def setup_host(self, lo, hi):
        a, b, sa, sb = gemm_i8_inputs(hi - lo, self.N, self.K)
        self.ha, self.hb, self.hsa, self.hsb = a.pin_memory(), b.pin_memory(), sa.pin_memory(), sb.pin_memory()
        self.hacc = torch.empty(hi - lo, self.N, dtype=torch.int32).pin_memory() if not self.dequant else None
        self.hdeq = torch.empty(hi - lo, self.N, dtype=torch.float16).pin_memory() if self.dequant else None

    def e2e_step(self):
        from pyasc_b200 import tutorials as T
        if self.dequant:
            T.matmul_int8_dequant_launch(self.ha, self.hb, self.hsa, self.hsb, self.hdeq, core_num=148)
        else:
            T.matmul_int8_launch(self.ha, self.hb, self.hacc, core_num=148)

    def cpu_sample(self):
        from oracle import golden as G
        if not hasattr(self, "ca"):
            self.ca, self.cb, self.csa, self.csb = gemm_i8_inputs(self.CPU_M, self.N, self.K)
        acc = G.gemm_i8(self.ca, self.cb)
        if self.dequant:
            G.dequant(acc, self.csa, self.csb)
        return 2.0 * self.CPU_M * self.N * self.K


class GemmI8Dequant(GemmI8):
    name, label = "gemm_i8_dequant", "gemm_i8_8192x8192x8192_dequant_f16out"
    dequant = True
    replicated = ("B", "b_scale")
    d2h_bytes = 2 * GemmI8.M * GemmI8.N
    h2d_bytes = GemmI8.h2d_bytes + 4 * (GemmI8.M + GemmI8.N)
    replicated_h2d_bytes = GemmI8.replicated_h2d_bytes + 4 * GemmI8.N
    cpu_sample_desc = "A.int32 @ B.int32 then acc * a_scale[row] * b_scale[col] -> fp16 on 256 of the 8192 rows"


class Attention(Workload):
    name, label, dtype, unit, bound = "attention", "attention_fwd_f16_b4_h32_s4096_d128", "f16", "TFLOP/s", "tensor"
    B, H, S, D = 4, 32, 4096, 128
    units, granule, axis = B * H, 1, "batch x heads"
    causal = False
    work = 4.0 * B * H * S * S * D
    h2d_bytes, d2h_bytes = 3 * 2 * B * H * S * D, 2 * B * H * S * D
    CPU_HEADS = 2
    cpu_sample_desc = "fp32 softmax(QK^T*scale)V on 2 of the 128 (batch, head) pairs"

    def setup_device(self, dev):
        self.q, self.k, self.v = attention_inputs(self.units, self.S, self.D, dev)     # [B*H, S, D]
        self.o = torch.empty_like(self.q)

    def launch_units(self, lib, stream, lo, hi):
        return lib.asc_cuda_attn_fwd_f16(P(self.q[lo:hi]), P(self.k[lo:hi]), P(self.v[lo:hi]), P(self.o[lo:hi]), 1,
                                         hi - lo, self.S, self.D, ctypes.c_float(self.D ** -0.5), int(self.causal), 0,
                                         stream)

    def output(self):
        return self.o

    def setup_host(self, lo, hi):
        q, k, v = attention_inputs(hi - lo, self.S, self.D)
        self.hq, self.hk, self.hv = (t.reshape(1, hi - lo, self.S, self.D).pin_memory() for t in (q, k, v))
        self.ho = torch.empty_like(self.hq).pin_memory()

    def e2e_step(self):
        from pyasc_b200 import tutorials as T
        T.attention_launch(self.hq, self.hk, self.hv, self.ho, causal=self.causal, core_num=148)

    def cpu_sample(self):
        from oracle import golden as G
        if not hasattr(self, "cq"):
            self.cq, self.ck, self.cv = (t[None] for t in attention_inputs(self.CPU_HEADS, self.S, self.D))
        G.attention(self.cq, self.ck, self.cv, self.causal)
        return self.work * self.CPU_HEADS / (self.B * self.H)


class AttentionCausal(Attention):
    name, label = "attention_causal", "attention_fwd_f16_b4_h32_s4096_d128_causal"
    causal = True
    work = Attention.work / 2                    # the usual convention: masked half not counted
    cpu_sample_desc = "fp32 causal softmax(QK^T*scale + mask)V on 2 of the 128 (batch, head) pairs"


class _Planned(Workload):
    """An asc2 kernel whose device leg launches the C-ABI calls the launcher plans for it: the plan of the whole
    configuration is built once (with the launch itself suppressed), and units [lo, hi) are launched through the
    plan's own chunking rule (the one the launcher's copy/compute pipeline uses)."""

    def plan(self, launch_fn, kernel, ptr_args: Dict[int, torch.Tensor], patterns=("elementwise:program", "row:program")):
        prev = os.environ.get("DRY_RUN")
        os.environ["DRY_RUN"] = "1"
        try:
            launch_fn()
        finally:
            if prev is None:
                del os.environ["DRY_RUN"]
            else:
                os.environ["DRY_RUN"] = prev
        plan = kernel.last_plan
        assert plan.pattern in patterns and len(plan.steps) == 1 and plan.pipeline is not None, plan
        from pyasc_b200 import jit
        jit.prepare(plan, wait=True)        # the kernel specialised for this expression: built (or found in the cache) now
        self.spec = plan.pipeline
        self.units, self.granule = self.spec.units, self.spec.granule
        self.ptrs = {i: t.data_ptr() for i, t in ptr_args.items()}

    def launch_units(self, lib, stream, lo, hi):
        rc = 0
        for step in self.spec.make_steps(lo, hi):
            rc = rc or getattr(lib, step.fn_name)(*step.build(self.ptrs, stream))
        return rc

    def output(self):
        return self.out


class Gelu(_Planned):
    name, label, dtype = "gelu", "gelu_erf_f32_16384x4096", "f32"
    approximate = False
    R, C = 16384, 4096
    units, granule, axis = R * C, 1 << 16, "elements"
    work = 2.0 * 4 * R * C
    h2d_bytes, d2h_bytes = 4 * R * C, 4 * R * C
    CPU_R = 4096
    cpu_sample_desc = "0.5*x*(1+erf(x/sqrt(2))) in torch on 4096 of the 16384 rows"

    def make_x(self, rows, device="cpu"):
        return torch.rand((rows, self.C), device=device, generator=seeded(device)) * 6 - 3

    def setup_device(self, dev):
        from pyasc_b200 import tutorials as T
        self.x = self.make_x(self.R, dev)
        self.out = torch.empty_like(self.x)
        self.plan(lambda: T.gelu_launch(self.x, self.out, self.approximate, core_num=148), T.gelu_kernel,
                  {0: self.x, 1: self.out})

    def setup_host(self, lo, hi):
        self.hx = self.make_x((hi - lo) // self.C).pin_memory()
        self.hout = torch.empty_like(self.hx).pin_memory()

    def e2e_step(self):
        from pyasc_b200 import tutorials as T
        T.gelu_launch(self.hx, self.hout, self.approximate, core_num=148)

    def cpu_sample(self):
        import math
        if not hasattr(self, "cx"):
            self.cx = self.make_x(self.CPU_R)
        x = self.cx
        if self.approximate:
            _ = 0.5 * x * (1 + torch.tanh(math.sqrt(2 / math.pi) * (x + 0.044715 * torch.pow(x, 3))))
        else:
            _ = 0.5 * x * (1 + torch.erf(x / math.sqrt(2)))
        return 2.0 * 4 * self.CPU_R * self.C


class GeluTanh(Gelu):
    name, label = "gelu_tanh", "gelu_tanh_f32_16384x4096"
    approximate = True
    cpu_sample_desc = "the tanh-form GELU expression in torch on 4096 of the 16384 rows"


class Mish(Gelu):
    """x * tanh(log(exp(x) + 1)): an expression a user writes that is not one of the reference's own kernels."""
    name, label = "mish", "mish_f32_16384x4096"
    cpu_sample_desc = "x * tanh(log(exp(x) + 1)) in torch on 4096 of the 16384 rows"

    @staticmethod
    def kernel():
        import pyasc_b200  # noqa: F401  (makes `asc` / `asc2` importable)
        import asc
        import asc2

        @asc2.jit
        def mish_kernel(x_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, num_rows: int,
                        num_columns: asc.ConstExpr):
            x_gm = asc2.tensor(x_ptr, [num_rows, num_columns])
            out_gm = asc2.tensor(out_ptr, [num_rows, num_columns])
            for i in range(asc2.block_idx(), num_rows, asc2.block_num()):
                row = asc2.load(x_gm, [1, num_columns], offsets=[i, 0])
                asc2.store(row * asc2.tanh(asc2.log(asc2.exp(row) + 1)), out_gm, offsets=[i, 0])
        return mish_kernel

    def setup_device(self, dev):
        self.x = self.make_x(self.R, dev)
        self.out = torch.empty_like(self.x)
        self.k = self.kernel()
        self.plan(lambda: self.k[148](self.x, self.out, self.R, self.C), self.k, {0: self.x, 1: self.out})

    def setup_host(self, lo, hi):
        self.hx = self.make_x((hi - lo) // self.C).pin_memory()
        self.hout = torch.empty_like(self.hx).pin_memory()
        if not hasattr(self, "k"):
            self.k = self.kernel()

    def e2e_step(self):
        self.k[148](self.hx, self.hout, self.hx.shape[0], self.C)

    def cpu_sample(self):
        if not hasattr(self, "cx"):
            self.cx = self.make_x(self.CPU_R)
        _ = self.cx * torch.tanh(torch.log(torch.exp(self.cx) + 1))
        return 2.0 * 4 * self.CPU_R * self.C


class RowSum(Workload):
    """asc2.reduce_sum over the rows of [65536, 4096] fp32 (1 GiB read, 256 KiB written)."""
    name, label, dtype = "row_sum", "row_sum_f32_65536x4096", "f32"
    R, C = 65536, 4096
    units, granule, axis = R, 64, "rows"
    work = 4.0 * R * C + 4.0 * R
    h2d_bytes, d2h_bytes = 4 * R * C, 4 * R
    CPU_R = 16384
    cpu_sample_desc = "x.sum(1) in torch on 16384 of the 65536 rows"

    def setup_device(self, dev):
        self.x = torch.randn((self.R, self.C), device=dev, generator=seeded(dev))
        self.out = torch.empty(self.R, device=dev)

    def launch_units(self, lib, stream, lo, hi):
        return lib.asc_cuda_reduce_f32(P(self.x[lo:hi]), P(self.out[lo:hi]), hi - lo, self.C, self.C, 1, 0, 1, stream)

    def output(self):
        return self.out

    @staticmethod
    def kernel():
        import pyasc_b200  # noqa: F401  (makes `asc` / `asc2` importable)
        import asc
        import asc2

        @asc2.jit
        def row_sum_kernel(x_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, num_rows: int,
                           num_cols: asc.ConstExpr[int], rows_per_tile: asc.ConstExpr[int]):
            x_gm = asc2.tensor(x_ptr, [num_rows, num_cols])
            out_gm = asc2.tensor(out_ptr, [num_rows])
            for i in range(asc2.block_idx() * rows_per_tile, num_rows, asc2.block_num() * rows_per_tile):
                tile = asc2.load(x_gm, [rows_per_tile, num_cols], offsets=[i, 0])
                asc2.store(asc2.reduce_sum(tile, 1), out_gm, offsets=[i])
        return row_sum_kernel

    def setup_host(self, lo, hi):
        self.hx = torch.randn((hi - lo, self.C), generator=seeded()).pin_memory()
        self.hout = torch.empty(hi - lo).pin_memory()
        self.k = self.kernel()

    def e2e_step(self):
        self.k[148](self.hx, self.hout, self.hx.shape[0], self.C, 8)

    def cpu_sample(self):
        if not hasattr(self, "cx"):
            self.cx = torch.randn((self.CPU_R, self.C), generator=seeded())
        _ = self.cx.sum(1)
        return 4.0 * self.CPU_R * self.C


class RmsNorm(Workload):
    """asc2.rms_norm over the rows of [16384, 4096] fp32 (256 MiB read, 256 MiB written, gamma resident)."""
    name, label, dtype = "rms_norm", "rms_norm_f32_16384x4096", "f32"
    R, C = 16384, 4096
    units, granule, axis, replicated = R, 1, "rows", ("gamma", )
    EPS = 1e-5
    work = 2.0 * 4 * R * C
    h2d_bytes, d2h_bytes, replicated_h2d_bytes = 4 * R * C + 4 * C, 4 * R * C, 4 * C
    CPU_R = 4096
    cpu_sample_desc = "x * rsqrt(mean(x^2, 1) + eps) * gamma in torch on 4096 of the 16384 rows"

    def make(self, rows, device="cpu"):
        g = seeded(device)
        return (torch.randn((rows, self.C), device=device, generator=g),
                torch.rand((1, self.C), device=device, generator=g) + 0.5,
                torch.randn((1, self.C), device=device, generator=g))

    def setup_device(self, dev):
        self.x, self.gamma, _ = self.make(self.R, dev)
        self.out = torch.empty_like(self.x)

    def launch_units(self, lib, stream, lo, hi):
        return lib.asc_cuda_rms_norm_f32(P(self.x[lo:hi]), P(self.gamma), P(self.out[lo:hi]), hi - lo, self.C, self.C,
                                         self.EPS, stream)

    def output(self):
        return self.out

    @staticmethod
    def kernel():
        import pyasc_b200  # noqa: F401  (makes `asc` / `asc2` importable)
        import asc
        import asc2

        @asc2.jit
        def rms_norm_kernel(x_ptr: asc.GlobalAddress, gamma_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress,
                            num_rows: int, num_cols: asc.ConstExpr[int], rows_per_tile: asc.ConstExpr[int],
                            epsilon: float):
            x_gm = asc2.tensor(x_ptr, [num_rows, num_cols])
            out_gm = asc2.tensor(out_ptr, [num_rows, num_cols])
            gamma = asc2.load(asc2.tensor(gamma_ptr, [1, num_cols]), [1, num_cols], offsets=[0, 0])
            for i in range(asc2.block_idx() * rows_per_tile, num_rows, asc2.block_num() * rows_per_tile):
                tile = asc2.load(x_gm, [rows_per_tile, num_cols], offsets=[i, 0])
                asc2.store(asc2.rms_norm(tile, gamma, epsilon), out_gm, offsets=[i, 0])
        return rms_norm_kernel

    def setup_host(self, lo, hi):
        x, gamma, _ = self.make(hi - lo)
        self.hx, self.hgamma = x.pin_memory(), gamma.pin_memory()
        self.hout = torch.empty_like(self.hx).pin_memory()
        self.k = self.kernel()

    def e2e_step(self):
        self.k[148](self.hx, self.hgamma, self.hout, self.hx.shape[0], self.C, 4, self.EPS)

    def cpu_sample(self):
        if not hasattr(self, "cx"):
            self.cx, self.cg, _ = self.make(self.CPU_R)
        _ = self.cx * torch.rsqrt(self.cx.pow(2).mean(1, keepdim=True) + self.EPS) * self.cg
        return 2.0 * 4 * self.CPU_R * self.C


class LayerNorm(_Planned):
    """Layer norm written with asc2 reductions and broadcasts (mean, centred variance, scale and shift): one row
    program over [16384, 4096] fp32 (256 MiB read, 256 MiB written; gamma and beta resident)."""
    name, label, dtype = "layer_norm", "layer_norm_f32_16384x4096_row_program", "f32"
    R, C = 16384, 4096
    units, granule, axis, replicated = R, 1, "rows", ("gamma", "beta")
    EPS = 1e-5
    work = 2.0 * 4 * R * C
    h2d_bytes, d2h_bytes, replicated_h2d_bytes = 4 * R * C + 8 * C, 4 * R * C, 8 * C
    CPU_R = 4096
    cpu_sample_desc = "torch.nn.functional.layer_norm on 4096 of the 16384 rows"
    make = RmsNorm.make

    @staticmethod
    def kernel():
        import pyasc_b200  # noqa: F401  (makes `asc` / `asc2` importable)
        import asc
        import asc2

        @asc2.jit
        def layer_norm_kernel(x_ptr: asc.GlobalAddress, gamma_ptr: asc.GlobalAddress, beta_ptr: asc.GlobalAddress,
                              out_ptr: asc.GlobalAddress, num_rows: int, num_cols: asc.ConstExpr[int],
                              rows_per_tile: asc.ConstExpr[int], epsilon: float):
            x_gm = asc2.tensor(x_ptr, [num_rows, num_cols])
            out_gm = asc2.tensor(out_ptr, [num_rows, num_cols])
            gamma = asc2.load(asc2.tensor(gamma_ptr, [1, num_cols]), [1, num_cols], offsets=[0, 0])
            beta = asc2.load(asc2.tensor(beta_ptr, [1, num_cols]), [1, num_cols], offsets=[0, 0])
            for i in range(asc2.block_idx() * rows_per_tile, num_rows, asc2.block_num() * rows_per_tile):
                x = asc2.load(x_gm, [rows_per_tile, num_cols], offsets=[i, 0])
                mean = (asc2.reduce_sum(x, 1, keep_dims=True) / num_cols).broadcast_to(rows_per_tile, num_cols)
                xc = x - mean
                var = (asc2.reduce_sum(xc * xc, 1, keep_dims=True) / num_cols).broadcast_to(rows_per_tile, num_cols)
                y = xc * asc2.rsqrt(var + epsilon)
                asc2.store(y * gamma.broadcast_to(rows_per_tile, num_cols) + beta.broadcast_to(rows_per_tile, num_cols),
                           out_gm, offsets=[i, 0])
        return layer_norm_kernel

    def setup_device(self, dev):
        self.x, self.gamma, self.beta = self.make(self.R, dev)
        self.out = torch.empty_like(self.x)
        self.k = self.kernel()
        self.plan(lambda: self.k[148](self.x, self.gamma, self.beta, self.out, self.R, self.C, 4, self.EPS), self.k,
                  {0: self.x, 1: self.gamma, 2: self.beta, 3: self.out})

    def setup_host(self, lo, hi):
        x, gamma, beta = self.make(hi - lo)
        self.hx, self.hgamma, self.hbeta = x.pin_memory(), gamma.pin_memory(), beta.pin_memory()
        self.hout = torch.empty_like(self.hx).pin_memory()
        if not hasattr(self, "k"):
            self.k = self.kernel()

    def e2e_step(self):
        self.k[148](self.hx, self.hgamma, self.hbeta, self.hout, self.hx.shape[0], self.C, 4, self.EPS)

    def cpu_sample(self):
        if not hasattr(self, "cx"):
            self.cx, cg, cb = self.make(self.CPU_R)
            self.cg, self.cb = cg[0], cb[0]
        _ = torch.nn.functional.layer_norm(self.cx, (self.C, ), self.cg, self.cb, self.EPS)
        return 2.0 * 4 * self.CPU_R * self.C


class LeakyReluBF16(_Planned):
    name, label, dtype = "leaky_relu_bf16", "leaky_relu_bf16_2^28", "bf16"
    N = 1 << 28
    units, granule, axis = N, 1 << 16, "elements"
    work = 2.0 * 2 * N
    h2d_bytes, d2h_bytes = 2 * N, 2 * N
    CPU_N = 1 << 26
    cpu_sample_desc = "torch.where(x >= 0, x, x * alpha) on 2^26 of the 2^28 bf16 elements"

    def make_x(self, n, device="cpu"):
        return (torch.rand(n, device=device, generator=seeded(device)) * 10 - 5).to(torch.bfloat16)

    def setup_device(self, dev):
        from pyasc_b200 import tutorials as T
        self.x = self.make_x(self.N, dev)
        self.out = torch.empty_like(self.x)
        self.alpha = torch.tensor(0.1, dtype=torch.bfloat16)
        self.plan(lambda: T.leaky_relu_launch(self.x, self.alpha, self.out, core_num=148, tile_size=1 << 16),
                  T.leaky_relu_kernel, {0: self.x, 2: self.out})

    def setup_host(self, lo, hi):
        self.hx = self.make_x(hi - lo).pin_memory()
        self.hout = torch.empty_like(self.hx).pin_memory()
        self.alpha = torch.tensor(0.1, dtype=torch.bfloat16)

    def e2e_step(self):
        from pyasc_b200 import tutorials as T
        T.leaky_relu_launch(self.hx, self.alpha, self.hout, core_num=148, tile_size=1 << 16)

    def cpu_sample(self):
        if not hasattr(self, "cx"):
            self.cx = self.make_x(self.CPU_N)
        _ = torch.where(self.cx >= 0, self.cx, self.cx * torch.tensor(0.1, dtype=torch.bfloat16))
        return 2.0 * 2 * self.CPU_N


REGISTRY = {w.name: w for w in (Softmax, VAdd, GemmF16, GemmI8, GemmI8Dequant, Attention, AttentionCausal, Gelu, GeluTanh,
                                LeakyReluBF16, Mish, RowSum, RmsNorm, LayerNorm)}


# ---------------------------------------------------------------------------------------------------
# measurement
# ---------------------------------------------------------------------------------------------------
class Dist:
    """torch.distributed plumbing for the multi-rank run (one rank per GPU under torchrun)."""

    def __init__(self, n_gpus: int):
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        if n_gpus > 1 and self.world != n_gpus:
            raise SystemExit(f"--gpus {n_gpus} needs torchrun with {n_gpus} ranks (WORLD_SIZE={self.world})")
        self.enabled = self.world > 1

    def init(self, backend: str) -> None:
        if self.enabled:
            import torch.distributed as dist
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            kwargs = {"device_id": torch.device("cuda", self.local_rank)} if backend == "nccl" else {}
            dist.init_process_group(backend, rank=self.rank, world_size=self.world, **kwargs)

    def barrier(self) -> None:
        if self.enabled:
            import torch.distributed as dist
            dist.barrier()

    def max_over_ranks(self, value: float, device) -> float:
        if not self.enabled:
            return value
        import torch.distributed as dist
        t = torch.tensor([value], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def shutdown(self) -> None:
        if self.enabled:
            import torch.distributed as dist
            dist.destroy_process_group()


def checked_launch(w: Workload, lib, stream, lo: int, hi: int) -> None:
    from pyasc_b200 import capi
    rc = w.launch_units(lib, stream, lo, hi)
    if rc != 0:
        raise RuntimeError(f"{w.name}: C-ABI call returned {rc} ({capi.status_string(rc)}: {capi.last_cuda_error()})")


def time_device(w: Workload, lib, steps: int, warmup: int, dist: Dist, dev, slices: List[tuple],
                use_graph: bool) -> Dict[str, Any]:
    """Milliseconds per step.  Step i launches the C-ABI call(s) for `slices[i % len(slices)]`.  After the warm-up
    the `steps` timed launches are recorded into one CUDA graph (on torch's current stream, whose handle the C
    ABI receives) between two event-record nodes, and the graph is replayed once: the time is what those two events
    of the launching stream measure, first launch to last, so that the host's launch cost, which would dominate the
    short kernels of a 1/8 shard, stays out of the device time (where the graph cannot hold event nodes, two events
    around the replay); without graph support the same launches are issued back to back.  Barrier + synchronize on both sides, max over ranks."""
    from pyasc_b200 import capi
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for i in range(max(warmup, 3)):
        checked_launch(w, lib, stream, *slices[i % len(slices)])
    capi.check_device_status(stream)
    graph = None
    inner = None          # events recorded by nodes of the graph itself: first launch's start to last launch's end
    if use_graph:
        try:
            g = torch.cuda.CUDAGraph()
            try:
                first, last = (torch.cuda.Event(enable_timing=True, external=True) for _ in range(2))
            except TypeError:                      # this torch has no external events: time around the replay
                first = last = None
            with torch.cuda.graph(g):
                cap = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
                if first is not None:
                    first.record()
                for i in range(steps):
                    checked_launch(w, lib, cap, *slices[i % len(slices)])
                if last is not None:
                    last.record()
            g.replay()                             # one untimed replay: the graph's upload
            torch.cuda.synchronize()
            graph = g
            inner = (first, last) if first is not None else None
        except Exception as e:                     # capture refused: time eager launches instead
            print(f"[bench] {w.name}: CUDA graph capture failed ({e}); timing eager launches", file=sys.stderr)
            torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dist.barrier()
    torch.cuda.synchronize()
    start.record()
    if graph is not None:
        graph.replay()
    else:
        for i in range(steps):
            w.launch_units(lib, stream, *slices[i % len(slices)])
    stop.record()
    torch.cuda.synchronize()
    dist.barrier()
    ms = start.elapsed_time(stop) / steps
    if inner is not None:
        try:
            # the same K launches between two event nodes of the graph: the host's one graph launch stays outside
            ms_inner = inner[0].elapsed_time(inner[1]) / steps
            if 0 < ms_inner <= ms:
                ms = ms_inner
        except RuntimeError:
            pass
    capi.check_device_status(stream)
    used_graph = graph is not None
    del graph
    return {"ms": dist.max_over_ranks(ms, dev), "graph": used_graph}


NOMINAL = {"hbm": 8000.0, "tensor": 2250.0}     # B200 datasheet: 8 TB/s HBM3e, 2.25 PFLOP/s dense fp16/bf16


def time_sustained(w: Workload, lib, seconds: float, ms_per_launch: float) -> Dict[str, Any]:
    """Throughput over a loop of at least `seconds` of back-to-back launches of the whole configuration (the power
    cap pulls the clock down within about a second, so a tensor-bound kernel settles below its burst rate)."""
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    n = max(8, int(seconds * 1e3 / max(ms_per_launch, 1e-3)))
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for _ in range(n):
        w.launch_units(lib, stream, 0, w.units)
    stop.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop) / n
    return {"launches": n, "ms_per_step": round(ms, 5), "value": round(w.throughput(w.work, ms * 1e-3), 2)}


def time_e2e(w: Workload, steps: int, dist: Dist, dev) -> float:
    """Seconds per step through the public asc2 surface with pinned host tensors (the launcher copies
    in, launches, copies out and synchronises before returning)."""
    w.e2e_step()                                   # warm-up: tracing, plan cache, device buffer pool
    w.e2e_step()
    dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        w.e2e_step()
    torch.cuda.synchronize()
    sec = (time.perf_counter() - t0) / steps
    dist.barrier()
    return dist.max_over_ranks(sec, dev)


def host_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def time_cpu(w: Workload, steps: int, warmup: int) -> Dict[str, Any]:
    # torchrun exports OMP_NUM_THREADS=1 to its ranks: the CPU arm takes every core it may run on
    torch.set_num_threads(host_threads())
    for _ in range(warmup):
        w.cpu_sample()
    best = float("inf")
    work = 0.0
    for _ in range(steps):
        t0 = time.perf_counter()
        work = w.cpu_sample()
        best = min(best, time.perf_counter() - t0)
    return {"value": round(w.throughput(work, best), 4), "unit": w.unit, "cores": torch.get_num_threads(),
            "kind": "reference", "sample": w.cpu_sample_desc, "seconds_per_sample": round(best, 4),
            "host_cpus": os.cpu_count()}


def time_gather(w: Workload, lib, dist: Dist, own: tuple) -> Dict[str, float]:
    """The NCCL all-gather that reassembles the output on every rank, in place on the full-size output (every
    rank's shard already sits at its slot): alone, and right after the kernel that produces this rank's shard."""
    from pyasc_b200 import sharding
    out = w.output()
    lo, hi = own
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def gather():
        sharding.all_gather_in_place(out, w.units, dist.world, w.granule)

    def timed(fn, reps=3):
        fn()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dist.barrier()
        torch.cuda.synchronize()
        start.record()
        for _ in range(reps):
            fn()
        stop.record()
        torch.cuda.synchronize()
        return dist.max_over_ranks(start.elapsed_time(stop) / reps, out.device)

    def both():
        checked_launch(w, lib, stream, lo, hi)
        gather()

    return {"allgather_ms": timed(gather), "compute_plus_allgather_ms": timed(both)}


def time_overlapped_gather(w: Workload, lib, dist: Dist, own: tuple, chunks: int = 4) -> Optional[float]:
    """Milliseconds for the shard's kernel in `chunks` pieces with each piece's all-gather started as soon as
    the piece is enqueued (pyasc_b200.sharding.compute_and_gather): kernel and NCCL traffic overlap."""
    from pyasc_b200 import sharding
    lo0, hi0 = own
    out = w.output()
    if out.shape[0] != w.units or (hi0 - lo0) * dist.world != w.units:
        return None
    local = out[lo0:hi0]
    full = torch.empty_like(out)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def compute(lo, hi):
        checked_launch(w, lib, stream, lo0 + lo, lo0 + hi)

    sharding.compute_and_gather(compute, local, full, dist.world, chunks)
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dist.barrier()
    start.record()
    for _ in range(3):
        sharding.compute_and_gather(compute, local, full, dist.world, chunks)
    stop.record()
    torch.cuda.synchronize()
    ms = dist.max_over_ranks(start.elapsed_time(stop) / 3, local.device)
    del full
    return ms


def sharding_note(w, world: int) -> str:
    if world <= 1:
        return "one GPU: the whole configuration"
    return (f"the one {w.label} configuration split {world} ways along its {w.axis} ({w.units // world} per rank), inputs "
            "resident, no data-path collective; the NCCL all-gather that reassembles the output is timed separately")


SUMMARY_KEYS = ["value", "unit", "frac_of_measured_peak", "sustained_frac", "e2e_value", "cpu_value", "speedup_vs_one_gpu"]


def summarise(results: Dict[str, Dict[str, Any]]) -> Dict[str, Any]:
    """One short row per workload (SUMMARY_KEYS order), so that the tail of the line alone carries every
    configuration's throughput, roofline fraction, end-to-end and CPU figures."""
    rows = {}
    for name, r in results.items():
        rows[name] = [r["value"], r["unit"], r["roofline"]["frac"], (r.get("sustained") or {}).get("frac"),
                      (r.get("e2e") or {}).get("value"), (r.get("cpu_baseline") or {}).get("value"),
                      r.get("speedup_vs_one_gpu")]
    return {"keys": SUMMARY_KEYS, "rows": rows}


def run_ours(args) -> Dict[str, Any]:
    dist = Dist(args.gpus)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the CUDA platform has no CPU fallback")
    torch.cuda.set_device(dist.local_rank)
    dev = torch.device("cuda", dist.local_rank)
    dist.init("nccl")
    import pyasc_b200  # noqa: F401
    import asc
    from pyasc_b200 import capi, sharding
    lib = capi.load()
    asc.runtime.config.set_platform("CUDA", device_id=dist.local_rank)
    peaks = load_peaks()
    names = args.workloads
    sampler = ClockSampler(dist.local_rank)
    results: Dict[str, Dict[str, Any]] = {}
    launches_before = capi.launch_count()
    timed_launches = 0
    sampler.start()
    for name in names:
        w: Workload = REGISTRY[name]()
        w.setup_device(dev)
        n0 = capi.launch_count()
        ranges = sharding.all_shard_ranges(w.units, dist.world, w.granule)
        own = ranges[dist.rank]
        # step i: this rank's turn at shard (rank + i) mod N -- every step is one pass over the configuration
        slices = sharding.rotated_shards(w.units, dist.world, dist.rank, w.granule)
        timing = time_device(w, lib, args.steps, args.warmup, dist, dev, slices, not args.no_graph)
        ms = timing["ms"]
        timed_launches += args.steps
        whole_job = w.throughput(w.work, ms * 1e-3)
        per_gpu = whole_job / dist.world
        peak = w.peak(peaks)
        i8 = name.startswith("gemm_i8")
        res: Dict[str, Any] = {
            "workload": w.label, "value": round(whole_job, 2), "unit": w.unit, "ms_per_step": round(ms, 5),
            "dtype": w.dtype, "cuda_graph": timing["graph"],
            "roofline": {"bound": w.bound, "achieved": round(per_gpu, 2), "peak": round(peak, 1),
                         "unit": w.unit, "frac": round(per_gpu / peak, 4), "traffic": None,
                         "peak_source": peaks["source"] + (" (2 x bf16 burst)" if i8 else
                                                           " (bf16 burst)" if w.bound == "tensor" else " (copy)")},
        }
        res["roofline"]["nominal_peak"] = NOMINAL[w.bound] * (2 if i8 else 1)
        res["roofline"]["frac_of_nominal"] = round(per_gpu / res["roofline"]["nominal_peak"], 4)
        if dist.enabled:
            res["sharding"] = {"axis": w.axis, "units": w.units, "units_per_rank": own[1] - own[0],
                               "replicated": list(w.replicated)}
            full = time_device(w, lib, args.steps, args.warmup, dist, dev, [(0, w.units)], not args.no_graph)["ms"]
            timed_launches += args.steps
            res["weak"] = {"note": "every rank runs the whole configuration on its own (replicas)",
                           "ms_per_step": round(full, 5), "value": round(w.throughput(w.work, full * 1e-3) * dist.world, 2)}
            res["speedup_vs_one_gpu"] = round(full / ms, 3)
            gathered = time_gather(w, lib, dist, own)
            res.update({k: round(v, 4) for k, v in gathered.items()})
            res["speedup_with_allgather"] = round(full / gathered["compute_plus_allgather_ms"], 3)
            if name in ("softmax", "vadd"):
                ov = time_overlapped_gather(w, lib, dist, own)
                if ov is not None:
                    res["overlapped_compute_and_allgather_ms"] = round(ov, 4)
        elif w.bound == "tensor" and args.sustained_seconds > 0:
            timed_launches_before = capi.launch_count()
            sus = time_sustained(w, lib, args.sustained_seconds, ms)
            timed_launches += capi.launch_count() - timed_launches_before
            sus_peak = float(peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"])) * (2 if i8 else 1)
            sus.update({"unit": w.unit, "peak": round(sus_peak, 1), "frac": round(sus["value"] / sus_peak, 4),
                        "peak_source": peaks["source"] + " (bf16 sustained" + (", x 2)" if i8 else ")")})
            res["sustained"] = sus
        if not args.no_e2e:
            w.setup_host(*own)
            e2e_steps = max(1, min(args.steps, args.e2e_steps))
            sec = time_e2e(w, e2e_steps, dist, dev)
            timed_launches += e2e_steps
            share = (own[1] - own[0]) / w.units
            res["e2e"] = {"value": round(w.throughput(w.work, sec), 3), "unit": w.unit,
                          "h2d_bytes_per_step": int((w.h2d_bytes - w.replicated_h2d_bytes) * share) + w.replicated_h2d_bytes,
                          "d2h_bytes_per_step": int(w.d2h_bytes * share),
                          "ms_per_step": round(sec * 1e3, 3), "steps": e2e_steps}
            if dist.enabled:
                res["e2e"]["bytes_are"] = "per rank"
        res["launches"] = capi.launch_count() - n0
        if dist.rank == 0 and dist.world == 1 and not args.no_cpu:
            res["cpu_baseline"] = time_cpu(w, 3, 1)
        results[name] = res
        del w
        torch.cuda.empty_cache()
        from asc.lib import runtime as rt
        rt.release_pool()
    clocks = sampler.stop()
    total_launches = capi.launch_count() - launches_before
    dist.shutdown()
    head_name = HEADLINE if HEADLINE in results else names[0]
    head = results[head_name]
    hw = REGISTRY[head_name]
    traffic = load_traffic()
    for name, res in results.items():
        if name in traffic and dist.world == 1:
            res["roofline"]["traffic"] = traffic[name]
    split = sharding_note(hw, dist.world)
    line = {
        "metric": "HBM GB/s (fp32 row softmax, whole job); per-kernel HBM GB/s and tensor TFLOP/s under 'workloads'",
        "value": head["value"], "unit": head["unit"], "n_gpus": dist.world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": head["dtype"], "data": "synthetic (seeded, shapes and distributions of the named configs)",
        "config": {"workload": head["workload"], "sharding": split},
        "method": {"l2": "inputs larger than L2 (126 MB); with N > 1 a rank takes another shard every step, so nothing it "
                   "reads is still in its L2",
                   "timing": "two CUDA event nodes inside one CUDA graph, before the first and after the last of the K launches; one replay; max over ranks"},
        "roofline": head["roofline"], "e2e": head.get("e2e"), "cpu_baseline": head.get("cpu_baseline"),
        "gpu_launches": total_launches + timed_launches, "gpu_launches_timed": timed_launches, "clocks": clocks,
        "workloads": results, "native_so_jit": [os.path.relpath(b, ROOT) for b in jit_builds()],
        "summary": summarise(results),
    }
    if args.summary_file and dist.rank == 0:
        with open(args.summary_file, "w") as f:
            json.dump({"n_gpus": dist.world, "steps": args.steps, "peaks": {k: peaks.get(k) for k in
                       ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained", "source")}, "clocks": clocks,
                       "summary": line["summary"]}, f, indent=1)
    return line if dist.rank == 0 else {}


def jit_builds() -> List[str]:
    """Libraries of kernels specialised at first use that this process built or loaded (pyasc_b200/jit.py)."""
    from pyasc_b200 import jit
    failed = jit.failures()
    if failed:
        print(f"[bench] {len(failed)} specialised kernels failed to build: {list(failed.values())[0][:400]}", file=sys.stderr)
    return list(jit.builds)


def load_traffic() -> Dict[str, float]:
    """DRAM bytes per launch from the committed ncu summaries (profiles/dram_traffic.json)."""
    path = os.path.join(ROOT, "profiles", "dram_traffic.json")
    if not os.path.exists(path):
        return {}
    with open(path) as f:
        return {k: v for k, v in json.load(f).items() if isinstance(v, (int, float))}


def run_reference(args) -> Dict[str, Any]:
    """The reference's CPU computation of the path (its tests' torch expressions), all host threads."""
    if int(os.environ.get("RANK", "0")) != 0:
        return {}
    results = {}
    for name in args.workloads:
        w: Workload = REGISTRY[name]()
        steps = args.steps if name == HEADLINE else min(args.steps, 3)
        results[name] = time_cpu(w, max(1, steps), max(1, min(args.warmup, 2)))
        results[name]["workload"] = w.label
        del w
    head_name = HEADLINE if HEADLINE in results else args.workloads[0]
    head = results[head_name]
    w = REGISTRY[head_name]
    return {
        "impl": "reference",
        "metric": "HBM GB/s (fp32 row softmax, whole job); per-kernel HBM GB/s and tensor TFLOP/s under 'workloads'",
        "value": head["value"], "unit": head["unit"], "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(head["seconds_per_sample"] * 1e3, 3), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": w.dtype, "data": "synthetic (seeded, shapes and distributions of the named configs)",
        "config": {"workload": w.label, "sharding": sharding_note(w, args.gpus)},
        "method": {"note": "CPU arm: the torch expressions of the reference's tests on the host cores of rank 0, each step a "
                   "bounded sample of the configuration (cpu_baseline.sample)"},
        "cpu_baseline": head,
        "e2e": {"value": head["value"], "unit": head["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "workloads": results,
        "summary": {"keys": ["value", "unit"], "rows": {n: [r["value"], r["unit"]] for n, r in results.items()}},
    }


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--sustained-seconds", type=float, default=2.0,
                    help="length of the extra sustained loop for tensor-bound workloads at one GPU (0: skip)")
    ap.add_argument("--workloads", type=lambda s: s.split(","), default=ALL_WORKLOADS,
                    help="comma-separated subset of: " + ",".join(ALL_WORKLOADS))
    ap.add_argument("--e2e-steps", type=int, default=5, help="timed end-to-end steps per workload (<= --steps)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-graph", action="store_true", help="time eager back-to-back launches instead of a CUDA graph")
    ap.add_argument("--summary-file", default=None, help="also write the per-workload summary table to this JSON file")
    args = ap.parse_args()
    unknown = [n for n in args.workloads if n not in REGISTRY]
    if unknown:
        raise SystemExit(f"unknown workloads: {unknown}")
    # Libraries (NCCL's version banner, for one) write to stdout; the contract is ONE JSON line there.
    # Everything else goes to stderr: stdout is parked on a duplicate descriptor until the line is ready.
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    try:
        line = run_reference(args) if args.impl == "reference" else run_ours(args)
    finally:
        sys.stdout.flush()
        os.dup2(real_stdout, 1)
        os.close(real_stdout)
    if line:
        print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
