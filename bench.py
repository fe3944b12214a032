#!/usr/bin/env python
"""Benchmark of the five hot-path kernels on B200: HBM GB/s and tensor TFLOP/s per GPU against the
measured roofline, next to the same computation on the host CPU.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workloads a,b,...]

One JSON line on stdout (rank 0).  The headline workload is the fp32 row softmax [16384, 4096]; the
other four workloads (vadd 2^28, fp16 GEMM 8192^3, int8 GEMM 8192^3 with dequant, attention forward
[4,32,4096,128] non-causal and causal) are reported under "workloads" with the same sub-keys.

value      device-resident throughput: K back-to-back C-ABI launches timed with CUDA events on the
           launching stream (max over ranks), algorithmic bytes or FLOPs per launch / time.
e2e        the same metric through the public asc2 surface (`kernel[cores](host tensors)`): pinned host
           tensors in, host tensor out, H2D and D2H copies inside the timed region.
roofline   achieved (= value per GPU) over the measured peak from MEASURED_PEAKS.json.
cpu_baseline / --impl reference
           the reference's own CPU computation of the path (the torch expressions its tests assert
           against, oracle/golden.py) timed on a bounded sample with all host threads.

Multi-GPU (launched under torchrun, one rank per GPU): weak scaling, every rank runs the full
single-GPU workload on its own shard; there is no data-path collective.  The output all-gather over
NCCL is timed separately and reported as "allgather_ms".
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
                 "gelu", "gelu_tanh", "leaky_relu_bf16", "mish_interpreted", "row_sum", "rms_norm", "layer_norm"]

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
# workloads
# ---------------------------------------------------------------------------------------------------
def P(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


class Workload:
    """One benchmarked configuration.  `work` is algorithmic bytes (HBM-bound) or FLOPs (tensor-bound)
    per launch; `units` names what a launch processes."""
    name = ""
    label = ""
    unit = "GB/s"
    bound = "hbm"
    dtype = "f32"
    work = 0.0
    h2d_bytes = 0
    d2h_bytes = 0

    def setup_device(self, dev: torch.device) -> None: ...
    def launch(self, lib, stream) -> int: ...
    def setup_host(self) -> None: ...
    def e2e_step(self) -> None: ...
    def cpu_sample(self) -> float: ...          # runs the bounded CPU sample once, returns its work
    cpu_sample_desc = ""

    def throughput(self, work: float, seconds: float) -> float:
        return work / seconds / (1e9 if self.unit == "GB/s" else 1e12)

    def peak(self, peaks: Dict[str, Any]) -> float:
        return float(peaks["hbm_gbs"]) if self.bound == "hbm" else float(peaks["bf16_tflops"])


class Softmax(Workload):
    name, label, dtype = "softmax", "softmax_f32_16384x4096", "f32"
    R, C = 16384, 4096
    work = 2.0 * 4 * R * C                      # one 4-byte read + one 4-byte write per element
    h2d_bytes, d2h_bytes = 4 * R * C, 4 * R * C
    cpu_sample_desc = "torch.softmax(x, -1) on the full [16384, 4096] input"

    def setup_device(self, dev):
        from oracle import golden as G
        self.x = G.softmax_input(self.R, self.C).to(dev)
        self.out = torch.empty_like(self.x)

    def launch(self, lib, stream):
        return lib.asc_cuda_softmax_f32(P(self.x), P(self.out), self.R, self.C, self.C, stream)

    def launch_range(self, lib, stream, lo, hi):      # rows [lo, hi) of this rank's shard
        return lib.asc_cuda_softmax_f32(P(self.x[lo:hi]), P(self.out[lo:hi]), hi - lo, self.C, self.C, stream)

    def setup_host(self):
        from oracle import golden as G
        self.hx = G.softmax_input(self.R, self.C).pin_memory()
        self.hout = torch.empty_like(self.hx).pin_memory()

    def e2e_step(self):
        from pyasc_b200 import tutorials as T
        T.softmax_launch(self.hx, self.hout, core_num=148)

    def cpu_sample(self):
        if not hasattr(self, "cx"):
            from oracle import golden as G
            self.cx = G.softmax_input(self.R, self.C)
        from oracle import golden as G
        G.softmax(self.cx)
        return self.work


class VAdd(Workload):
    name, label, dtype = "vadd", "vadd_f32_2^28", "f32"
    N = 1 << 28
    work = 3.0 * 4 * N
    h2d_bytes, d2h_bytes = 2 * 4 * N, 4 * N
    CPU_N = 1 << 26
    cpu_sample_desc = "x + y on 2^26 of the 2^28 elements"

    def setup_device(self, dev):
        g = torch.Generator(device=dev).manual_seed(2026)
        self.x = torch.rand(self.N, device=dev, generator=g)
        self.y = torch.rand(self.N, device=dev, generator=g)
        self.out = torch.empty_like(self.x)

    def launch(self, lib, stream):
        return lib.asc_cuda_vadd_f32(P(self.x), P(self.y), P(self.out), self.N, stream)

    def launch_range(self, lib, stream, lo, hi):      # elements [lo, hi) of this rank's shard
        return lib.asc_cuda_vadd_f32(P(self.x[lo:hi]), P(self.y[lo:hi]), P(self.out[lo:hi]), hi - lo, stream)

    def setup_host(self):
        g = torch.Generator().manual_seed(2026)
        self.hx = torch.rand(self.N, generator=g).pin_memory()
        self.hy = torch.rand(self.N, generator=g).pin_memory()
        self.hout = torch.empty(self.N).pin_memory()

    def e2e_step(self):
        from pyasc_b200 import tutorials as T
        T.vadd_launch(self.hx, self.hy, self.hout, core_num=148, tile_size=1 << 16)

    def cpu_sample(self):
        if not hasattr(self, "cx"):
            from oracle import golden as G
            self.cx, self.cy = G.vadd_inputs(self.CPU_N)
        from oracle import golden as G
        G.vadd(self.cx, self.cy)
        return 3.0 * 4 * self.CPU_N


class GemmF16(Workload):
    name, label, dtype, unit, bound = "gemm_f16", "gemm_f16_8192x8192x8192_f32acc_f16out", "f16", "TFLOP/s", "tensor"
    M = N = K = 8192
    work = 2.0 * M * N * K
    h2d_bytes, d2h_bytes = 2 * (M * K + K * N), 2 * M * N
    CPU_M = 1024
    cpu_sample_desc = "(A.float() @ B.float()).half() on 1024 of the 8192 rows of A"

    def setup_device(self, dev):
        from oracle import golden as G
        a, b = G.gemm_f16_inputs(self.M, self.N, self.K)
        self.a, self.b = a.to(dev), b.to(dev)
        self.c = torch.empty(self.M, self.N, dtype=torch.float16, device=dev)

    def launch(self, lib, stream):
        return lib.asc_cuda_gemm_f16(P(self.a), P(self.b), P(self.c), self.M, self.N, self.K, self.K, self.N, self.N,
                                     0, 0, 0, stream)

    def setup_host(self):
        from oracle import golden as G
        a, b = G.gemm_f16_inputs(self.M, self.N, self.K)
        self.ha, self.hb = a.pin_memory(), b.pin_memory()
        self.hc = torch.empty(self.M, self.N, dtype=torch.float16).pin_memory()

    def e2e_step(self):
        from pyasc_b200 import tutorials as T
        T.matmul_fp16_launch(self.ha, self.hb, self.hc, core_num=148)

    def cpu_sample(self):
        from oracle import golden as G
        if not hasattr(self, "ca"):
            a, b = G.gemm_f16_inputs(self.CPU_M, self.N, self.K)
            self.ca, self.cb = a, b
        G.gemm_f16(self.ca, self.cb)
        return 2.0 * self.CPU_M * self.N * self.K


class GemmI8(Workload):
    name, label, dtype, unit, bound = "gemm_i8", "gemm_i8_8192x8192x8192_int32out", "s8", "TFLOP/s", "tensor"
    M = N = K = 8192
    work = 2.0 * M * N * K
    h2d_bytes, d2h_bytes = M * K + K * N, 4 * M * N
    CPU_M = 256
    dequant = False
    cpu_sample_desc = "A.int32 @ B.int32 (evaluated exactly in fp64) on 256 of the 8192 rows of A"

    def peak(self, peaks):
        return 2.0 * float(peaks["bf16_tflops"])    # dense int8 runs at twice the 16-bit rate

    def setup_device(self, dev):
        from oracle import golden as G
        a, b, sa, sb = G.gemm_i8_inputs(self.M, self.N, self.K)
        self.a, self.b, self.sa, self.sb = a.to(dev), b.to(dev), sa.to(dev), sb.to(dev)
        self.acc = None if self.dequant else torch.empty(self.M, self.N, dtype=torch.int32, device=dev)
        self.deq = torch.empty(self.M, self.N, dtype=torch.float16, device=dev) if self.dequant else None

    def launch(self, lib, stream):
        return lib.asc_cuda_gemm_i8(P(self.a), P(self.b), P(self.acc), P(self.deq),
                                    P(self.sa) if self.dequant else None, P(self.sb) if self.dequant else None,
                                    self.M, self.N, self.K, self.K, self.N, self.N, stream)

    def setup_host(self):
        from oracle import golden as G
        a, b, sa, sb = G.gemm_i8_inputs(self.M, self.N, self.K)
        self.ha, self.hb, self.hsa, self.hsb = a.pin_memory(), b.pin_memory(), sa.pin_memory(), sb.pin_memory()
        self.hacc = torch.empty(self.M, self.N, dtype=torch.int32).pin_memory() if not self.dequant else None
        self.hdeq = torch.empty(self.M, self.N, dtype=torch.float16).pin_memory() if self.dequant else None

    def e2e_step(self):
        from pyasc_b200 import tutorials as T
        if self.dequant:
            T.matmul_int8_dequant_launch(self.ha, self.hb, self.hsa, self.hsb, self.hdeq, core_num=148)
        else:
            T.matmul_int8_launch(self.ha, self.hb, self.hacc, core_num=148)

    def cpu_sample(self):
        from oracle import golden as G
        if not hasattr(self, "ca"):
            self.ca, self.cb, self.csa, self.csb = G.gemm_i8_inputs(self.CPU_M, self.N, self.K)
        acc = G.gemm_i8(self.ca, self.cb)
        if self.dequant:
            G.dequant(acc, self.csa, self.csb)
        return 2.0 * self.CPU_M * self.N * self.K


class GemmI8Dequant(GemmI8):
    name, label = "gemm_i8_dequant", "gemm_i8_8192x8192x8192_dequant_f16out"
    dequant = True
    d2h_bytes = 2 * GemmI8.M * GemmI8.N
    h2d_bytes = GemmI8.h2d_bytes + 4 * (GemmI8.M + GemmI8.N)
    cpu_sample_desc = "A.int32 @ B.int32 then acc * a_scale[row] * b_scale[col] -> fp16 on 256 of the 8192 rows"


class Attention(Workload):
    name, label, dtype, unit, bound = "attention", "attention_fwd_f16_b4_h32_s4096_d128", "f16", "TFLOP/s", "tensor"
    B, H, S, D = 4, 32, 4096, 128
    causal = False
    work = 4.0 * B * H * S * S * D
    h2d_bytes, d2h_bytes = 3 * 2 * B * H * S * D, 2 * B * H * S * D
    CPU_HEADS = 2
    cpu_sample_desc = "fp32 softmax(QK^T*scale)V on 2 of the 128 (batch, head) pairs"

    def setup_device(self, dev):
        from oracle import golden as G
        q, k, v = G.attention_inputs(self.B, self.H, self.S, self.D)
        self.q, self.k, self.v = q.to(dev), k.to(dev), v.to(dev)
        self.o = torch.empty_like(self.q)

    def launch(self, lib, stream):
        return lib.asc_cuda_attn_fwd_f16(P(self.q), P(self.k), P(self.v), P(self.o), self.B, self.H, self.S, self.D,
                                         ctypes.c_float(self.D ** -0.5), int(self.causal), 0, stream)

    def setup_host(self):
        from oracle import golden as G
        q, k, v = G.attention_inputs(self.B, self.H, self.S, self.D)
        self.hq, self.hk, self.hv = q.pin_memory(), k.pin_memory(), v.pin_memory()
        self.ho = torch.empty_like(q).pin_memory()

    def e2e_step(self):
        from pyasc_b200 import tutorials as T
        T.attention_launch(self.hq, self.hk, self.hv, self.ho, causal=self.causal, core_num=148)

    def cpu_sample(self):
        from oracle import golden as G
        if not hasattr(self, "cq"):
            self.cq, self.ck, self.cv = G.attention_inputs(1, self.CPU_HEADS, self.S, self.D)
        G.attention(self.cq, self.ck, self.cv, self.causal)
        return self.work * self.CPU_HEADS / (self.B * self.H)


class AttentionCausal(Attention):
    name, label = "attention_causal", "attention_fwd_f16_b4_h32_s4096_d128_causal"
    causal = True
    work = Attention.work / 2                    # the usual convention: masked half not counted
    cpu_sample_desc = "fp32 causal softmax(QK^T*scale + mask)V on 2 of the 128 (batch, head) pairs"


class _Elementwise(Workload):
    """An asc2 elementwise kernel: the device leg launches the C-ABI call the launcher plans for it (the
    plan is built once, with the launch itself suppressed), the end-to-end leg goes through the kernel
    launch a user writes."""

    def plan_step(self, launch_fn, kernel, ptr_args):
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
        assert plan.pattern in ("elementwise:program", "row:program") and len(plan.steps) == 1, plan
        self.step = plan.steps[0]
        self.ptrs = {i: t.data_ptr() for i, t in ptr_args.items()}

    def launch(self, lib, stream):
        return getattr(lib, self.step.fn_name)(*self.step.build(self.ptrs, stream))


class Gelu(_Elementwise):
    name, label, dtype = "gelu", "gelu_erf_f32_16384x4096", "f32"
    approximate = False
    R, C = 16384, 4096
    work = 2.0 * 4 * R * C
    h2d_bytes, d2h_bytes = 4 * R * C, 4 * R * C
    CPU_R = 4096
    cpu_sample_desc = "0.5*x*(1+erf(x/sqrt(2))) in torch on 4096 of the 16384 rows"

    def setup_device(self, dev):
        from pyasc_b200 import tutorials as T
        g = torch.Generator(device=dev).manual_seed(2026)
        self.x = torch.rand((self.R, self.C), device=dev, generator=g) * 6 - 3
        self.out = torch.empty_like(self.x)
        self.plan_step(lambda: T.gelu_launch(self.x, self.out, self.approximate, core_num=148), T.gelu_kernel,
                       {0: self.x, 1: self.out})

    def setup_host(self):
        g = torch.Generator().manual_seed(2026)
        self.hx = (torch.rand((self.R, self.C), generator=g) * 6 - 3).pin_memory()
        self.hout = torch.empty_like(self.hx).pin_memory()

    def e2e_step(self):
        from pyasc_b200 import tutorials as T
        T.gelu_launch(self.hx, self.hout, self.approximate, core_num=148)

    def cpu_sample(self):
        import math
        if not hasattr(self, "cx"):
            self.cx = torch.rand((self.CPU_R, self.C), generator=torch.Generator().manual_seed(2026)) * 6 - 3
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


class MishInterpreted(Gelu):
    """x * tanh(log(exp(x) + 1)): an expression without a compiled instance, so the interpreter runs it."""
    name, label = "mish_interpreted", "mish_f32_16384x4096_interpreter"
    cpu_sample_desc = "x * tanh(log(exp(x) + 1)) in torch on 4096 of the 16384 rows"

    @staticmethod
    def kernel():
        import pyasc_b200  # noqa: F401  (makes `asc` / `asc2` importable)
        import asc
        import asc2

        @asc2.jit
        def mish_kernel(x_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, num_rows: asc.ConstExpr,
                        num_columns: asc.ConstExpr):
            x_gm = asc2.tensor(x_ptr, [num_rows, num_columns])
            out_gm = asc2.tensor(out_ptr, [num_rows, num_columns])
            for i in range(asc2.block_idx(), num_rows, asc2.block_num()):
                row = asc2.load(x_gm, [1, num_columns], offsets=[i, 0])
                asc2.store(row * asc2.tanh(asc2.log(asc2.exp(row) + 1)), out_gm, offsets=[i, 0])
        return mish_kernel

    def setup_device(self, dev):
        g = torch.Generator(device=dev).manual_seed(2026)
        self.x = torch.rand((self.R, self.C), device=dev, generator=g) * 6 - 3
        self.out = torch.empty_like(self.x)
        self.k = self.kernel()
        self.plan_step(lambda: self.k[148](self.x, self.out, self.R, self.C), self.k, {0: self.x, 1: self.out})

    def e2e_step(self):
        if not hasattr(self, "k"):
            self.k = self.kernel()
        self.k[148](self.hx, self.hout, self.R, self.C)

    def cpu_sample(self):
        if not hasattr(self, "cx"):
            self.cx = torch.rand((self.CPU_R, self.C), generator=torch.Generator().manual_seed(2026)) * 6 - 3
        _ = self.cx * torch.tanh(torch.log(torch.exp(self.cx) + 1))
        return 2.0 * 4 * self.CPU_R * self.C


class RowSum(Workload):
    """asc2.reduce_sum over the rows of [65536, 4096] fp32 (1 GiB read, 256 KiB written)."""
    name, label, dtype = "row_sum", "row_sum_f32_65536x4096", "f32"
    R, C = 65536, 4096
    work = 4.0 * R * C + 4.0 * R
    h2d_bytes, d2h_bytes = 4 * R * C, 4 * R
    CPU_R = 16384
    cpu_sample_desc = "x.sum(1) in torch on 16384 of the 65536 rows"

    def setup_device(self, dev):
        g = torch.Generator(device=dev).manual_seed(2026)
        self.x = torch.randn((self.R, self.C), device=dev, generator=g)
        self.out = torch.empty(self.R, device=dev)

    def launch(self, lib, stream):
        return lib.asc_cuda_reduce_f32(P(self.x), P(self.out), self.R, self.C, self.C, 1, 0, 1, stream)

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

    def setup_host(self):
        g = torch.Generator().manual_seed(2026)
        self.hx = torch.randn((self.R, self.C), generator=g).pin_memory()
        self.hout = torch.empty(self.R).pin_memory()
        self.k = self.kernel()

    def e2e_step(self):
        self.k[148](self.hx, self.hout, self.R, self.C, 8)

    def cpu_sample(self):
        if not hasattr(self, "cx"):
            self.cx = torch.randn((self.CPU_R, self.C), generator=torch.Generator().manual_seed(2026))
        _ = self.cx.sum(1)
        return 4.0 * self.CPU_R * self.C


class RmsNorm(Workload):
    """asc2.rms_norm over the rows of [16384, 4096] fp32 (256 MiB read, 256 MiB written, gamma resident)."""
    name, label, dtype = "rms_norm", "rms_norm_f32_16384x4096", "f32"
    R, C = 16384, 4096
    EPS = 1e-5
    work = 2.0 * 4 * R * C
    h2d_bytes, d2h_bytes = 4 * R * C + 4 * C, 4 * R * C
    CPU_R = 4096
    cpu_sample_desc = "x * rsqrt(mean(x^2, 1) + eps) * gamma in torch on 4096 of the 16384 rows"

    def setup_device(self, dev):
        g = torch.Generator(device=dev).manual_seed(2026)
        self.x = torch.randn((self.R, self.C), device=dev, generator=g)
        self.gamma = torch.rand((1, self.C), device=dev, generator=g) + 0.5
        self.out = torch.empty_like(self.x)

    def launch(self, lib, stream):
        return lib.asc_cuda_rms_norm_f32(P(self.x), P(self.gamma), P(self.out), self.R, self.C, self.C, self.EPS, stream)

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

    def setup_host(self):
        g = torch.Generator().manual_seed(2026)
        self.hx = torch.randn((self.R, self.C), generator=g).pin_memory()
        self.hgamma = (torch.rand((1, self.C), generator=g) + 0.5).pin_memory()
        self.hout = torch.empty_like(self.hx).pin_memory()
        self.k = self.kernel()

    def e2e_step(self):
        self.k[148](self.hx, self.hgamma, self.hout, self.R, self.C, 4, self.EPS)

    def cpu_sample(self):
        if not hasattr(self, "cx"):
            g = torch.Generator().manual_seed(2026)
            self.cx = torch.randn((self.CPU_R, self.C), generator=g)
            self.cg = torch.rand((1, self.C), generator=g) + 0.5
        _ = self.cx * torch.rsqrt(self.cx.pow(2).mean(1, keepdim=True) + self.EPS) * self.cg
        return 2.0 * 4 * self.CPU_R * self.C


class LayerNorm(_Elementwise):
    """Layer norm written with asc2 reductions and broadcasts (mean, centred variance, scale and shift): one row
    program over [16384, 4096] fp32 (256 MiB read, 256 MiB written; gamma and beta resident)."""
    name, label, dtype = "layer_norm", "layer_norm_f32_16384x4096_row_program", "f32"
    R, C = 16384, 4096
    EPS = 1e-5
    work = 2.0 * 4 * R * C
    h2d_bytes, d2h_bytes = 4 * R * C + 8 * C, 4 * R * C
    CPU_R = 4096
    cpu_sample_desc = "torch.nn.functional.layer_norm on 4096 of the 16384 rows"

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
        g = torch.Generator(device=dev).manual_seed(2026)
        self.x = torch.randn((self.R, self.C), device=dev, generator=g)
        self.gamma = torch.rand((1, self.C), device=dev, generator=g) + 0.5
        self.beta = torch.randn((1, self.C), device=dev, generator=g)
        self.out = torch.empty_like(self.x)
        self.k = self.kernel()
        self.plan_step(lambda: self.k[148](self.x, self.gamma, self.beta, self.out, self.R, self.C, 4, self.EPS), self.k,
                       {0: self.x, 1: self.gamma, 2: self.beta, 3: self.out})

    def setup_host(self):
        g = torch.Generator().manual_seed(2026)
        self.hx = torch.randn((self.R, self.C), generator=g).pin_memory()
        self.hgamma = (torch.rand((1, self.C), generator=g) + 0.5).pin_memory()
        self.hbeta = torch.randn((1, self.C), generator=g).pin_memory()
        self.hout = torch.empty_like(self.hx).pin_memory()
        if not hasattr(self, "k"):
            self.k = self.kernel()

    def e2e_step(self):
        self.k[148](self.hx, self.hgamma, self.hbeta, self.hout, self.R, self.C, 4, self.EPS)

    def cpu_sample(self):
        if not hasattr(self, "cx"):
            g = torch.Generator().manual_seed(2026)
            self.cx = torch.randn((self.CPU_R, self.C), generator=g)
            self.cg, self.cb = torch.rand(self.C, generator=g) + 0.5, torch.randn(self.C, generator=g)
        _ = torch.nn.functional.layer_norm(self.cx, (self.C, ), self.cg, self.cb, self.EPS)
        return 2.0 * 4 * self.CPU_R * self.C


class LeakyReluBF16(_Elementwise):
    name, label, dtype = "leaky_relu_bf16", "leaky_relu_bf16_2^28", "bf16"
    N = 1 << 28
    work = 2.0 * 2 * N
    h2d_bytes, d2h_bytes = 2 * N, 2 * N
    CPU_N = 1 << 26
    cpu_sample_desc = "torch.where(x >= 0, x, x * alpha) on 2^26 of the 2^28 bf16 elements"

    def setup_device(self, dev):
        from pyasc_b200 import tutorials as T
        g = torch.Generator(device=dev).manual_seed(2026)
        self.x = (torch.rand(self.N, device=dev, generator=g) * 10 - 5).to(torch.bfloat16)
        self.out = torch.empty_like(self.x)
        self.alpha = torch.tensor(0.1, dtype=torch.bfloat16)
        self.plan_step(lambda: T.leaky_relu_launch(self.x, self.alpha, self.out, core_num=148, tile_size=1 << 16),
                       T.leaky_relu_kernel, {0: self.x, 2: self.out})

    def setup_host(self):
        g = torch.Generator().manual_seed(2026)
        self.hx = (torch.rand(self.N, generator=g) * 10 - 5).to(torch.bfloat16).pin_memory()
        self.hout = torch.empty_like(self.hx).pin_memory()
        self.alpha = torch.tensor(0.1, dtype=torch.bfloat16)

    def e2e_step(self):
        from pyasc_b200 import tutorials as T
        T.leaky_relu_launch(self.hx, self.alpha, self.hout, core_num=148, tile_size=1 << 16)

    def cpu_sample(self):
        if not hasattr(self, "cx"):
            g = torch.Generator().manual_seed(2026)
            self.cx = (torch.rand(self.CPU_N, generator=g) * 10 - 5).to(torch.bfloat16)
        _ = torch.where(self.cx >= 0, self.cx, self.cx * torch.tensor(0.1, dtype=torch.bfloat16))
        return 2.0 * 2 * self.CPU_N


REGISTRY = {w.name: w for w in (Softmax, VAdd, GemmF16, GemmI8, GemmI8Dequant, Attention, AttentionCausal, Gelu, GeluTanh,
                                LeakyReluBF16, MishInterpreted, RowSum, RmsNorm, LayerNorm)}


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
            dist.init_process_group(backend, rank=self.rank, world_size=self.world)

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


def time_device(w: Workload, lib, steps: int, warmup: int, dist: Dist, dev) -> float:
    """Milliseconds per launch: `steps` back-to-back launches between two CUDA events on the launching
    (torch current) stream, barrier + synchronize on both sides, max over ranks."""
    from pyasc_b200 import capi
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for _ in range(max(warmup, 3)):
        rc = w.launch(lib, stream)
        if rc != 0:
            raise RuntimeError(f"{w.name}: C-ABI call returned {rc} ({capi.status_string(rc)}: {capi.last_cuda_error()})")
    capi.check_device_status(stream)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dist.barrier()
    torch.cuda.synchronize()
    start.record()
    for _ in range(steps):
        w.launch(lib, stream)
    stop.record()
    torch.cuda.synchronize()
    dist.barrier()
    ms = start.elapsed_time(stop) / steps
    capi.check_device_status(stream)
    return dist.max_over_ranks(ms, dev)


NOMINAL = {"hbm": 8000.0, "tensor": 2250.0}     # B200 datasheet: 8 TB/s HBM3e, 2.25 PFLOP/s dense fp16/bf16


def time_sustained(w: Workload, lib, seconds: float, ms_per_launch: float) -> Dict[str, Any]:
    """Throughput over a loop of at least `seconds` of back-to-back launches (the power cap pulls the clock
    down within about a second, so a tensor-bound kernel settles below its burst rate)."""
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    n = max(8, int(seconds * 1e3 / max(ms_per_launch, 1e-3)))
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for _ in range(n):
        w.launch(lib, stream)
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


def time_cpu(w: Workload, steps: int, warmup: int) -> Dict[str, Any]:
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


def time_allgather(w: Workload, dist: Dist) -> Optional[float]:
    """Milliseconds for the NCCL all-gather that reassembles this workload's output on every rank."""
    if not dist.enabled:
        return None
    import torch.distributed as tdist
    local = next(t for t in (getattr(w, "out", None), getattr(w, "c", None), getattr(w, "deq", None),
                             getattr(w, "acc", None), getattr(w, "o", None)) if t is not None)
    flat = local.reshape(-1)
    full = torch.empty(flat.numel() * dist.world, dtype=flat.dtype, device=flat.device)
    tdist.all_gather_into_tensor(full, flat)
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dist.barrier()
    start.record()
    for _ in range(3):
        tdist.all_gather_into_tensor(full, flat)
    stop.record()
    torch.cuda.synchronize()
    ms = dist.max_over_ranks(start.elapsed_time(stop) / 3, flat.device)
    del full
    return ms


def time_overlapped_gather(w: Workload, lib, dist: Dist, chunks: int = 4) -> Optional[float]:
    """Milliseconds for the shard's kernel in `chunks` pieces with each piece's all-gather started as soon as
    the piece is enqueued (pyasc_b200.sharding.compute_and_gather): kernel and NCCL traffic overlap."""
    if not dist.enabled or not hasattr(w, "launch_range"):
        return None
    from pyasc_b200 import sharding
    local = w.out
    full = torch.empty((local.shape[0] * dist.world, ) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def compute(lo, hi):
        rc = w.launch_range(lib, stream, lo, hi)
        if rc != 0:
            raise RuntimeError(f"{w.name}: chunk launch returned {rc}")

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


def run_ours(args) -> Dict[str, Any]:
    dist = Dist(args.gpus)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the CUDA platform has no CPU fallback")
    torch.cuda.set_device(dist.local_rank)
    dev = torch.device("cuda", dist.local_rank)
    dist.init("nccl")
    import pyasc_b200  # noqa: F401
    import asc
    from pyasc_b200 import capi
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
        ms = time_device(w, lib, args.steps, args.warmup, dist, dev)
        timed_launches += args.steps
        per_gpu = w.throughput(w.work, ms * 1e-3)
        peak = w.peak(peaks)
        res: Dict[str, Any] = {
            "workload": w.label, "value": round(per_gpu * dist.world, 2), "unit": w.unit, "ms_per_step": round(ms, 5),
            "dtype": w.dtype,
            "roofline": {"bound": w.bound, "achieved": round(per_gpu, 2), "peak": round(peak, 1),
                         "unit": w.unit, "frac": round(per_gpu / peak, 4), "traffic": None,
                         "peak_source": peaks["source"] + (" (2 x bf16 burst)" if name.startswith("gemm_i8") else
                                                           " (bf16 burst)" if w.bound == "tensor" else " (copy)")},
        }
        res["roofline"]["nominal_peak"] = NOMINAL[w.bound] * (2 if name.startswith("gemm_i8") else 1)
        res["roofline"]["frac_of_nominal"] = round(per_gpu / res["roofline"]["nominal_peak"], 4)
        if w.bound == "tensor" and args.sustained_seconds > 0:
            timed_launches_before = capi.launch_count()
            sus = time_sustained(w, lib, args.sustained_seconds, ms)
            timed_launches += capi.launch_count() - timed_launches_before
            sus_peak = float(peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"])) * (2 if name.startswith("gemm_i8") else 1)
            sus.update({"unit": w.unit, "peak": round(sus_peak, 1), "frac": round(sus["value"] / sus_peak, 4),
                        "peak_source": peaks["source"] + " (bf16 sustained" + (", x 2)" if name.startswith("gemm_i8") else ")")})
            res["sustained"] = sus
        ag = time_allgather(w, dist)
        if ag is not None:
            res["allgather_ms"] = round(ag, 4)
            res["compute_plus_allgather_ms"] = round(ms + ag, 4)
            ov = time_overlapped_gather(w, lib, dist)
            if ov is not None:
                res["overlapped_compute_and_allgather_ms"] = round(ov, 4)
        if not args.no_e2e:
            w.setup_host()
            e2e_steps = max(1, min(args.steps, args.e2e_steps))
            sec = time_e2e(w, e2e_steps, dist, dev)
            timed_launches += e2e_steps
            res["e2e"] = {"value": round(w.throughput(w.work, sec) * dist.world, 3), "unit": w.unit,
                          "h2d_bytes_per_step": w.h2d_bytes, "d2h_bytes_per_step": w.d2h_bytes,
                          "ms_per_step": round(sec * 1e3, 3), "steps": e2e_steps}
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
    head = results[HEADLINE] if HEADLINE in results else results[names[0]]
    traffic = load_traffic()
    for name, res in results.items():
        if name in traffic:
            res["roofline"]["traffic"] = traffic[name]
    line = {
        "metric": "HBM GB/s (fp32 row softmax, whole job); per-kernel HBM GB/s and tensor TFLOP/s under 'workloads'",
        "value": head["value"], "unit": head["unit"], "n_gpus": dist.world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": head["dtype"], "data": "synthetic (seeded, shapes and distributions of the named configs)",
        "config": {"workload": head["workload"], "l2": "inputs larger than L2 (126 MB)", "timing": "CUDA events, max over ranks",
                   "sharding": "every rank runs the full single-GPU workload on its own shard; no data-path collective"},
        "roofline": head["roofline"], "e2e": head.get("e2e"), "cpu_baseline": head.get("cpu_baseline"),
        "gpu_launches": total_launches, "gpu_launches_timed": timed_launches, "clocks": clocks, "workloads": results,
    }
    return line if dist.rank == 0 else {}


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
        "ms_per_step": round(head["seconds_per_sample"] * 1e3, 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": w.dtype, "data": "synthetic (seeded, shapes and distributions of the named configs)",
        "config": {"workload": w.label, "note": "CPU arm: torch expressions of the reference's tests on host cores"},
        "cpu_baseline": head,
        "e2e": {"value": head["value"], "unit": head["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "workloads": results,
    }


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--sustained-seconds", type=float, default=2.0,
                    help="length of the extra sustained loop for tensor-bound workloads (0: skip)")
    ap.add_argument("--workloads", type=lambda s: s.split(","), default=ALL_WORKLOADS,
                    help="comma-separated subset of: " + ",".join(ALL_WORKLOADS))
    ap.add_argument("--e2e-steps", type=int, default=5, help="timed end-to-end steps per workload (<= --steps)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
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
