"""The oracle: the CPU expressions the reference's own asc2 tests assert against, as functions.

TEST INFRASTRUCTURE, NOT PRODUCT: nothing under ``pyasc_b200/`` imports this module.

The reference computes every golden at test time with torch / NumPy on the host; it ships no golden
files and cannot itself be built or imported without MLIR and the CANN toolkit, so these expressions
ARE its side of the parity contract:

* vector add        ``x + y``                         python/test/asc2/kernels/test_vadd.py:48, README.md:53
* multiply-add      ``x * y + z``                     python/test/asc2/kernels/test_vmuladd.py:51
* row softmax       ``torch.softmax(x, dim=1)``       python/test/asc2/kernels/test_softmax.py:43,
                                                      test_softmax_fused.py:41
* fp16/bf16 matmul  ``a.float() @ b.float()``         python/test/asc2/kernels/test_matmul_tiled.py:49,
                                                      test_matmul_mnblock.py:91
  with epilogue     ``(...).relu().to(float16)``      python/test/asc2/kernels/test_matmul_fixpipe.py:47
* int8 matmul       ``a.int32 @ b.int32``             python/test/generalization/adv/test_matmul_quant.py:134
                    (a skipped v1 test; the reference has no asc2 int8 kernel, and its per-column
                    truncated-mantissa scale differs from the workload's definition, so the dequantised
                    form below is pinned by the workload definition, not by a reference test:
                    PARITY UNPINNED BY THE REFERENCE)
* attention         no counterpart in the reference; defined by the workload as
                    ``softmax((Q.float() @ K.float().T) * scale + mask, -1) @ V.float()``:
                    PARITY UNPINNED BY THE REFERENCE

Pins: tests/test_oracle.py checks every function against the committed fixtures under tests/golden/
(generated here by tests/golden/make_golden.py) and against the independent plain-C restatement in
oracle/oracle.c.
"""
from __future__ import annotations

import math

import numpy as np
import torch

SEED = 2026  # the reference's own asc2 seed (python/test/asc2/kernels/test_vadd.py:43)


# ---------------------------------------------------------------------------------------------------
# seeded synthetic inputs with the workloads' shapes and distributions
# ---------------------------------------------------------------------------------------------------
def gen(seed: int = SEED) -> torch.Generator:
    return torch.Generator(device="cpu").manual_seed(seed)


def vadd_inputs(n: int, seed: int = SEED):
    g = gen(seed)
    return torch.rand(n, generator=g), torch.rand(n, generator=g)


def softmax_input(rows: int, cols: int, seed: int = SEED):
    return torch.randn(rows, cols, generator=gen(seed))


def gemm_f16_inputs(m: int, n: int, k: int, dtype=torch.float16, seed: int = SEED):
    g = gen(seed)
    a = (torch.randn(m, k, generator=g) * k ** -0.5).to(dtype)
    b = (torch.randn(k, n, generator=g) * k ** -0.5).to(dtype)
    return a, b


def gemm_i8_inputs(m: int, n: int, k: int, seed: int = SEED):
    g = gen(seed)
    a = torch.randint(-128, 128, (m, k), dtype=torch.int8, generator=g)
    b = torch.randint(-128, 128, (k, n), dtype=torch.int8, generator=g)
    a_scale = torch.rand(m, generator=g) * (1e-2 - 1e-3) + 1e-3
    b_scale = torch.rand(n, generator=g) * (1e-2 - 1e-3) + 1e-3
    return a, b, a_scale, b_scale


def attention_inputs(batch: int, heads: int, seq: int, dim: int = 128, dtype=torch.float16, seed: int = SEED):
    g = gen(seed)
    return tuple(torch.randn(batch, heads, seq, dim, generator=g).to(dtype) for _ in range(3))


# ---------------------------------------------------------------------------------------------------
# goldens
# ---------------------------------------------------------------------------------------------------
def vadd(x, y):
    """python/test/asc2/kernels/test_vadd.py:48 — works for NumPy arrays and torch tensors."""
    return x + y


def vmuladd(x, y, z):
    """python/test/asc2/kernels/test_vmuladd.py:51 — separately rounded multiply and add."""
    return x * y + z


def softmax(x: torch.Tensor) -> torch.Tensor:
    """python/test/asc2/kernels/test_softmax.py:43"""
    return torch.softmax(x, dim=-1)


def rms_norm(x: torch.Tensor, gamma: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2, last dim) + eps) * gamma in fp32: the formula of the Ascend C RmsNorm routine that
    asc2.rms_norm lowers to (python/asc/language/tile/unary_ops.py:225-237; the tiling's
    ``reciprocalOfHLength`` = 1 / row length, lib/Conversion/LowerToAsc/LowerAscTile.cpp:223)."""
    x = x.float()
    return x * torch.rsqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps) * gamma.float().reshape(-1)


def gemm_f32acc(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """python/test/asc2/kernels/test_matmul_tiled.py:49 — fp32 product of the up-cast operands."""
    return a.to(torch.float32) @ b.to(torch.float32)


def gemm_f16(a: torch.Tensor, b: torch.Tensor, relu: bool = False, out_dtype=torch.float16) -> torch.Tensor:
    """python/test/asc2/kernels/test_matmul_fixpipe.py:47 (with ReLU) / the workload's
    ``(A.float() @ B.float()).half()``."""
    c = gemm_f32acc(a, b)
    if relu:
        c = c.relu()
    return c.to(out_dtype)


def gemm_i8(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """python/test/generalization/adv/test_matmul_quant.py:134 — ``a.int32 @ b.int32``.  Evaluated as
    fp64 matmul, which is exact here (|acc| <= K * 128^2 < 2^53) and much faster on CPU than torch's
    int32 matmul; tests/test_oracle.py checks the two agree."""
    return (a.to(torch.float64) @ b.to(torch.float64)).to(torch.int32)


def gemm_i8_int32_form(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """The reference's literal expression (slow on CPU; small sizes only)."""
    return a.to(torch.int32) @ b.to(torch.int32)


def dequant(acc: torch.Tensor, a_scale: torch.Tensor, b_scale: torch.Tensor) -> torch.Tensor:
    """Workload definition: ``out_fp16 = acc * a_scale[row] * b_scale[col]``, left to right in fp32."""
    return (acc.to(torch.float32) * a_scale[:, None] * b_scale[None, :]).to(torch.float16)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = False, scale=None) -> torch.Tensor:
    """Workload definition, fp32 throughout, result in the input dtype.  One (batch, head) at a time so
    that the score matrix stays small."""
    b, h, s, d = q.shape
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    out = torch.empty_like(q)
    mask = None
    if causal:
        mask = torch.full((s, s), float("-inf")).triu(1)
    for i in range(b):
        for j in range(h):
            scores = (q[i, j].float() @ k[i, j].float().transpose(-1, -2)) * scale
            if mask is not None:
                scores = scores + mask
            out[i, j] = (torch.softmax(scores, dim=-1) @ v[i, j].float()).to(q.dtype)
    return out


# ---------------------------------------------------------------------------------------------------
# tolerances (the workload's: bit-exact / rtol 1e-5 / atol=rtol 2e-3)
# ---------------------------------------------------------------------------------------------------
def assert_exact(out, ref) -> None:
    """Bit-for-bit equality (signed zeros and denormals included).  NaNs only have to sit at the same
    positions: sign and payload of a generated NaN are not defined by IEEE 754 and differ between
    x86 (0xFFC00000) and CUDA (0x7FFFFFFF)."""
    o = out if isinstance(out, np.ndarray) else out.detach().cpu().numpy()
    r = ref if isinstance(ref, np.ndarray) else ref.detach().cpu().numpy()
    if o.shape != r.shape or o.dtype != r.dtype:
        raise AssertionError(f"shape/dtype mismatch: {o.shape} {o.dtype} vs {r.shape} {r.dtype}")
    if o.dtype.kind == "f":
        nan_o, nan_r = np.isnan(o), np.isnan(r)
        ob = np.where(nan_o, 0, o).view(np.uint8)
        rb = np.where(nan_r, 0, r).view(np.uint8)
        ok = np.array_equal(nan_o, nan_r) and np.array_equal(ob, rb)
    else:
        ok = np.array_equal(o, r)
    if not ok:
        bad = int((o != r).sum())
        raise AssertionError(f"not bit-exact: {bad} mismatching elements")


def assert_softmax_close(out: torch.Tensor, ref: torch.Tensor) -> None:
    torch.testing.assert_close(out.cpu(), ref, rtol=1e-5, atol=0)


def assert_half_close(out: torch.Tensor, ref: torch.Tensor) -> None:
    torch.testing.assert_close(out.cpu().float(), ref.float(), rtol=2e-3, atol=2e-3)
