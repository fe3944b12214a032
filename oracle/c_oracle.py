"""torch-tensor front end of the plain-C oracle (oracle/oracle.c).  TEST INFRASTRUCTURE ONLY."""
from __future__ import annotations

import torch

from . import build_oracle


def _p(t: torch.Tensor) -> int:
    assert t.is_contiguous() and t.device.type == "cpu"
    return t.data_ptr()


def vadd(x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    out = torch.empty_like(x)
    build_oracle.load().oracle_vadd_f32(_p(x), _p(y), _p(out), x.numel())
    return out


def vmuladd(x, y, z):
    out = torch.empty_like(x)
    build_oracle.load().oracle_vmuladd_f32(_p(x), _p(y), _p(z), _p(out), x.numel())
    return out


def softmax(x: torch.Tensor) -> torch.Tensor:
    out = torch.empty_like(x)
    build_oracle.load().oracle_softmax_f32(_p(x), _p(out), x.shape[0], x.shape[1])
    return out


def gemm_f32acc(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    c = torch.empty(a.shape[0], b.shape[1], dtype=torch.float32)
    build_oracle.load().oracle_gemm_16(_p(a), _p(b), _p(c), a.shape[0], b.shape[1], a.shape[1],
                                       int(a.dtype == torch.bfloat16))
    return c


def gemm_i8(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    c = torch.empty(a.shape[0], b.shape[1], dtype=torch.int32)
    build_oracle.load().oracle_gemm_i8(_p(a), _p(b), _p(c), a.shape[0], b.shape[1], a.shape[1])
    return c


def dequant(acc: torch.Tensor, a_scale: torch.Tensor, b_scale: torch.Tensor) -> torch.Tensor:
    out = torch.empty(acc.shape, dtype=torch.float16)
    build_oracle.load().oracle_dequant_f16(_p(acc), _p(a_scale), _p(b_scale), _p(out), acc.shape[0], acc.shape[1])
    return out


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool, scale: float) -> torch.Tensor:
    b, h, s, d = q.shape
    o = torch.empty(b, h, s, d, dtype=torch.float32)
    build_oracle.load().oracle_attention_f16(_p(q), _p(k), _p(v), _p(o), b * h, s, d, scale, int(causal))
    return o
