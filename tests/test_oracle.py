"""The oracle pinned: the reference's CPU expressions (oracle/golden.py) against the committed
fixtures and against the independent plain-C restatement (oracle/oracle.c).  CPU only."""
import os

import numpy as np
import torch

from oracle import c_oracle as C
from oracle import golden as G


def _load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name))


def test_vadd_fixture(golden_dir):
    d = _load(golden_dir, "vadd_8192.npz")
    G.assert_exact(G.vadd(d["x"], d["y"]), d["out"])
    G.assert_exact(G.vmuladd(d["x"], d["y"], d["z"]), d["muladd"])
    x, y, z = (torch.from_numpy(d[k]) for k in "xyz")
    G.assert_exact(C.vadd(x, y), d["out"])
    G.assert_exact(C.vmuladd(x, y, z), d["muladd"])
    t = _load(golden_dir, "vadd_torch_8192.npz")
    tx, ty = G.vadd_inputs(8192)
    G.assert_exact(tx, t["x"])          # the seeded generator reproduces the committed inputs
    G.assert_exact(G.vadd(tx, ty), t["out"])


def test_softmax_fixture(golden_dir):
    d = _load(golden_dir, "softmax.npz")
    for tag in ("rand", "randn"):
        x = torch.from_numpy(d["x_" + tag])
        ref = torch.from_numpy(d["out_" + tag])
        G.assert_softmax_close(G.softmax(x), ref)
        G.assert_softmax_close(C.softmax(x), ref)
        assert torch.allclose(ref.sum(-1), torch.ones(x.shape[0]), atol=1e-5)


def test_gemm_f16_fixture(golden_dir):
    d = _load(golden_dir, "gemm_f16.npz")
    a, b = torch.from_numpy(d["a"]), torch.from_numpy(d["b"])
    torch.testing.assert_close(G.gemm_f32acc(a, b), torch.from_numpy(d["c_f32"]))
    torch.testing.assert_close(C.gemm_f32acc(a, b), torch.from_numpy(d["c_f32"]))
    a2, b2 = torch.from_numpy(d["a2"]), torch.from_numpy(d["b2"])
    ref = torch.from_numpy(d["c2_relu_f16"])
    G.assert_half_close(G.gemm_f16(a2, b2, relu=True), ref)
    G.assert_half_close(C.gemm_f32acc(a2, b2).relu().half(), ref)
    assert (ref >= 0).all()


def test_gemm_bf16_c_matches_torch():
    a, b = G.gemm_f16_inputs(48, 64, 96, torch.bfloat16)
    torch.testing.assert_close(C.gemm_f32acc(a, b), G.gemm_f32acc(a, b))


def test_gemm_i8_fixture(golden_dir):
    d = _load(golden_dir, "gemm_i8.npz")
    a, b = torch.from_numpy(d["a"]), torch.from_numpy(d["b"])
    sa, sb = torch.from_numpy(d["a_scale"]), torch.from_numpy(d["b_scale"])
    acc = torch.from_numpy(d["acc"])
    G.assert_exact(G.gemm_i8(a, b), acc)               # fp64 route == the reference's int32 expression
    G.assert_exact(G.gemm_i8_int32_form(a, b), acc)
    G.assert_exact(C.gemm_i8(a, b), acc)
    G.assert_exact(G.dequant(acc, sa, sb), d["deq"])
    G.assert_exact(C.dequant(acc, sa, sb), d["deq"])
    a2, b2, _, _ = G.gemm_i8_inputs(96, 144, 160)
    G.assert_exact(a2, d["a"])


def test_gemm_i8_extremes():
    a = torch.full((8, 256), -128, dtype=torch.int8)
    b = torch.full((256, 16), -128, dtype=torch.int8)
    assert int(G.gemm_i8(a, b)[0, 0]) == 256 * 128 * 128
    G.assert_exact(C.gemm_i8(a, b), G.gemm_i8(a, b))


def test_attention_fixture(golden_dir):
    d = _load(golden_dir, "attention.npz")
    q, k, v = (torch.from_numpy(d[n]) for n in "qkv")
    for causal, key in ((False, "o"), (True, "o_causal")):
        ref = torch.from_numpy(d[key])
        G.assert_half_close(G.attention(q, k, v, causal), ref)
        G.assert_half_close(C.attention(q, k, v, causal, 128 ** -0.5).half(), ref)
    # causal row 0 attends to key 0 only
    torch.testing.assert_close(torch.from_numpy(d["o_causal"])[:, :, 0].float(), v[:, :, 0].float(), atol=1e-3, rtol=0)
