"""Parity of the CUDA kernels with the CPU oracle, called through the C ABI (ctypes) the way the
runtime binding calls them.  Bit-exact for fp32 add and the int8 product, rtol 1e-5 (atol 0) for
softmax, atol = rtol = 2e-3 for fp16 GEMM and attention."""
import ctypes
import os

import numpy as np
import pytest
import torch

from oracle import golden as G
from pyasc_b200 import capi

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def lib():
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    torch.cuda.set_device(0)
    return capi.load()


def P(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def run(lib, name, *args):
    """Call on torch's current (legacy default) stream, then check the device status word."""
    rc = getattr(lib, name)(*args, None)
    assert rc == 0, f"{name} returned {rc}: {capi.status_string(rc)} {capi.last_cuda_error()}"
    capi.check_device_status(None)


def dev(t):
    return t.cuda()


# --------------------------------------------------------------------------------------------- vadd
def test_vadd_fixtures_bit_exact(lib, golden_dir):
    d = np.load(os.path.join(golden_dir, "vadd_8192.npz"))
    x, y, z = (dev(torch.from_numpy(d[k])) for k in "xyz")
    out = torch.empty_like(x)
    run(lib, "asc_cuda_vadd_f32", P(x), P(y), P(out), 8192)
    G.assert_exact(out, d["out"])
    run(lib, "asc_cuda_vmuladd_f32", P(x), P(y), P(z), P(out), 8192)
    G.assert_exact(out, d["muladd"])        # no FMA contraction
    t = np.load(os.path.join(golden_dir, "vadd_torch_8192.npz"))
    x, y = dev(torch.from_numpy(t["x"])), dev(torch.from_numpy(t["y"]))
    run(lib, "asc_cuda_vadd_f32", P(x), P(y), P(out), 8192)
    G.assert_exact(out, t["out"])


@pytest.mark.parametrize("n", [1, 2, 3, 4, 5, 127, 1023, 4097, 100003, (1 << 20) + 1])
def test_vadd_ragged_sizes_and_misalignment(lib, n):
    x, y = G.vadd_inputs(n + 1, seed=n)
    xd, yd = dev(x), dev(y)
    out = torch.full((n + 1, ), -1.0, device="cuda")
    run(lib, "asc_cuda_vadd_f32", P(xd), P(yd), P(out), n)
    G.assert_exact(out[:n], G.vadd(x, y)[:n])
    assert float(out[n]) == -1.0                      # nothing written past n
    out.fill_(-1.0)
    off = lambda t: ctypes.c_void_p(t.data_ptr() + 4)   # pointers 4 bytes off a 16-byte boundary
    run(lib, "asc_cuda_vadd_f32", off(xd), off(yd), off(out), n)
    G.assert_exact(out[1:], G.vadd(x, y)[1:])
    assert float(out[0]) == -1.0


def test_vadd_special_values(lib):
    x = torch.tensor([0.0, -0.0, float("inf"), float("-inf"), float("nan"), 1e-45, 3.4e38, 1.0], device="cuda")
    y = torch.tensor([-0.0, -0.0, float("-inf"), 1.0, 1.0, 1e-45, 3.4e38, 2.0 ** -24], device="cuda")
    out = torch.empty_like(x)
    run(lib, "asc_cuda_vadd_f32", P(x), P(y), P(out), 8)
    G.assert_exact(out, G.vadd(x.cpu(), y.cpu()))     # signed zeros, NaN payload, denormals, overflow


def test_vadd_full_size_bit_exact(lib):
    n = 1 << 28
    g = torch.Generator(device="cuda").manual_seed(G.SEED)
    x = torch.rand(n, device="cuda", generator=g)
    y = torch.rand(n, device="cuda", generator=g)
    out = torch.empty_like(x)
    run(lib, "asc_cuda_vadd_f32", P(x), P(y), P(out), n)
    # first and last 4 Mi elements against the CPU oracle, everything against IEEE properties:
    # commutativity (bit-exact) and the exact residual (out - x) - y == 0 for operands in [0, 1)
    for sl in (slice(0, 1 << 22), slice(n - (1 << 22), n)):
        G.assert_exact(out[sl], G.vadd(x[sl].cpu(), y[sl].cpu()))
    out2 = torch.empty_like(x)
    run(lib, "asc_cuda_vadd_f32", P(y), P(x), P(out2), n)
    assert torch.equal(out, out2)
    assert torch.equal(out, x + y)


# ------------------------------------------------------------------------------------------ softmax
def test_softmax_fixtures(lib, golden_dir):
    d = np.load(os.path.join(golden_dir, "softmax.npz"))
    for tag in ("rand", "randn"):
        x = dev(torch.from_numpy(d["x_" + tag]))
        out = torch.empty_like(x)
        run(lib, "asc_cuda_softmax_f32", P(x), P(out), x.shape[0], x.shape[1], x.shape[1])
        G.assert_softmax_close(out, torch.from_numpy(d["out_" + tag]))


@pytest.mark.parametrize("rows, cols", [(1, 1), (7, 4), (33, 100), (17, 516), (64, 1024), (9, 2052), (5, 4100),
                                        (3, 8192), (2, 10000), (2, 70000), (300, 4096), (70, 1536), (45, 3072), (31, 2560),
                                        (29, 5120), (23, 6144)])
def test_softmax_shapes(lib, rows, cols):
    x = G.softmax_input(rows, cols, seed=rows * 131 + cols)
    xd = dev(x)
    out = torch.empty_like(xd)
    run(lib, "asc_cuda_softmax_f32", P(xd), P(out), rows, cols, cols)
    G.assert_softmax_close(out, G.softmax(x))


def test_softmax_pitched_rows_and_extreme_values(lib):
    x = G.softmax_input(40, 1024)
    xd = dev(x)
    out = torch.full_like(xd, -1.0)
    run(lib, "asc_cuda_softmax_f32", P(xd), P(out), 40, 512, 1024)   # first 512 columns of each row only
    G.assert_softmax_close(out[:, :512], G.softmax(x[:, :512]))
    assert bool((out[:, 512:] == -1.0).all())
    big = torch.tensor([[1e4, 1e4 - 1, -1e4, 0.0] * 256, [-80.0, 0.0, -60.0, -100.0] * 256], dtype=torch.float32)
    bd = dev(big)
    o = torch.empty_like(bd)
    run(lib, "asc_cuda_softmax_f32", P(bd), P(o), 2, 1024, 1024)
    ref = G.softmax(big)
    torch.testing.assert_close(o.cpu(), ref, rtol=1e-5, atol=1e-37)   # values down to the denormal range


@pytest.mark.parametrize("cols", [516, 1536, 3072, 4096, 5000, 9000])
def test_softmax_rows_of_minus_infinity_and_nan(lib, cols):
    """A row that is all -inf has no finite maximum: torch.softmax gives NaN for the whole row, whether or not the
    kernel's register tile has idle vector slots for this width (516, 1536, 3072: it has; 4096: none; 5000 and 9000
    take the staged kernel).  A row with one NaN is NaN throughout; a row with some -inf entries gives them 0."""
    x = G.softmax_input(6, cols, seed=cols)
    x[1] = float("-inf")
    x[3, cols // 2] = float("nan")
    x[4, ::3] = float("-inf")
    xd = dev(x)
    out = torch.empty_like(xd)
    run(lib, "asc_cuda_softmax_f32", P(xd), P(out), 6, cols, cols)
    ref = G.softmax(x)
    assert bool(ref[1].isnan().all()) and bool(ref[3].isnan().all())
    got = out.cpu()
    assert torch.equal(got.isnan(), ref.isnan())
    assert bool((got[4, ::3] == 0).all())
    keep = [0, 2, 4, 5]
    torch.testing.assert_close(got[keep], ref[keep], rtol=1e-5, atol=0)


def test_softmax_full_size(lib):
    x = G.softmax_input(16384, 4096)
    xd = dev(x)
    out = torch.empty_like(xd)
    run(lib, "asc_cuda_softmax_f32", P(xd), P(out), 16384, 4096, 4096)
    G.assert_softmax_close(out, G.softmax(x))
    torch.testing.assert_close(out.sum(-1).cpu(), torch.ones(16384), atol=2e-6, rtol=0)


# ----------------------------------------------------------------------------------------- fp16 GEMM
def gemm16(lib, a, b, out_dtype, flags=0, c=None):
    m, k = a.shape
    n = b.shape[1]
    if c is None:
        c = torch.full((m, n), -7.0, dtype=out_dtype, device="cuda")
    in_code = 0 if a.dtype == torch.float16 else 1
    out_code = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}[out_dtype]
    run(lib, "asc_cuda_gemm_f16", P(a), P(b), P(c), m, n, k, k, n, n, in_code, out_code, flags)
    return c


def test_gemm_f16_fixtures(lib, golden_dir):
    d = np.load(os.path.join(golden_dir, "gemm_f16.npz"))
    c = gemm16(lib, dev(torch.from_numpy(d["a"])), dev(torch.from_numpy(d["b"])), torch.float32)
    torch.testing.assert_close(c.cpu(), torch.from_numpy(d["c_f32"]))          # reference default fp32 tolerance
    c2 = gemm16(lib, dev(torch.from_numpy(d["a2"])), dev(torch.from_numpy(d["b2"])), torch.float16, flags=1)
    torch.testing.assert_close(c2.cpu(), torch.from_numpy(d["c2_relu_f16"]), atol=1e-3, rtol=1e-3)


@pytest.mark.parametrize("m, n, k", [(16, 16, 16), (16, 16, 160), (32, 32, 16), (64, 256, 128), (100, 200, 72),
                                     (128, 256, 64), (129, 257, 72), (480, 1344, 224), (1024, 1024, 1024),
                                     (2048, 4096, 512), (300, 8, 4096)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_gemm_f16_shapes(lib, m, n, k, dtype):
    if (n * 2) % 16:
        pytest.skip("row pitch of B must be a multiple of 16 bytes")
    a, b = G.gemm_f16_inputs(m, n, k, dtype, seed=m + n + k)
    c = gemm16(lib, dev(a), dev(b), torch.float32)
    if m * n * k <= 1 << 28:        # small fp32 results come from the FMA pipe: torch's default fp32 tolerance holds
        torch.testing.assert_close(c.cpu(), G.gemm_f32acc(a, b))
    assert lib.asc_cuda_gemm_set_mode(0x10) == 0          # ... and from the tensor core when asked to
    try:
        c = gemm16(lib, dev(a), dev(b), torch.float32)
    finally:
        assert lib.asc_cuda_gemm_set_mode(0) == 0
    torch.testing.assert_close(c.cpu(), G.gemm_f32acc(a, b), atol=2e-5 * (k ** 0.5) / 8 + 1e-5, rtol=1e-4)
    c16 = gemm16(lib, dev(a), dev(b), dtype)
    ref = G.gemm_f16(a, b, out_dtype=dtype)
    tol = 2e-3 if dtype == torch.float16 else 1.6e-2
    torch.testing.assert_close(c16.cpu().float(), ref.float(), atol=tol, rtol=tol)


@pytest.mark.parametrize("tensor_core", [False, True], ids=["fma_pipe", "tensor_core"])
def test_gemm_f16_accumulate_relu_and_linearity(lib, tensor_core):
    assert lib.asc_cuda_gemm_set_mode(0x10 if tensor_core else 0) == 0
    try:
        _accumulate_relu_and_linearity(lib)
    finally:
        assert lib.asc_cuda_gemm_set_mode(0) == 0


def _accumulate_relu_and_linearity(lib):
    a, b = G.gemm_f16_inputs(256, 512, 384)
    ad, bd = dev(a), dev(b)
    base = gemm16(lib, ad, bd, torch.float32)
    c = base.clone()
    gemm16(lib, ad, bd, torch.float32, flags=2, c=c)                 # C += A @ B
    torch.testing.assert_close(c, 2 * base)
    r = gemm16(lib, ad, bd, torch.float32, flags=1)
    assert torch.equal(r, base.relu())
    # (2A) @ B == 2 (A @ B) exactly: scaling by two is exact in fp16 and fp32
    assert torch.equal(gemm16(lib, (ad * 2), bd, torch.float32), 2 * base)
    # identity: A @ I == A exactly
    eye = torch.eye(384, dtype=torch.float16, device="cuda")
    assert torch.equal(gemm16(lib, ad, eye, torch.float16), ad)


@pytest.mark.parametrize("m, n, k", [(256, 256, 8192), (128, 256, 2048), (100, 520, 4104), (384, 768, 4096),
                                     (1024, 1024, 16384), (64, 64, 65536)])
@pytest.mark.parametrize("out_dtype", [torch.float16, torch.float32])
def test_gemm_f16_split_k(lib, m, n, k, out_dtype):
    """A long K over a C of a few tiles: K is split over several CTAs per tile and the partial tiles are summed
    from a workspace.  Against the CPU oracle at the workload's tolerance, against the unsplit kernel, and
    bit-identical from run to run (the slices are always summed in the same order)."""
    a, b = G.gemm_f16_inputs(m, n, k, seed=k + m)
    ad, bd = dev(a), dev(b)
    assert lib.asc_cuda_gemm_set_mode(0x10) == 0           # fp32 results from the tensor core as well
    try:
        c = gemm16(lib, ad, bd, out_dtype, flags=1)
        again = gemm16(lib, ad, bd, out_dtype, flags=1)
        assert lib.asc_cuda_gemm_set_mode(0x30) == 0       # the same without split-K
        whole = gemm16(lib, ad, bd, out_dtype, flags=1)
    finally:
        assert lib.asc_cuda_gemm_set_mode(0) == 0
    assert torch.equal(c, again)
    ref = G.gemm_f16(a, b, relu=True, out_dtype=out_dtype)
    if out_dtype == torch.float16:
        G.assert_half_close(c, ref)
        G.assert_half_close(c, whole.cpu())
    else:
        torch.testing.assert_close(c.cpu(), ref, atol=2e-5 * (k ** 0.5) / 8 + 1e-5, rtol=1e-4)
        torch.testing.assert_close(c, whole, atol=2e-5 * (k ** 0.5) / 8 + 1e-5, rtol=1e-4)
    if out_dtype == torch.float32:                         # C += A @ B through the split-K epilogue
        assert lib.asc_cuda_gemm_set_mode(0x10) == 0
        try:
            acc = c.clone()
            gemm16(lib, ad, bd, torch.float32, flags=2, c=acc)
            plain = gemm16(lib, ad, bd, torch.float32)
        finally:
            assert lib.asc_cuda_gemm_set_mode(0) == 0
        assert torch.equal(acc, c + plain)


def gemm16_bias(lib, a, b, bias, out_dtype, flags=0):
    m, k = a.shape
    n = b.shape[1]
    c = torch.full((m, n), -7.0, dtype=out_dtype, device="cuda")
    code = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}
    run(lib, "asc_cuda_gemm_f16_bias", P(a), P(b), P(c), P(bias), m, n, k, k, n, n, code[a.dtype], code[out_dtype],
        code[bias.dtype], flags)
    return c


@pytest.mark.parametrize("m, n, k", [(16, 16, 16), (129, 264, 72), (256, 256, 8192), (1024, 1024, 1024),
                                     (2048, 4096, 512), (300, 8, 4096), (500, 704, 128)])
@pytest.mark.parametrize("bias_dtype", [torch.float32, torch.float16, torch.bfloat16], ids=str)
def test_gemm_f16_bias_row_in_the_epilogue(lib, m, n, k, bias_dtype):
    """C = cast(relu?(A @ B + bias)): the same accumulators as the plain product, one fp32 addition rounded to
    nearest, then the ReLU and the one rounding of the store, so the result equals the fp32 product finished in
    torch bit for bit, in every kernel variant (one CTA per tile, CTA pairs, split-K, the FMA pipe)."""
    a, b = G.gemm_f16_inputs(m, n, k, seed=m + k)
    ad, bd = dev(a), dev(b)
    bias = (torch.randn(n, generator=torch.Generator().manual_seed(n)) * 0.5).to(bias_dtype).cuda()
    for mode in (0x10, 0):                                  # fp32 results from the tensor core, then as dispatched
        assert lib.asc_cuda_gemm_set_mode(mode) == 0
        try:
            plain = gemm16(lib, ad, bd, torch.float32)
            outs = (torch.float32, torch.float16, torch.bfloat16) if mode else (torch.float32, )
            for out_dtype in outs:
                for relu in (0, 1):
                    got = gemm16_bias(lib, ad, bd, bias, out_dtype, flags=relu)
                    want = plain + bias.float()
                    want = (want.relu() if relu else want).to(out_dtype)
                    assert torch.equal(got, want), (hex(mode), out_dtype, relu)
        finally:
            assert lib.asc_cuda_gemm_set_mode(0) == 0
    ref = G.gemm_f32acc(a, b) + bias.float().cpu()          # ... and against the CPU expression
    got = gemm16_bias(lib, ad, bd, bias, torch.float16, flags=1)
    G.assert_half_close(got, ref.relu().half())


def test_gemm_f16_bias_argument_checks_and_nan(lib):
    a, b = G.gemm_f16_inputs(256, 512, 384)
    ad, bd = dev(a), dev(b)
    bias = torch.zeros(512, device="cuda")
    c = torch.zeros(256, 512, device="cuda")
    args = (256, 512, 384, 384, 512, 512, 0, 2)
    assert lib.asc_cuda_gemm_f16_bias(P(ad), P(bd), P(c), None, *args, 2, 0, None) == 1       # no bias
    assert lib.asc_cuda_gemm_f16_bias(P(ad), P(bd), P(c), P(bias), *args, 3, 0, None) == 1    # bad bias type
    assert lib.asc_cuda_gemm_f16_bias(P(ad), P(bd), P(c), P(bias), *args, 2, 2, None) == 3    # C += ... + bias
    # a NaN in the accumulator stays a NaN through the ReLU, as in torch.relu (fmaxf would have returned 0)
    ad[3, 5] = float("nan")
    for out_dtype in (torch.float32, torch.float16):
        for mode in (0, 0x10):
            assert lib.asc_cuda_gemm_set_mode(mode) == 0
            try:
                got = gemm16_bias(lib, ad, bd, bias, out_dtype, flags=1)
                plain = gemm16(lib, ad, bd, out_dtype, flags=1)
            finally:
                assert lib.asc_cuda_gemm_set_mode(0) == 0
            for t in (got, plain):
                assert t[3].isnan().all() and not t[:3].isnan().any() and not t[4:].isnan().any()


def test_gemm_f16_full_size(lib):
    m = n = k = 8192
    a, b = G.gemm_f16_inputs(m, n, k)
    ad, bd = dev(a), dev(b)
    c = gemm16(lib, ad, bd, torch.float16)
    rows = torch.arange(0, m, 61)                                     # 135 rows against the CPU oracle
    G.assert_half_close(c[rows.cuda()], G.gemm_f16(a[rows], b))
    # checksum of checksums: (1^T A) B == 1^T C  up to fp16 rounding of C
    col_sum = (ad.float().sum(0, keepdim=True) @ bd.float()).squeeze(0)
    torch.testing.assert_close(c.float().sum(0), col_sum, atol=5e-3, rtol=5e-3)
    # every element: a second, independent implementation (torch.matmul on the GPU) as cross-check; the CPU oracle
    # above stays the reference for the sampled rows
    torch.testing.assert_close(c, torch.matmul(ad, bd), atol=2e-3, rtol=2e-3)


# ----------------------------------------------------------------------------------------- int8 GEMM
def gemm8(lib, a, b, a_scale=None, b_scale=None, want_acc=True):
    m, k = a.shape
    n = b.shape[1]
    acc = torch.full((m, n), -7, dtype=torch.int32, device="cuda") if want_acc else None
    deq = torch.full((m, n), -7.0, dtype=torch.float16, device="cuda") if a_scale is not None else None
    run(lib, "asc_cuda_gemm_i8", P(a), P(b), P(acc), P(deq), P(a_scale), P(b_scale), m, n, k, k, n, n)
    return acc, deq


def test_gemm_i8_fixture_bit_exact(lib, golden_dir):
    d = np.load(os.path.join(golden_dir, "gemm_i8.npz"))
    a, b = dev(torch.from_numpy(d["a"])), dev(torch.from_numpy(d["b"]))
    sa, sb = dev(torch.from_numpy(d["a_scale"])), dev(torch.from_numpy(d["b_scale"]))
    acc, deq = gemm8(lib, a, b, sa, sb)
    G.assert_exact(acc, d["acc"])
    G.assert_exact(deq, d["deq"])
    _, deq_only = gemm8(lib, a, b, sa, sb, want_acc=False)
    G.assert_exact(deq_only, d["deq"])


@pytest.mark.parametrize("m, n, k", [(1, 16, 16), (16, 16, 16), (100, 208, 80), (128, 256, 128), (130, 272, 144),
                                     (333, 992, 4096), (1024, 1024, 1024)])
def test_gemm_i8_shapes_bit_exact(lib, m, n, k):
    a, b, sa, sb = G.gemm_i8_inputs(m, n, k, seed=m * 7 + n)
    acc, deq = gemm8(lib, dev(a), dev(b), dev(sa), dev(sb))
    ref = G.gemm_i8(a, b)
    G.assert_exact(acc, ref)
    G.assert_exact(deq, G.dequant(ref, sa, sb))


@pytest.mark.parametrize("m, n, k", [(256, 256, 8192), (130, 272, 16400), (512, 512, 32768)])
def test_gemm_i8_split_k_bit_exact(lib, m, n, k):
    """Integer partial sums add exactly, so the split-K result equals the unsplit one and the oracle bit for bit,
    dequantised output included."""
    a, b, sa, sb = G.gemm_i8_inputs(m, n, k, seed=k)
    acc, deq = gemm8(lib, dev(a), dev(b), dev(sa), dev(sb))
    ref = G.gemm_i8(a, b)
    G.assert_exact(acc, ref)
    G.assert_exact(deq, G.dequant(ref, sa, sb))
    assert lib.asc_cuda_gemm_set_mode(0x20) == 0
    try:
        acc2, deq2 = gemm8(lib, dev(a), dev(b), dev(sa), dev(sb))
    finally:
        assert lib.asc_cuda_gemm_set_mode(0) == 0
    assert torch.equal(acc, acc2) and torch.equal(deq, deq2)


def test_gemm_i8_extreme_values(lib):
    a = torch.full((128, 8192), -128, dtype=torch.int8, device="cuda")
    b = torch.full((8192, 256), -128, dtype=torch.int8, device="cuda")
    acc, _ = gemm8(lib, a, b)
    assert bool((acc == 8192 * 128 * 128).all())                     # 2^27: the largest accumulator the workload allows
    b.fill_(127)
    acc, _ = gemm8(lib, a, b)
    assert bool((acc == -8192 * 128 * 127).all())


def test_gemm_i8_full_size_bit_exact(lib):
    m = n = k = 8192
    a, b, sa, sb = G.gemm_i8_inputs(m, n, k)
    ad, bd = dev(a), dev(b)
    acc, deq = gemm8(lib, ad, bd, dev(sa), dev(sb))
    rows = torch.arange(0, m, 127)
    ref = G.gemm_i8(a[rows], b)
    G.assert_exact(acc[rows.cuda()], ref)
    G.assert_exact(deq[rows.cuda()], G.dequant(ref, sa[rows], sb))
    # exact checksum over the whole product in int64: 1^T (A B) == (1^T A) B
    lhs = acc.to(torch.int64).sum(0)
    rhs = (ad.to(torch.float64).sum(0, keepdim=True) @ bd.to(torch.float64)).squeeze(0).to(torch.int64)
    assert torch.equal(lhs, rhs)
    # every element, exactly: the product in float64 on the GPU (all integers involved are far below 2^53) as a
    # second, independent implementation; the CPU oracle above stays the reference for the sampled rows
    for r0 in range(0, m, 2048):
        full = (ad[r0:r0 + 2048].to(torch.float64) @ bd.to(torch.float64)).to(torch.int32)
        assert torch.equal(acc[r0:r0 + 2048], full)


# ----------------------------------------------------------------------------------------- attention
def attn(lib, q, k, v, causal, scale=None):
    b, h, s, d = q.shape
    o = torch.full_like(q, 7.0)
    scale = d ** -0.5 if scale is None else scale
    run(lib, "asc_cuda_attn_fwd_f16", P(q), P(k), P(v), P(o), b, h, s, d, ctypes.c_float(scale), int(causal),
        0 if q.dtype == torch.float16 else 1)
    return o


def test_attention_fixture(lib, golden_dir):
    d = np.load(os.path.join(golden_dir, "attention.npz"))
    q, k, v = (dev(torch.from_numpy(d[n])) for n in "qkv")
    G.assert_half_close(attn(lib, q, k, v, False), torch.from_numpy(d["o"]))
    G.assert_half_close(attn(lib, q, k, v, True), torch.from_numpy(d["o_causal"]))


@pytest.mark.parametrize("b, h, s", [(1, 1, 1), (1, 1, 100), (1, 1, 128), (1, 2, 129), (1, 1, 256), (1, 3, 333),
                                     (2, 2, 512), (1, 2, 1024)])
@pytest.mark.parametrize("causal", [False, True])
def test_attention_shapes(lib, b, h, s, causal):
    q, k, v = G.attention_inputs(b, h, s, seed=s)
    o = attn(lib, dev(q), dev(k), dev(v), causal)
    G.assert_half_close(o, G.attention(q, k, v, causal))


def test_attention_bf16_and_large_scores(lib):
    q, k, v = G.attention_inputs(1, 2, 512, dtype=torch.bfloat16)
    o = attn(lib, dev(q), dev(k), dev(v), True)
    torch.testing.assert_close(o.cpu().float(), G.attention(q, k, v, True).float(), atol=1.6e-2, rtol=1.6e-2)
    # scores with a large spread force the running maximum to move (output rescaling path)
    q, k, v = G.attention_inputs(1, 2, 1024)
    q = (q.float() * 6).half()
    o = attn(lib, dev(q), dev(k), dev(v), False)
    G.assert_half_close(o, G.attention(q, k, v, False))


def test_attention_properties_full_size(lib):
    b, h, s, d = 4, 32, 4096, 128
    q, k, v = G.attention_inputs(b, h, s)
    qd, kd, vd = dev(q), dev(k), dev(v)
    for causal in (False, True):
        o = attn(lib, qd, kd, vd, causal)
        for (bi, hi) in ((0, 0), (3, 31)):
            ref = G.attention(q[bi:bi + 1, hi:hi + 1], k[bi:bi + 1, hi:hi + 1], v[bi:bi + 1, hi:hi + 1], causal)
            G.assert_half_close(o[bi:bi + 1, hi:hi + 1], ref)
        if causal:   # row 0 sees key 0 only
            assert torch.equal(o[:, :, 0], vd[:, :, 0])
        # every (batch, head): a second, independent implementation (torch's fused attention on the GPU, fp32
        # inputs) as cross-check; the CPU oracle above stays the reference for the sampled heads
        sdpa = torch.nn.functional.scaled_dot_product_attention(qd.float(), kd.float(), vd.float(), is_causal=causal)
        torch.testing.assert_close(o.float(), sdpa, atol=2e-3, rtol=2e-3)
        del sdpa
    # with V == 1 every output is exactly 1 (softmax rows sum to one)
    ones = torch.ones_like(vd)
    o = attn(lib, qd, kd, ones, False)
    torch.testing.assert_close(o.float(), ones.float(), atol=1e-3, rtol=0)


# ----------------------------------------------------------------------------------------- bounded waits
def test_a_wait_that_runs_out_is_reported_and_leaves_the_device_usable(lib):
    """The one error path a healthy kernel never takes: a device-side wait whose limit expires.  The self-test
    kernel waits 0.5 ms on a barrier nobody arrives on, gives up and returns normally; the host then sees status 5
    with device code 0x500, the status word is clear again afterwards, and the next ordinary launch succeeds."""
    capi.check_device_status(None)                                     # starts clean
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert lib.asc_cuda_selftest_wait_runs_out(P(flag), None) == 0
    code = ctypes.c_uint32(0)
    rc = lib.asc_cuda_check_device_status(None, ctypes.addressof(code))
    assert rc == 5 and code.value == 0x500
    assert capi.status_string(rc) == "bounded device-side wait ran out"
    assert int(flag.item()) == 1
    rc = lib.asc_cuda_check_device_status(None, ctypes.addressof(code))
    assert rc == 0 and code.value == 0                                 # reported once, then clear
    with pytest.raises(RuntimeError, match="0x500"):
        lib.asc_cuda_selftest_wait_runs_out(None, None)
        capi.check_device_status(None)
    x, y = G.vadd_inputs(4096)
    xd, yd = dev(x), dev(y)
    out = torch.empty_like(xd)
    run(lib, "asc_cuda_vadd_f32", P(xd), P(yd), P(out), 4096)
    G.assert_exact(out, G.vadd(x, y))
