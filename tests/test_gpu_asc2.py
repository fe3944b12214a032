"""The reference's asc2 kernel tests, run on the CUDA platform through the public surface
(``@asc2.jit`` kernels launched as ``kernel[core_num](...)`` after
``asc.runtime.config.set_platform(backend, platform, device_id)``), plus the five workload scripts.
Test bodies follow python/test/asc2/kernels/test_*.py: same shapes, same input distributions, same
CPU goldens and tolerances."""
import numpy as np
import pytest
import torch

import asc
import asc.runtime.config as config
import asc2  # noqa: F401

import asc2_scripts as K
from oracle import golden as G
from pyasc_b200 import tutorials as T

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def select_platform(backend, platform, device_id):
    config.set_platform(backend, platform, device_id)


def test_vadd_numpy(backend):
    rng = np.random.default_rng(seed=2026)
    size = 8192
    x = rng.random(size, dtype=np.float32) * 10
    y = rng.random(size, dtype=np.float32) * 10
    out = np.empty_like(x)
    tile_size, core_num = 128, 16
    K.vadd[core_num](x, y, out, size, tile_size, asc.ceildiv(asc.ceildiv(size, tile_size), core_num))
    np.testing.assert_allclose(out, x + y)
    G.assert_exact(out, x + y)


def test_vadd_readme_form_torch_cpu():
    x = torch.rand(8192, dtype=torch.float32)
    y = torch.rand_like(x)
    out = torch.empty_like(x)
    tile_size, cores = 128, 16
    T.vadd_kernel[cores](x, y, out, out.numel(), tile_size, asc.ceildiv(out.numel() // tile_size, cores))
    torch.testing.assert_close(out, x + y)
    G.assert_exact(out, x + y)


def test_vadd_partial_coverage_leaves_tail_untouched():
    x, y = G.vadd_inputs(8192)
    out = torch.full_like(x, -1.0)
    K.vadd[16](x, y, out, 8192, 128, 3)                     # 16 * 3 * 128 = 6144 elements
    G.assert_exact(out[:6144], (x + y)[:6144])
    assert bool((out[6144:] == -1.0).all())


def test_vmuladd():
    rng = np.random.default_rng(seed=2026)
    size = 8192
    x, y, z = (rng.random(size, dtype=np.float32) * 10 for _ in range(3))
    out = np.empty_like(x)
    K.vmuladd[16](x, y, z, out, size, 32, asc.ceildiv(asc.ceildiv(size, 32), 16), buffer_factor=2)
    np.testing.assert_allclose(out, x * y + z)
    G.assert_exact(out, x * y + z)


def test_softmax_both_forms():
    x = torch.rand((64, 1024), dtype=torch.float32)
    out = torch.empty_like(x)
    K.softmax_rows[16](x, out, 64, 1024, tile_size=1024)
    torch.testing.assert_close(out, torch.softmax(x, dim=1))
    G.assert_softmax_close(out, G.softmax(x))
    out2 = torch.empty_like(x)
    K.softmax_blocks[16](x, out2, 64, 1024, 4)
    torch.testing.assert_close(out2, torch.softmax(x, dim=1))


@pytest.mark.parametrize("k_tiles", [2, 4, 8])
def test_matmul_tiled(k_tiles):
    m, k, n = 64, 128, 256
    a = torch.rand((m, k), dtype=torch.float16)
    b = torch.rand((k, n), dtype=torch.float16)
    c = torch.zeros((m, n), dtype=torch.float32)
    K.matmul_k_tiled[1](a, b, c, a.shape, b.shape, c.shape, k_tiles)
    torch.testing.assert_close(c, a.to(torch.float32) @ b.to(torch.float32))


@pytest.mark.parametrize("m, k, n, core_num, m_tile, n_tile, n_tiles_per_block", [
    (16, 16, 16, 1, 16, 16, 1), (16, 160, 16, 1, 16, 16, 1), (32, 16, 16, 2, 16, 16, 1), (16, 16, 32, 2, 16, 16, 1),
    (32, 16, 32, 2, 16, 16, 1), (32, 16, 32, 2, 16, 16, 2), (32, 16, 32, 4, 16, 16, 1),
    (480, 224, 1344, 30, 48, 32, 7)])
def test_matmul_mnblock(m, k, n, core_num, m_tile, n_tile, n_tiles_per_block):
    a = torch.rand((m, k), dtype=torch.float16)
    b = torch.rand((k, n), dtype=torch.float16)
    c = torch.zeros((m, n), dtype=torch.float32)
    mtpb = K.mn_tiles_per_block(m, n, core_num, m_tile, n_tile, n_tiles_per_block)
    K.matmul_mn_blocked[core_num](a, b, c, a.shape, b.shape, c.shape, m_tile, mtpb, n_tile, n_tiles_per_block)
    # torch's fp32 defaults (rtol 1.3e-6), as the reference asserts (python/test/asc2/kernels/test_matmul_mnblock.py:92):
    # a product of this size stored as fp32 runs on the FMA pipe with exact products and round-to-nearest sums
    torch.testing.assert_close(c, a.to(torch.float32) @ b.to(torch.float32))


@pytest.mark.parametrize("m, k, n, dtype", [(64, 128, 128, torch.float32), (64, 128, 256, torch.float16),
                                            (64, 128, 256, torch.bfloat16)])
def test_matmul_fixpipe(m, k, n, dtype):
    a = (torch.rand((m, k), dtype=dtype) - .5) * 10
    b = (torch.rand((k, n), dtype=dtype) - .5) * 10
    c = torch.zeros((m, n), dtype=torch.float16)
    K.matmul_relu_cast[1](a, b, c, a.shape, b.shape, c.shape)
    c_ref = (a.to(torch.float32) @ b.to(torch.float32)).relu().to(torch.float16)
    torch.testing.assert_close(c, c_ref, atol=1e-3, rtol=1e-3)


@asc2.jit(always_compile=True)
def dequant_scales_in_the_other_order(a_ptr: asc.GlobalAddress, b_ptr: asc.GlobalAddress, sa_ptr: asc.GlobalAddress,
                                      sb_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, m: asc.ConstExpr[int],
                                      n: asc.ConstExpr[int], k: asc.ConstExpr[int]):
    a_gm, b_gm, out_gm = asc2.tensor(a_ptr, [m, k]), asc2.tensor(b_ptr, [k, n]), asc2.tensor(out_ptr, [m, n])
    acc = asc2.matmul(asc2.load(a_gm, [m, k], offsets=[0, 0]), asc2.load(b_gm, [k, n], offsets=[0, 0]))
    sa = asc2.load(asc2.tensor(sa_ptr, [m]), [m], offsets=[0]).reshape(m, 1).broadcast_to(m, n)
    sb = asc2.load(asc2.tensor(sb_ptr, [n]), [n], offsets=[0]).reshape(1, n).broadcast_to(m, n)
    asc2.store((acc.to(asc.float32) * sb * sa).to(asc.float16), out_gm, offsets=[0, 0])


def test_int8_dequantisation_written_column_scale_first():
    """(acc * b_scale[col]) * a_scale[row] rounds differently from the fused epilogue's order: it takes the general
    path (int32 product in a temporary, then a program that multiplies in the order written) and is exact."""
    gen = torch.Generator().manual_seed(41)
    m, n, k = 128, 256, 512
    a = torch.randint(-128, 128, (m, k), generator=gen).to(torch.int8)
    b = torch.randint(-128, 128, (k, n), generator=gen).to(torch.int8)
    sa, sb = torch.rand(m, generator=gen) * 0.01 + 0.001, torch.rand(n, generator=gen) * 0.01 + 0.001
    out = torch.zeros(m, n, dtype=torch.float16)
    dequant_scales_in_the_other_order[1](a, b, sa, sb, out, m, n, k)
    assert dequant_scales_in_the_other_order.last_plan.pattern == "matmul+program"
    acc = (a.to(torch.int32) @ b.to(torch.int32)).to(torch.float32)
    assert torch.equal(out, ((acc * sb[None, :]) * sa[:, None]).to(torch.float16))


@pytest.mark.parametrize("form", ["to_fp32", "relu", "scaled"])
def test_int8_products_with_epilogues_the_gemm_does_not_fuse(form):
    """An int8 product cast to fp32, clamped by a ReLU or scaled by a scalar: the GEMM kernels refuse the epilogue, the
    general path (product in a temporary, then a program) computes it exactly."""
    body = {"to_fp32": lambda acc: acc.to(asc.float32), "relu": lambda acc: asc2.relu(acc),
            "scaled": lambda acc: acc.to(asc.float32) * 0.5}[form]

    @asc2.jit
    def kernel(a_ptr: asc.GlobalAddress, b_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, m: asc.ConstExpr[int],
               n: asc.ConstExpr[int], k: asc.ConstExpr[int]):
        a_gm, b_gm, out_gm = asc2.tensor(a_ptr, [m, k]), asc2.tensor(b_ptr, [k, n]), asc2.tensor(out_ptr, [m, n])
        acc = asc2.matmul(asc2.load(a_gm, [m, k], offsets=[0, 0]), asc2.load(b_gm, [k, n], offsets=[0, 0]))
        asc2.store(body(acc), out_gm, offsets=[0, 0])

    gen = torch.Generator().manual_seed(43)
    m, n, k = 128, 256, 192
    a = torch.randint(-128, 128, (m, k), generator=gen).to(torch.int8)
    b = torch.randint(-128, 128, (k, n), generator=gen).to(torch.int8)
    acc = a.to(torch.int32) @ b.to(torch.int32)
    want = {"to_fp32": acc.float(), "relu": acc.relu(), "scaled": acc.float() * 0.5}[form]
    out = torch.zeros(m, n, dtype=want.dtype)
    kernel[1](a, b, out, m, n, k)
    assert kernel.last_plan.pattern == "matmul+program" and torch.equal(out, want)


def test_k_loop_accumulator_with_an_epilogue_and_glu():
    gen = torch.Generator().manual_seed(77)
    m, n, k = 128, 256, 1024
    a = ((torch.rand(m, k, generator=gen) - .5) * 2 * k ** -0.5).half()
    b = (torch.rand(k, n, generator=gen) - .5).half()
    bias = torch.randn(1, n, generator=gen)
    c = torch.zeros(m, n)
    K.matmul_k_tiled_bias_relu[1](a, b, bias, c, m, n, k, 128)
    torch.testing.assert_close(c, (a.float() @ b.float() + bias).relu(), atol=2e-3, rtol=2e-3)
    x = torch.randn(256, 1024, generator=gen)
    out = torch.zeros(256, 512)
    K.glu_rows[4](x, out, 256, 512, 8)
    torch.testing.assert_close(out, x[:, :512] / (torch.exp(-x[:, 512:]) + 1), rtol=2e-6, atol=1e-6)


def test_expressions_over_several_products_and_fused_row_kernels_over_a_product():
    """SwiGLU (two products of one input combined elementwise), softmax and rms_norm of a product: every product is
    written to its own temporary, then one program or fused row kernel reads them like loaded tiles."""
    gen = torch.Generator().manual_seed(21)
    m, k, n = 512, 256, 1024
    x = ((torch.rand(m, k, generator=gen) - .5) * 2 * k ** -0.5).half()
    w1, w3 = ((torch.rand(k, n, generator=gen) - .5).half() for _ in range(2))

    @asc2.jit
    def swiglu(x_ptr: asc.GlobalAddress, w1_ptr: asc.GlobalAddress, w3_ptr: asc.GlobalAddress, o_ptr: asc.GlobalAddress,
               m: asc.ConstExpr[int], k: asc.ConstExpr[int], n: asc.ConstExpr[int], m_tile: asc.ConstExpr[int]):
        x_gm, w1_gm, w3_gm = asc2.tensor(x_ptr, [m, k]), asc2.tensor(w1_ptr, [k, n]), asc2.tensor(w3_ptr, [k, n])
        o_gm = asc2.tensor(o_ptr, [m, n])
        for i in range(asc2.block_idx() * m_tile, m, asc2.block_num() * m_tile):
            xt = asc2.load(x_gm, [m_tile, k], offsets=[i, 0])
            g = asc2.matmul(xt, asc2.load(w1_gm, [k, n], offsets=[0, 0]))
            u = asc2.matmul(xt, asc2.load(w3_gm, [k, n], offsets=[0, 0]))
            asc2.store((g / (asc2.exp(-g) + 1) * u).to(asc.float16), o_gm, offsets=[i, 0])
    out = torch.zeros(m, n, dtype=torch.float16)
    swiglu[4](x, w1, w3, out, m, k, n, 128)
    plan = swiglu.last_plan
    assert plan.pattern == "matmul+program" and len(plan.temps) == 2 and len(plan.steps) == 3
    g, u = x.float() @ w1.float(), x.float() @ w3.float()
    torch.testing.assert_close(out, (g / (torch.exp(-g) + 1) * u).half(), atol=2e-3, rtol=2e-3)

    @asc2.jit
    def scores(a_ptr: asc.GlobalAddress, b_ptr: asc.GlobalAddress, g_ptr: asc.GlobalAddress, o_ptr: asc.GlobalAddress,
               m: asc.ConstExpr[int], k: asc.ConstExpr[int], n: asc.ConstExpr[int], m_tile: asc.ConstExpr[int],
               norm: asc.ConstExpr[int]):
        a_gm, b_gm, o_gm = asc2.tensor(a_ptr, [m, k]), asc2.tensor(b_ptr, [k, n]), asc2.tensor(o_ptr, [m, n])
        gamma = asc2.load(asc2.tensor(g_ptr, [n]), [n], offsets=[0])
        for i in range(asc2.block_idx() * m_tile, m, asc2.block_num() * m_tile):
            s = asc2.matmul(asc2.load(a_gm, [m_tile, k], offsets=[i, 0]), asc2.load(b_gm, [k, n], offsets=[0, 0]))
            if norm == 2:
                asc2.store(asc2.softmax(s * 0.5), o_gm, offsets=[i, 0])        # a computed tile: a row program
            else:
                asc2.store(asc2.rms_norm(s, gamma, 1e-6) if norm else asc2.softmax(s), o_gm, offsets=[i, 0])
    xs = (x.float() * 8).half()                     # scores with a spread of a few units
    s = xs.float() @ w1.float()
    gamma = torch.rand(n, generator=gen) + 0.5
    out = torch.zeros(m, n)
    scores[4](xs, w1, gamma, out, m, k, n, 128, 0)
    assert [st.fn_name for st in scores.last_plan.steps] == ["asc_cuda_gemm_f16", "asc_cuda_softmax_f32"]
    torch.testing.assert_close(out, torch.softmax(s, dim=-1), atol=1e-5, rtol=2e-3)
    scores[4](xs, w1, gamma, out, m, k, n, 128, 1)
    assert [st.fn_name for st in scores.last_plan.steps] == ["asc_cuda_gemm_f16", "asc_cuda_rms_norm_f32"]
    want = s * torch.rsqrt((s * s).mean(dim=-1, keepdim=True) + 1e-6) * gamma
    torch.testing.assert_close(out, want, atol=2e-3, rtol=2e-3)
    scores[4](xs, w1, gamma, out, m, k, n, 128, 2)
    assert [st.fn_name for st in scores.last_plan.steps] == ["asc_cuda_gemm_f16", "asc_cuda_row_program"]
    torch.testing.assert_close(out, torch.softmax(s * 0.5, dim=-1), atol=1e-5, rtol=2e-3)


@pytest.mark.parametrize("m, k, n, m_tile, k_tile", [(512, 256, 128, 128, 64), (1000, 512, 272, 128, 128)])
def test_matmul_of_operands_computed_from_loaded_tiles(m, k, n, m_tile, k_tile):
    """relu(A).to(fp16) @ (B * S) over a K loop: each operand is written to a temporary by one program, then one GEMM.
    Golden: the same expression in torch on the CPU (operands rounded to fp16 exactly as the kernel rounds them)."""
    gen = torch.Generator().manual_seed(m)
    a = (torch.rand(m, k, generator=gen) - .5) * 2 * k ** -0.5
    b = (torch.rand(k, n, generator=gen) - .5).half()
    s = (torch.rand(k, n, generator=gen) + .5).half()
    c = torch.zeros(m, n)
    K.matmul_of_computed_operands[8](a, b, s, c, m, k, n, m_tile, k_tile)
    plan = K.matmul_of_computed_operands.last_plan
    assert plan.pattern == "matmul" and len(plan.temps) == 2 and plan.steps[-1].fn_name == "asc_cuda_gemm_f16"
    want = a.relu().half().float() @ (b * s).float()
    torch.testing.assert_close(c, want, atol=2e-3, rtol=2e-3)


@pytest.mark.parametrize("n, tile", [(5000, 512), (1 << 20, 4096)])
def test_quantise_and_dequantise_through_8_bit_tensors(n, tile):
    gen = torch.Generator().manual_seed(n)
    x = torch.randn(n, generator=gen) * 6
    q = torch.zeros(n, dtype=torch.int8)
    K.quantise_int8[8](x, q, 16.0, n, tile)
    want_q = torch.clamp(torch.floor(x * 16.0 + 0.5), -128, 127).to(torch.int8)
    assert torch.equal(q, want_q) and int(q.min()) == -128 and int(q.max()) == 127
    keep = (torch.rand(n, generator=gen) > 0.25).to(torch.uint8)
    back = torch.full((n, ), 7.0)
    K.dequantise_int8[8](q, keep, back, 0.0625, n, tile)
    assert torch.equal(back, torch.where(keep != 0, q.float() * 0.0625, torch.zeros(n)))
    # a kernel that writes part of an 8-bit tensor leaves the other bytes as they were
    part = torch.full((n, ), 5, dtype=torch.int8)
    K.quantise_int8[8](x, part, 16.0, n - 1000, tile)
    assert torch.equal(part[:n - 1000], want_q[:n - 1000]) and bool((part[n - 1000:] == 5).all())
    # arithmetic on 8-bit tiles is refused

    @asc2.jit
    def add_bytes(a_ptr: asc.GlobalAddress, o_ptr: asc.GlobalAddress):
        a_gm, o_gm = asc2.tensor(a_ptr, [1024]), asc2.tensor(o_ptr, [1024])
        a = asc2.load(a_gm, [1024], offsets=[0])
        asc2.store(a + a, o_gm, offsets=[0])
    with pytest.raises(NotImplementedError):
        add_bytes[1](q[:1024].clone(), torch.zeros(1024, dtype=torch.int8))


def test_launches_over_empty_tensors_do_nothing():
    for dev in ("cpu", "cuda"):
        x = torch.zeros(0, device=dev)
        K.vadd[16](x, x.clone(), x.clone(), 0, 128, 4)
        K.add_vector_bias[4](torch.zeros(0, 64, device=dev), torch.ones(64, device=dev), torch.zeros(0, 64, device=dev), 0, 64, 32)
    # tensors with elements, a length argument of 0: the output keeps its contents
    out = torch.full((256, ), 3.0)
    K.vadd[16](torch.ones(256), torch.ones(256), out, 0, 128, 4)
    assert bool((out == 3.0).all())


def test_device_tensors_that_share_a_buffer():
    """x += y through two arguments that are one device buffer works (every element is read before it is written);
    a GEMM whose output argument is also an operand argument is refused before anything is launched."""
    gen = torch.Generator().manual_seed(9)
    x, y = torch.randn(8192, generator=gen).cuda(), torch.randn(8192, generator=gen).cuda()
    want = (x + y).cpu()
    K.vadd[16](x, y, x, 8192, 128, 4)
    assert torch.equal(x.cpu(), want)
    a = torch.randn(128, 128, generator=gen).half().cuda()
    b = torch.randn(128, 128, generator=gen).half().cuda()
    before = a.clone()
    with pytest.raises(ValueError, match="overlap in device memory"):
        K.matmul_relu_cast[1](a, b, a, a.shape, b.shape, a.shape)
    assert torch.equal(a, before)


def test_matmul_stored_over_its_own_operand():
    """x = x @ w, tile by tile: every product is complete (in a temporary) before any row of x is overwritten."""
    @asc2.jit
    def in_place(a_ptr: asc.GlobalAddress, b_ptr: asc.GlobalAddress, m: asc.ConstExpr[int], k: asc.ConstExpr[int],
                 m_tile: asc.ConstExpr[int]):
        a_gm, b_gm = asc2.tensor(a_ptr, [m, k]), asc2.tensor(b_ptr, [k, k])
        for i in range(asc2.block_idx() * m_tile, m, asc2.block_num() * m_tile):
            x, y = asc2.load(a_gm, [m_tile, k], offsets=[i, 0]), asc2.load(b_gm, [k, k], offsets=[0, 0])
            asc2.store(asc2.matmul(x, y).to(asc.float16), a_gm, offsets=[i, 0])

    gen = torch.Generator().manual_seed(5)
    m, k = 2048, 1024
    a = ((torch.rand(m, k, generator=gen) - .5) * 2 * k ** -0.5).half()
    w = (torch.rand(k, k, generator=gen) - .5).half()
    want = (a.float() @ w.float()).half()
    in_place[8](a, w, m, k, 128)
    assert in_place.last_plan.pattern == "matmul+program"
    torch.testing.assert_close(a, want, atol=2e-3, rtol=2e-3)


@pytest.mark.parametrize("batch, m, n, k", [(8, 128, 256, 64), (5, 200, 144, 80), (3, 1024, 1024, 1024)])
def test_matmul_batched_loop(batch, m, n, k):
    gen = torch.Generator().manual_seed(batch * m)
    a = ((torch.rand(batch, m, k, generator=gen) - .5) * 2 * k ** -0.5).half()
    b = (torch.rand(batch, k, n, generator=gen) - .5).half()
    c = torch.zeros(batch * m, n)
    K.matmul_batched[4](a.reshape(batch * m, k), b.reshape(batch * k, n), c, batch, m, n, k)
    torch.testing.assert_close(c.reshape(batch, m, n), torch.bmm(a.float(), b.float()), atol=2e-3, rtol=2e-3)


@pytest.mark.parametrize("bias_dtype", [torch.float32, torch.float16, torch.bfloat16], ids=str)
@pytest.mark.parametrize("m, n, k, m_tile, n_tile, relu, out_dtype, torch_dtype", [
    (512, 768, 128, 128, 256, 1, asc.float16, torch.float16), (500, 704, 128, 128, 256, 0, asc.float32, torch.float32),
    (2048, 2048, 1024, 256, 512, 1, asc.bfloat16, torch.bfloat16), (96, 160, 64, 32, 32, 1, asc.float32, torch.float32)])
def test_linear_layer_tiled_over_m_and_n_with_bias_slices(m, n, k, m_tile, n_tile, relu, out_dtype, torch_dtype, bias_dtype):
    """Every tile adds its own slice of the bias vector: the tiles merge into one GEMM call with the bias row in its
    epilogue.  Golden: the expression in torch on the CPU, fp32 accumulation."""
    gen = torch.Generator().manual_seed(m + n)
    a = ((torch.rand(m, k, generator=gen) - .5) * 2 * k ** -0.5).half()
    b = (torch.rand(k, n, generator=gen) - .5).half()
    bias = torch.randn(n, generator=gen).to(bias_dtype)
    c = torch.zeros(m, n, dtype=torch_dtype)
    K.linear_mn_tiles[8](a, b, bias, c, m, n, k, m_tile, n_tile, relu, out_dtype)
    plan = K.linear_mn_tiles.last_plan
    assert plan.pattern == "matmul" and [s.fn_name for s in plan.steps] == ["asc_cuda_gemm_f16_bias"]
    t = a.float() @ b.float() + bias.float()
    t = (t.relu() if relu else t).to(torch_dtype)
    tol = 1.6e-2 if torch_dtype == torch.bfloat16 else 2e-3
    torch.testing.assert_close(c, t, atol=tol, rtol=tol)


@pytest.mark.parametrize("out_dtype, torch_dtype", [(asc.float32, torch.float32), (asc.float16, torch.float16)], ids=str)
@pytest.mark.parametrize("mode", [0, 1, 2, 3])
@pytest.mark.parametrize("m, n, k, m_tile", [(512, 256, 128, 64), (2048, 1024, 2048, 128)])
def test_matmul_bias_activation(m, n, k, m_tile, mode, out_dtype, torch_dtype):
    """A product followed by a bias row and an activation (and a residual, and a cast).  The bias row, a ReLU and the
    cast ride in the GEMM's epilogue; for any other activation the GEMM writes fp32 to a temporary and one elementwise
    program finishes the expression.  Golden: the same expression in torch on the CPU."""
    gen = torch.Generator().manual_seed(m + mode)
    a = ((torch.rand(m, k, generator=gen) - .5) * 2 * k ** -0.5).half()
    b = (torch.rand(k, n, generator=gen) - .5).half()
    bias = torch.randn(1, n, generator=gen)
    res = torch.randn(m, n, generator=gen)
    c = torch.zeros(m, n, dtype=torch_dtype)
    K.matmul_bias_act[8](a, b, bias, res, c, m, n, k, m_tile, mode, out_dtype)
    assert K.matmul_bias_act.last_plan.pattern == ("matmul" if mode < 2 else "matmul+program")
    t = a.float() @ b.float() + bias
    if mode == 1:
        t = t.relu()
    elif mode == 2:
        t = torch.where(t >= 0, t, t * 0.01)
    elif mode == 3:
        t = t - t / (torch.exp(t * (t * t * 0.0713548162726 + 1.5957691216057308)) + 1) + res
    torch.testing.assert_close(c, t.to(torch_dtype), atol=2e-3, rtol=2e-3)


@pytest.mark.parametrize("m, k, n, torch_dtype, pyasc_dtype", [(32, 64, 64, torch.float16, asc.float16),
                                                              (64, 64, 64, torch.bfloat16, asc.bfloat16)])
def test_matmul_l0c_to_l1(m, k, n, torch_dtype, pyasc_dtype):
    torch.manual_seed(0)
    a = (torch.rand((m, k), dtype=torch_dtype) - .5) * 10
    b = (torch.rand((k, n), dtype=torch_dtype) - .5) * 10
    c = torch.zeros((m, n), dtype=torch.float32)
    K.matmul_chained[1](a, b, c, a.shape, b.shape, c.shape, pyasc_dtype)
    c_ref = (a.to(torch.float32) @ b.to(torch.float32)).to(torch_dtype)
    c_ref = c_ref.to(torch.float32) @ b.to(torch.float32)
    torch.testing.assert_close(c, c_ref, atol=1e-3, rtol=1e-3)


# ------------------------------------------------------------------------- the five workload scripts
def test_workload_softmax_device_tensors_zero_copy():
    x = G.softmax_input(2048, 4096).cuda()
    out = torch.empty_like(x)
    T.softmax_launch(x, out)
    G.assert_softmax_close(out, G.softmax(x.cpu()))
    out2 = torch.empty_like(x)
    T.softmax_fused_launch(x, out2)
    assert torch.equal(out, out2)


def test_workload_vadd_host_and_device_paths_agree():
    x, y = G.vadd_inputs(1 << 22)
    out_h = torch.empty_like(x)
    T.vadd_launch(x, y, out_h, core_num=16, tile_size=4096)
    xd, yd = x.cuda(), y.cuda()
    out_d = torch.empty_like(xd)
    T.vadd_launch(xd, yd, out_d, core_num=16, tile_size=4096)
    G.assert_exact(out_h, x + y)
    G.assert_exact(out_d, x + y)
    xp, yp = x.pin_memory(), y.pin_memory()
    out_p = torch.empty_like(x).pin_memory()
    T.vadd_launch(xp, yp, out_p, core_num=16, tile_size=4096)
    G.assert_exact(out_p, x + y)


def test_workload_matmul_fp16_script():
    a, b = G.gemm_f16_inputs(1024, 1536, 2048)
    c = torch.empty(1024, 1536, dtype=torch.float16)
    T.matmul_fp16_launch(a, b, c, core_num=32)
    G.assert_half_close(c, G.gemm_f16(a, b))
    c_relu = torch.empty_like(c)
    T.matmul_fp16_launch(a, b, c_relu, core_num=32, relu=True)
    G.assert_half_close(c_relu, G.gemm_f16(a, b, relu=True))


def test_workload_matmul_int8_scripts():
    a, b, sa, sb = G.gemm_i8_inputs(512, 768, 1024)
    acc = torch.empty(512, 768, dtype=torch.int32)
    T.matmul_int8_launch(a, b, acc, core_num=8)
    ref = G.gemm_i8(a, b)
    G.assert_exact(acc, ref)
    out = torch.empty(512, 768, dtype=torch.float16)
    T.matmul_int8_dequant_launch(a, b, sa, sb, out, core_num=8)
    G.assert_exact(out, G.dequant(ref, sa, sb))


@pytest.mark.parametrize("causal", [False, True])
def test_workload_attention_script(causal):
    q, k, v = G.attention_inputs(2, 3, 512)
    o = torch.empty_like(q)
    T.attention_launch(q, k, v, o, causal=causal, core_num=24)
    G.assert_half_close(o, G.attention(q, k, v, causal))


def test_attention_stored_over_its_queries():
    """O written into Q's tensor: a query tile is read by the one CTA that later stores the same rows."""
    @asc2.jit
    def attn(q_ptr: asc.GlobalAddress, k_ptr: asc.GlobalAddress, v_ptr: asc.GlobalAddress, heads: asc.ConstExpr[int],
             seq: asc.ConstExpr[int]):
        q_gm, k_gm, v_gm = (asc2.tensor(p, [heads * seq, 128]) for p in (q_ptr, k_ptr, v_ptr))
        per_head = seq // 128
        for t in range(asc2.block_idx(), heads * per_head, asc2.block_num()):
            head_row, q_off = (t // per_head) * seq, (t % per_head) * 128
            q = asc2.load(q_gm, [128, 128], offsets=[head_row + q_off, 0])
            k = asc2.load(k_gm, [seq, 128], offsets=[head_row, 0])
            v = asc2.load(v_gm, [seq, 128], offsets=[head_row, 0])
            p = asc2.softmax(asc2.matmul(q, k, trans_b=True) * 0.08838834764831845).to(asc.float16)
            asc2.store(asc2.matmul(p, v).to(asc.float16), q_gm, offsets=[head_row + q_off, 0])

    q, k, v = G.attention_inputs(2, 40, 1024)             # 640 query tiles: several per CTA
    want = G.attention(q, k, v, False)
    qd = q.cuda()
    attn[148](qd, k.cuda(), v.cuda(), 80, 1024)
    assert attn.last_plan.pattern == "attention"
    G.assert_half_close(qd.cpu(), want)


def test_user_stream_and_profiler():
    import ctypes
    from asc.lib import runtime as rt
    from asc.lib.profiling import Profiler, task_time_median
    x, y = (t.cuda() for t in G.vadd_inputs(1 << 20))
    out = torch.empty_like(x)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        T.vadd_launch(x, y, out, core_num=16, tile_size=65536, stream=ctypes.c_void_p(stream.cuda_stream))
    stream.synchronize()
    G.assert_exact(out, x.cpu() + y.cpu())
    prof = Profiler()
    xh, yh = G.vadd_inputs(1 << 16)
    oh = torch.empty_like(xh)
    for _ in range(3):
        with prof.profile():
            T.vadd_launch(xh, yh, oh, core_num=16, tile_size=4096)
    assert task_time_median(prof.last_result.tasks, skip=1) > 0
    assert rt.launch_count() > 0


# ------------------------------------------------------------------------- chunked (pipelined) launches
def _pinned(*tensors):
    return [t.pin_memory() for t in tensors]


def test_pipelined_launch_matches_plain_launch(monkeypatch):
    """Page-locked host arguments of >= 16 MiB take the three-stream chunked path; results must be
    identical to the one-shot path and to the oracle."""
    from asc.runtime import launcher
    calls = []
    real = launcher.Launcher._run_pipelined
    monkeypatch.setattr(launcher.Launcher, "_run_pipelined", lambda self, plan, handles: (calls.append(plan.pattern),
                                                                                          real(self, plan, handles))[1])
    # softmax: 4096 x 4096 fp32
    x = G.softmax_input(4096, 4096)
    (xp, ) = _pinned(x)
    out = torch.empty_like(x).pin_memory()
    T.softmax_launch(xp, out)
    G.assert_softmax_close(out, G.softmax(x))
    plain = torch.empty_like(x)
    T.softmax_launch(x, plain)                                # pageable memory: one-shot path
    assert torch.equal(out, plain)
    # vector add with a ragged size
    n = (1 << 23) + 12345
    a, b = G.vadd_inputs(n)
    ap, bp = _pinned(a, b)
    o = torch.empty(n).pin_memory()
    T.vadd_launch(ap, bp, o, core_num=64, tile_size=1 << 14)
    G.assert_exact(o, a + b)
    # fp16 GEMM 4096 x 2048 x 2048 and int8 GEMM with dequantisation
    ga, gb = G.gemm_f16_inputs(4096, 2048, 2048)
    gap, gbp = _pinned(ga, gb)
    gc = torch.empty(4096, 2048, dtype=torch.float16).pin_memory()
    T.matmul_fp16_launch(gap, gbp, gc)
    gplain = torch.empty(4096, 2048, dtype=torch.float16)
    T.matmul_fp16_launch(ga, gb, gplain)
    assert torch.equal(gc, gplain)
    rows = torch.arange(0, 4096, 97)
    G.assert_half_close(gc[rows], G.gemm_f16(ga[rows], gb))
    ia, ib, sa, sb = G.gemm_i8_inputs(4096, 2048, 1024)
    iap, ibp, sap, sbp = _pinned(ia, ib, sa, sb)
    dq = torch.empty(4096, 2048, dtype=torch.float16).pin_memory()
    T.matmul_int8_dequant_launch(iap, ibp, sap, sbp, dq)
    G.assert_exact(dq[rows], G.dequant(G.gemm_i8(ia[rows], ib), sa[rows], sb))
    # attention 2 x 8 x 1024 x 128
    q, k, v = G.attention_inputs(2, 8, 1024)
    qp, kp, vp = _pinned(q, k, v)
    ao = torch.empty_like(q).pin_memory()
    T.attention_launch(qp, kp, vp, ao, causal=True)
    aplain = torch.empty_like(q)
    T.attention_launch(q, k, v, aplain, causal=True)
    assert torch.equal(ao, aplain)
    G.assert_half_close(ao[:, :2], G.attention(q[:, :2], k[:, :2], v[:, :2], True))
    assert calls == ["softmax", "elementwise:asc_cuda_vadd_f32", "matmul", "matmul", "attention"], calls


def test_pipelined_launch_after_a_device_reset(backend, platform, device_id):
    """``reset_device`` destroys the runtime's streams on that device, the three pipeline streams among them; the
    next chunked launch must make new ones (and new events) instead of using the destroyed handles."""
    from asc.lib import runtime as rt
    from asc.runtime import launcher
    x = G.softmax_input(2048, 4096)
    (xp, ) = _pinned(x)
    out = torch.empty_like(x).pin_memory()
    T.softmax_launch(xp, out)
    dev_id = rt.current_device()
    before = launcher._pipe_streams[dev_id]
    assert launcher._event_pool.get(dev_id)
    rt.reset_device()
    assert dev_id not in launcher._pipe_streams and not launcher._event_pool.get(dev_id)
    config.set_platform(backend, platform, device_id)
    out2 = torch.empty_like(x).pin_memory()
    T.softmax_launch(xp, out2)
    assert dev_id in launcher._pipe_streams and before is not None
    assert torch.equal(out2, out)
    G.assert_softmax_close(out2, G.softmax(x))
