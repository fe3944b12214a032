"""The asc / asc2 surface on CPU: tracing, pattern matching and launch planning without a device
(``DRY_RUN=1`` stops before the launch, as in the reference: python/asc/runtime/launcher.py:208-210),
plus the argument / option error behaviour of the reference's JITFunction and config."""
import numpy as np
import pytest
import torch

import asc
import asc2
from asc.codegen import matcher
from asc.language.core.ir_value import PlainValue
from asc.runtime import config

import asc2_scripts as K
from pyasc_b200 import tutorials as T


@pytest.fixture(autouse=True)
def dry_run(monkeypatch):
    monkeypatch.setenv("DRY_RUN", "1")


def only_step(jit_fn):
    plan = jit_fn.last_plan
    assert len(plan.steps) == 1, plan
    return plan, plan.steps[0]


# ----------------------------------------------------------------------------- scalar semantics
def test_plain_value_arithmetic_is_truncating():
    a = PlainValue.const(-7)
    assert (a // 2).value == -3 and (a / 2).value == -3 and (a % 2).value == -1   # C semantics, not Python's
    b = PlainValue.sym("block_idx")
    expr = (b * 6) % 4 + (b * 6) // 4
    vals = expr.evaluate({"block_idx": np.arange(5)})
    assert vals.tolist() == [0, 3, 3, 6, 6]
    assert asc.ceildiv(10, 4) == 3
    with pytest.raises(NotImplementedError):
        bool(b < 3)


def test_instances_and_intervals():
    ctx_loops = []
    env = matcher.enumerate_instances(3, tuple(ctx_loops))
    assert env["block_idx"].tolist() == [0, 1, 2]
    assert matcher.merge_intervals(np.array([0, 8, 4, 20]), np.array([4, 12, 8, 24])) == [(0, 12), (20, 24)]
    assert matcher.merge_intervals(np.array([5]), np.array([5])) == []


# ----------------------------------------------------------------------------- pattern matching
def test_vadd_plan_full_and_ragged():
    x = np.zeros(8192, np.float32)
    K.vadd[16](x, x, x.copy(), 8192, 128, 4)
    plan, step = only_step(K.vadd)
    assert step.fn_name == "asc_cuda_vadd_f32" and step.note == "[0, 8192)"
    assert plan.reads == {0, 1} and plan.writes == {2}
    # fewer tiles than elements: the tail stays untouched
    K.vadd[16](x, x, x.copy(), 8192, 128, 3)
    assert only_step(K.vadd)[1].note == "[0, 6144)"
    # more tiles than elements: stores are clipped to the tensor
    y = np.zeros(1000, np.float32)
    K.vadd[4](y, y, y.copy(), 1000, 128, 2)
    assert only_step(K.vadd)[1].note == "[0, 1000)"


def test_vmuladd_plan():
    x = np.zeros(8192, np.float32)
    K.vmuladd[16](x, x, x, x.copy(), 8192, 32, 16, buffer_factor=2)
    plan, step = only_step(K.vmuladd)
    assert step.fn_name == "asc_cuda_vmuladd_f32" and plan.reads == {0, 1, 2} and plan.writes == {3}


def test_softmax_plans():
    x = torch.zeros(64, 1024)
    K.softmax_rows[16](x, torch.empty_like(x), 64, 1024, tile_size=1024)
    assert only_step(K.softmax_rows)[1].note == "rows [0, 64) x 1024 cols"
    K.softmax_blocks[16](x, torch.empty_like(x), 64, 1024, 4)
    assert only_step(K.softmax_blocks)[1].note == "rows [0, 64) x 1024 cols"
    # blocks that cover only part of the rows
    K.softmax_blocks[4](x, torch.empty_like(x), 64, 1024, 4)
    assert only_step(K.softmax_blocks)[1].note == "rows [0, 16) x 1024 cols"
    # a tile wider than the row would feed zero padding into the softmax: refused, not approximated
    with pytest.raises(NotImplementedError):
        K.softmax_rows[16](x, torch.empty_like(x), 64, 1024, tile_size=2048)


@pytest.mark.parametrize("k_tiles", [2, 4, 8])
def test_matmul_k_tiled_plan(k_tiles):
    a = torch.zeros(64, 128, dtype=torch.float16)
    b = torch.zeros(128, 256, dtype=torch.float16)
    c = torch.zeros(64, 256)
    K.matmul_k_tiled[1](a, b, c, a.shape, b.shape, c.shape, k_tiles)
    _, step = only_step(K.matmul_k_tiled)
    assert step.fn_name == "asc_cuda_gemm_f16" and "C[0:64, 0:256] = A[0:, 0:128]" in step.note


@pytest.mark.parametrize("m, k, n, core_num, m_tile, n_tile, ntpb", [
    (16, 16, 16, 1, 16, 16, 1), (32, 16, 32, 2, 16, 16, 2), (32, 16, 32, 4, 16, 16, 1), (480, 224, 1344, 30, 48, 32, 7)])
def test_matmul_mn_blocked_merges_into_one_gemm(m, k, n, core_num, m_tile, n_tile, ntpb):
    a = torch.zeros(m, k, dtype=torch.float16)
    b = torch.zeros(k, n, dtype=torch.float16)
    c = torch.zeros(m, n)
    mtpb = K.mn_tiles_per_block(m, n, core_num, m_tile, n_tile, ntpb)
    K.matmul_mn_blocked[core_num](a, b, c, a.shape, b.shape, c.shape, m_tile, mtpb, n_tile, ntpb)
    _, step = only_step(K.matmul_mn_blocked)
    assert f"C[0:{m}, 0:{n}] = A[0:, 0:{k}]" in step.note


def test_matmul_epilogue_and_chain_plans():
    for dt, fn in ((torch.float32, "asc_cuda_gemm_f32"), (torch.float16, "asc_cuda_gemm_f16"),
                   (torch.bfloat16, "asc_cuda_gemm_f16")):
        a, b = torch.zeros(64, 128, dtype=dt), torch.zeros(128, 256, dtype=dt)
        c = torch.zeros(64, 256, dtype=torch.float16)
        K.matmul_relu_cast[1](a, b, c, a.shape, b.shape, c.shape)
        assert only_step(K.matmul_relu_cast)[1].fn_name == fn
    a, b = torch.zeros(32, 64, dtype=torch.float16), torch.zeros(64, 64, dtype=torch.float16)
    c = torch.zeros(32, 64)
    K.matmul_chained[1](a, b, c, a.shape, b.shape, c.shape, asc.float16)
    plan = K.matmul_chained.last_plan
    assert [s.fn_name for s in plan.steps] == ["asc_cuda_gemm_f16"] * 2 and plan.temps == {"tmp0": 32 * 64 * 2}


def test_workload_scripts_match_at_full_size():
    m = n = k = 8192
    a, b = torch.empty(m, k, dtype=torch.float16), torch.empty(k, n, dtype=torch.float16)
    c = torch.empty(m, n, dtype=torch.float16)
    T.matmul_fp16_launch(a, b, c)
    assert "C[0:8192, 0:8192] = A[0:, 0:8192]" in only_step(T.matmul_fp16_kernel)[1].note
    a8, b8 = torch.empty(m, k, dtype=torch.int8), torch.empty(k, n, dtype=torch.int8)
    T.matmul_int8_launch(a8, b8, torch.empty(m, n, dtype=torch.int32))
    assert only_step(T.matmul_int8_kernel)[1].fn_name == "asc_cuda_gemm_i8"
    T.matmul_int8_dequant_launch(a8, b8, torch.empty(m), torch.empty(n), c)
    plan, step = only_step(T.matmul_int8_dequant_kernel)
    assert step.fn_name == "asc_cuda_gemm_i8" and plan.reads == {0, 1, 2, 3} and plan.writes == {4}
    q = torch.empty(4, 32, 4096, 128, dtype=torch.float16)
    for causal in (False, True):
        T.attention_launch(q, q, q, torch.empty_like(q), causal=causal)
        assert only_step(T.attention_kernel)[1].note == f"128 heads x 4096 x 128, causal={causal}"
    s = torch.empty(16384, 4096)
    T.softmax_launch(s, torch.empty_like(s))
    assert only_step(T.softmax_kernel)[1].note == "rows [0, 16384) x 4096 cols"


def test_unsupported_pattern_raises_not_implemented():
    @asc2.jit
    def column_sums_of_squares(x_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, r: asc.ConstExpr[int],
                               c: asc.ConstExpr[int]):
        x = asc2.load(asc2.tensor(x_ptr, [r, c]), [r, c], offsets=[0, 0])
        asc2.store(asc2.reduce_sum(x * x, 0), asc2.tensor(out_ptr, [c]), offsets=[0])
    x = np.zeros((16, 64), np.int32)          # integer tiles: column reductions of computed tiles are floating-point only
    with pytest.raises(NotImplementedError, match="no kernel for this pattern"):
        column_sums_of_squares[1](x, np.zeros(64, np.int32), 16, 64)
    column_sums_of_squares[1](np.zeros((16, 64), np.float32), np.zeros(64, np.float32), 16, 64)
    assert column_sums_of_squares.last_plan.pattern == "reduce:sum:columns"

    @asc2.jit
    def bit_masked(x_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, n: asc.ConstExpr[int]):
        x = asc2.load(asc2.tensor(x_ptr, [n]), [n], offsets=[0])
        with asc2.mask(bits=(0, 0xff), other=0):          # lane masks of the Ascend vector unit: no counterpart here
            y = x + 1
        asc2.store(y, asc2.tensor(out_ptr, [n]), offsets=[0])
    with pytest.raises(NotImplementedError, match="mask"):
        bit_masked[1](np.zeros(64, np.float32), np.zeros(64, np.float32), 64)


# ----------------------------------------------------------------------------- reference error behaviour
def test_jit_option_and_argument_errors():
    with pytest.raises(RuntimeError, match="unknown"):
        asc2.jit(not_an_option=True)(lambda x_ptr: None)
    with pytest.raises(RuntimeError, match="conflict"):
        asc2.jit(lambda core_num: None)
    x = np.zeros(128, np.float32)
    with pytest.raises(ValueError, match="Core number"):
        K.vadd[0](x, x, x, 128, 128, 1)
    with pytest.raises(TypeError):
        K.vadd[1]("not a tensor", x, x, 128, 128, 1)
    with pytest.raises(RuntimeError, match="ConstExpr"):
        K.vadd[1](x, x, x, 128, 12.5, 1)
    with pytest.raises(TypeError):
        K.vadd["sixteen"]
    with pytest.raises(RuntimeError, match="aligned by 32 bytes"):
        @asc2.jit
        def bad_tile(x_ptr: asc.GlobalAddress):
            asc2.load(asc2.tensor(x_ptr, [4, 6]), [2, 6], offsets=[0, 0])
        bad_tile[1](np.zeros((4, 6), np.float32))
    with pytest.raises(ValueError, match="Exactly one"):
        @asc2.jit
        def both(x_ptr: asc.GlobalAddress):
            asc2.load(asc2.tensor(x_ptr, [8]), [8], offsets=[0], tile_id=[0])
        both[1](np.zeros(8, np.float32))


def test_matmul_argument_checks():
    @asc2.jit
    def mixed(a_ptr: asc.GlobalAddress, b_ptr: asc.GlobalAddress):
        a = asc2.load(asc2.tensor(a_ptr, [16, 16]), [16, 16], offsets=[0, 0])
        b = asc2.load(asc2.tensor(b_ptr, [16, 16]), [16, 16], offsets=[0, 0])
        a @ b
    with pytest.raises(RuntimeError, match="same types"):
        mixed[1](torch.zeros(16, 16, dtype=torch.float16), torch.zeros(16, 16))


def test_config_backend_selection():
    assert config.Backend("CUDA") is config.Backend.CUDA
    assert config.platform_to_arch(config.Platform.B200) is config.CompilationArch.SM100A
    assert config.platform_to_arch(config.Platform.Ascend950PR_9599) is config.CompilationArch.C310
    with pytest.raises(ValueError):
        config.set_platform("TPU")
    with pytest.raises(ValueError, match="not available"):
        config.set_platform("NPU")
    # no device in this process: check=True must fail loudly, check=False must not touch the device
    config.set_platform("CUDA", check=False)
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError, match="not available"):
            config.set_platform("CUDA")


def test_matmul_followed_by_an_elementwise_expression_plans_a_product_and_a_program(monkeypatch):
    """A bias row, a ReLU and a cast ride in the GEMM's epilogue (one step).  Any other activation (+ residual) after
    a matmul is not one of the GEMM epilogues: the product goes to a temporary fp32 matrix of the result's shape and
    one elementwise program reads it back."""
    monkeypatch.setenv("DRY_RUN", "1")
    import asc2_scripts as K
    m, n, k = 512, 256, 128
    a, b = torch.zeros(m, k, dtype=torch.float16), torch.zeros(k, n, dtype=torch.float16)
    for mode in (0, 1):
        for out_dtype, torch_dtype in ((asc.float32, torch.float32), (asc.float16, torch.float16)):
            K.matmul_bias_act[4](a, b, torch.zeros(1, n), torch.zeros(m, n), torch.zeros(m, n, dtype=torch_dtype), m, n, k,
                                 64, mode, out_dtype)
            plan = K.matmul_bias_act.last_plan
            assert plan.pattern == "matmul" and [s.fn_name for s in plan.steps] == ["asc_cuda_gemm_f16_bias"]
            assert plan.steps[0].note == "C[0:512, 0:256] = A[0:, 0:128] @ B[0:, 0:] + bias[0:256]"
            assert plan.reads == {0, 1, 2} and plan.writes == {4} and not plan.temps and not plan.partial_writes
            assert plan.pipeline is not None and 2 in plan.pipeline.resident
    for mode, reads in ((2, {0, 1, 2}), (3, {0, 1, 2, 3})):
        for out_dtype, torch_dtype in ((asc.float32, torch.float32), (asc.float16, torch.float16)):
            K.matmul_bias_act[4](a, b, torch.zeros(1, n), torch.zeros(m, n), torch.zeros(m, n, dtype=torch_dtype), m, n, k, 64,
                                 mode, out_dtype)
            plan = K.matmul_bias_act.last_plan
            assert plan.pattern == "matmul+program" and [s.fn_name for s in plan.steps] == \
                ["asc_cuda_gemm_f16", "asc_cuda_eltwise_program_2d"]          # the eight row blocks merge in both
            assert plan.reads == reads and plan.writes == {4} and not plan.partial_writes
            assert plan.temps == {"tmp0": m * n * 4} and plan.pipeline is None
    # several products in one expression: a temporary each, then one program over all of them
    @asc2.jit
    def products(a_ptr: asc.GlobalAddress, b_ptr: asc.GlobalAddress, c_ptr: asc.GlobalAddress, count: asc.ConstExpr[int]):
        a_gm, b_gm, c_gm = asc2.tensor(a_ptr, [64, 64]), asc2.tensor(b_ptr, [64, 64]), asc2.tensor(c_ptr, [64, 64])
        x = asc2.load(a_gm, [64, 64], offsets=[0, 0])
        y = asc2.load(b_gm, [64, 64], offsets=[0, 0])
        total = asc2.matmul(x, y)
        for scale in (2.0, 3.0, 4.0, 5.0)[:count - 1]:
            total = total + asc2.matmul(y, x) * scale
        asc2.store(total, c_gm, offsets=[0, 0])
    h = torch.zeros(64, 64, dtype=torch.float16)
    products[1](h, h, torch.zeros(64, 64), 2)
    plan = products.last_plan
    assert plan.pattern == "matmul+program" and plan.temps == {"tmp0": 64 * 64 * 4, "tmp1": 64 * 64 * 4}
    assert [s.fn_name for s in plan.steps] == ["asc_cuda_gemm_f16", "asc_cuda_gemm_f16", "asc_cuda_eltwise_program"]
    assert plan.reads == {0, 1} and plan.writes == {2}
    with pytest.raises(NotImplementedError, match="more than 4 matmul results"):
        products[1](h, h, torch.zeros(64, 64), 5)

    # a fused row kernel over the product: the product reads like a loaded tile once it is in its temporary
    @asc2.jit
    def product_softmax(a_ptr: asc.GlobalAddress, b_ptr: asc.GlobalAddress, c_ptr: asc.GlobalAddress):
        a_gm, b_gm, c_gm = asc2.tensor(a_ptr, [128, 64]), asc2.tensor(b_ptr, [64, 256]), asc2.tensor(c_ptr, [128, 256])
        for i in range(asc2.block_idx() * 64, 128, asc2.block_num() * 64):
            s = asc2.matmul(asc2.load(a_gm, [64, 64], offsets=[i, 0]), asc2.load(b_gm, [64, 256], offsets=[0, 0]))
            asc2.store(asc2.softmax(s), c_gm, offsets=[i, 0])
    product_softmax[2](torch.zeros(128, 64, dtype=torch.float16), torch.zeros(64, 256, dtype=torch.float16), torch.zeros(128, 256))
    plan = product_softmax.last_plan
    assert plan.pattern == "matmul+program" and [s.fn_name for s in plan.steps] == ["asc_cuda_gemm_f16", "asc_cuda_softmax_f32"]
    assert plan.steps[0].note == "C[0:128, 0:256] = A[0:, 0:64] @ B[0:, 0:]" and plan.temps == {"tmp0": 128 * 256 * 4}


def test_bias_slices_of_an_mn_tiled_linear_layer_merge_or_stay_per_tile(monkeypatch):
    monkeypatch.setenv("DRY_RUN", "1")
    import asc2_scripts as K
    h = torch.float16
    a, b = torch.zeros(512, 128, dtype=h), torch.zeros(128, 768, dtype=h)
    for bias_dtype in (torch.float32, torch.float16, torch.bfloat16):
        K.linear_mn_tiles[8](a, b, torch.zeros(768, dtype=bias_dtype), torch.zeros(512, 768, dtype=h), 512, 768, 128,
                             128, 256, 1, asc.float16)
        plan = K.linear_mn_tiles.last_plan        # the tiles form a grid and every tile's bias slice starts at its column
        assert plan.pattern == "matmul" and [s.note for s in plan.steps] == \
            ["C[0:512, 0:768] = A[0:, 0:128] @ B[0:, 0:] + bias[0:768]"]
    # ragged edges: 500 x 700 in 128 x 256 tiles is still one call, clipped to the tensor
    K.linear_mn_tiles[8](torch.zeros(500, 128, dtype=h), torch.zeros(128, 704, dtype=h), torch.zeros(704),
                         torch.zeros(500, 704), 500, 704, 128, 128, 256, 0, asc.float32)
    assert [s.note for s in K.linear_mn_tiles.last_plan.steps] == ["C[0:500, 0:704] = A[0:, 0:128] @ B[0:, 0:] + bias[0:704]"]

    # a bias row that is not the tile's own columns of one vector: per-tile calls, each with its own slice
    @asc2.jit
    def shifted_bias(a_ptr: asc.GlobalAddress, b_ptr: asc.GlobalAddress, bias_ptr: asc.GlobalAddress, c_ptr: asc.GlobalAddress):
        a_gm, b_gm, c_gm = asc2.tensor(a_ptr, [128, 64]), asc2.tensor(b_ptr, [64, 512]), asc2.tensor(c_ptr, [128, 512])
        bias_gm = asc2.tensor(bias_ptr, [2, 256])
        for j in range(2):
            x = asc2.load(a_gm, [128, 64], offsets=[0, 0])
            y = asc2.load(b_gm, [64, 256], offsets=[0, 256 * j])
            row = asc2.load(bias_gm, [1, 256], offsets=[1 - j, 0])
            asc2.store(asc2.matmul(x, y) + row.broadcast_to(128, 256), c_gm, offsets=[0, 256 * j])
    shifted_bias[1](torch.zeros(128, 64, dtype=h), torch.zeros(64, 512, dtype=h), torch.zeros(2, 256), torch.zeros(128, 512))
    assert [s.note for s in shifted_bias.last_plan.steps] == [
        "C[0:128, 0:256] = A[0:, 0:64] @ B[0:, 0:] + bias[256:512]",
        "C[0:128, 256:512] = A[0:, 0:64] @ B[0:, 256:] + bias[0:256]"]

    # a bias tile that reaches past its vector would add zero padding: neither the epilogue nor a program reads that
    @asc2.jit
    def padded_bias(a_ptr: asc.GlobalAddress, b_ptr: asc.GlobalAddress, bias_ptr: asc.GlobalAddress, c_ptr: asc.GlobalAddress):
        a_gm, b_gm, c_gm = asc2.tensor(a_ptr, [128, 64]), asc2.tensor(b_ptr, [64, 256]), asc2.tensor(c_ptr, [128, 256])
        row = asc2.load(asc2.tensor(bias_ptr, [1, 200]), [1, 256], offsets=[0, 0])
        x, y = asc2.load(a_gm, [128, 64], offsets=[0, 0]), asc2.load(b_gm, [64, 256], offsets=[0, 0])
        asc2.store(asc2.matmul(x, y) + row.broadcast_to(128, 256), c_gm, offsets=[0, 0])
    with pytest.raises(NotImplementedError, match="bias row that reaches past the end of its tensor"):
        padded_bias[1](torch.zeros(128, 64, dtype=h), torch.zeros(64, 256, dtype=h), torch.zeros(1, 200),
                       torch.zeros(128, 256))


def test_matmul_stored_into_its_own_operand_goes_through_a_temporary(monkeypatch):
    """Tiles of one GEMM call run concurrently, so a product may not land in a tensor the call reads: with a cast
    around it the product goes to a temporary first (every tile done before the program stores), bare it is refused;
    so is a bias row taken from the output tensor."""
    monkeypatch.setenv("DRY_RUN", "1")
    h = torch.float16

    @asc2.jit
    def in_place(a_ptr: asc.GlobalAddress, b_ptr: asc.GlobalAddress, cast: asc.ConstExpr[int], dtype: asc.ConstExpr):
        a_gm, b_gm = asc2.tensor(a_ptr, [256, 128]), asc2.tensor(b_ptr, [128, 128])
        for i in range(2):
            x, y = asc2.load(a_gm, [128, 128], offsets=[128 * i, 0]), asc2.load(b_gm, [128, 128], offsets=[0, 0])
            v = asc2.matmul(x, y)
            asc2.store(v.to(dtype) if cast else v, a_gm, offsets=[128 * i, 0])
    in_place[1](torch.zeros(256, 128, dtype=h), torch.zeros(128, 128, dtype=h), 1, asc.float16)
    plan = in_place.last_plan
    assert plan.pattern == "matmul+program" and plan.temps == {"tmp0": 256 * 128 * 4} and plan.writes == {0}
    assert [s.fn_name for s in plan.steps] == ["asc_cuda_gemm_f16", "asc_cuda_eltwise_program"]
    with pytest.raises(NotImplementedError, match="stored into one of its own operands"):
        in_place[1](torch.zeros(256, 128), torch.zeros(128, 128), 0, asc.float32)

    @asc2.jit
    def bias_from_the_output(a_ptr: asc.GlobalAddress, b_ptr: asc.GlobalAddress, c_ptr: asc.GlobalAddress):
        a_gm, b_gm, c_gm = asc2.tensor(a_ptr, [128, 64]), asc2.tensor(b_ptr, [64, 256]), asc2.tensor(c_ptr, [128, 256])
        row = asc2.load(c_gm, [1, 256], offsets=[5, 0])
        x, y = asc2.load(a_gm, [128, 64], offsets=[0, 0]), asc2.load(b_gm, [64, 256], offsets=[0, 0])
        asc2.store(asc2.matmul(x, y) + row.broadcast_to(128, 256), c_gm, offsets=[0, 0])
    with pytest.raises(NotImplementedError, match="bias row loaded from the tensor the product is stored to"):
        bias_from_the_output[1](torch.zeros(128, 64, dtype=h), torch.zeros(64, 256, dtype=h), torch.zeros(128, 256))


def test_matmul_operands_computed_from_loaded_tiles_are_written_to_temporaries(monkeypatch):
    monkeypatch.setenv("DRY_RUN", "1")
    import asc2_scripts as K
    h = torch.float16
    K.matmul_of_computed_operands[4](torch.zeros(512, 256), torch.zeros(256, 128, dtype=h), torch.zeros(256, 128, dtype=h),
                                     torch.zeros(512, 128), 512, 256, 128, 128, 64)
    plan = K.matmul_of_computed_operands.last_plan
    # one program per operand over the whole matrix (every block's and iteration's tile), then one product
    assert plan.pattern == "matmul" and plan.temps == {"tmp0": 512 * 256 * 2, "tmp1": 256 * 128 * 2}
    assert [s.fn_name for s in plan.steps] == ["asc_cuda_eltwise_program", "asc_cuda_eltwise_program", "asc_cuda_gemm_f16"]
    assert plan.steps[0].note.endswith("over [0, 131072)") and plan.steps[1].note.endswith("over [0, 32768)")
    assert plan.steps[2].note == "C[0:512, 0:128] = A[0:, 0:256] @ B[0:, 0:]"
    assert plan.reads == {0, 1, 2} and plan.writes == {3}

    # an operand normalised by its row maximum: a row program writes the temporary
    @asc2.jit
    def reduced_operand(a_ptr: asc.GlobalAddress, b_ptr: asc.GlobalAddress, c_ptr: asc.GlobalAddress):
        a_gm, b_gm, c_gm = asc2.tensor(a_ptr, [64, 64]), asc2.tensor(b_ptr, [64, 64]), asc2.tensor(c_ptr, [64, 64])
        x = asc2.load(a_gm, [64, 64], offsets=[0, 0])
        col = asc2.reduce_max(x, 1, keep_dims=True).broadcast_to(64, 64)
        asc2.store(asc2.matmul((x / col).to(asc.float16), asc2.load(b_gm, [64, 64], offsets=[0, 0])), c_gm, offsets=[0, 0])
    reduced_operand[1](torch.zeros(64, 64), torch.zeros(64, 64, dtype=h), torch.zeros(64, 64))
    assert [s.fn_name for s in reduced_operand.last_plan.steps] == ["asc_cuda_row_program", "asc_cuda_gemm_f16"]


def test_batched_matmul_loop_plans_one_product_per_matrix(monkeypatch):
    """B stacked along its rows: the K range of B starts at another row than the K range of A starts at a column."""
    monkeypatch.setenv("DRY_RUN", "1")
    import asc2_scripts as K
    a, b = torch.zeros(8 * 128, 64, dtype=torch.float16), torch.zeros(8 * 64, 256, dtype=torch.float16)
    K.matmul_batched[4](a, b, torch.zeros(8 * 128, 256), 8, 128, 256, 64)
    plan = K.matmul_batched.last_plan
    assert plan.pattern == "matmul" and len(plan.steps) == 8
    assert [s.note for s in plan.steps[:2]] == ["C[0:128, 0:256] = A[0:, 0:64] @ B[0:, 0:]",
                                                "C[128:256, 0:256] = A[128:, 0:64] @ B[64:, 0:]"]


def test_k_loop_accumulator_with_an_epilogue_and_windows_of_a_wider_matrix(monkeypatch):
    monkeypatch.setenv("DRY_RUN", "1")
    import asc2_scripts as K
    h = torch.float16
    K.matmul_k_tiled_bias_relu[1](torch.zeros(128, 512, dtype=h), torch.zeros(512, 128, dtype=h), torch.zeros(1, 128),
                                  torch.zeros(128, 128), 128, 128, 512, 128)
    plan = K.matmul_k_tiled_bias_relu.last_plan            # the K loop folds into one product of K = 512
    assert plan.pattern == "matmul" and [s.fn_name for s in plan.steps] == ["asc_cuda_gemm_f16_bias"]
    assert plan.steps[0].note == "C[0:128, 0:128] = A[0:, 0:512] @ B[0:, 0:] + bias[0:128]"
    # the two halves of every row: operand windows with the pitch of the wide matrix, a contiguous result
    K.glu_rows[4](torch.zeros(256, 1024), torch.zeros(256, 512), 256, 512, 8)
    plan = K.glu_rows.last_plan
    assert plan.pattern == "elementwise:program" and len(plan.steps) == 1 and not plan.partial_writes
    assert plan.steps[0].note.endswith("over [256, 512] pitches [1024, 1024, 512] from [0, 512] to 0")


def test_whole_tile_reduction_as_an_operand_and_a_reshaped_bias_vector(monkeypatch):
    monkeypatch.setenv("DRY_RUN", "1")
    import asc2_scripts as K
    x = torch.zeros(256, 64)
    K.tile_over_its_own_reduction[4](x, torch.zeros(64), torch.zeros_like(x), 256, 64, 32, asc2.reduce_max)
    plan = K.tile_over_its_own_reduction.last_plan
    # a [32, 64] tile is walked as one row of 2048 elements, so that the reduction spans the whole tile
    assert plan.pattern == "row:program" and len(plan.steps) == 1
    assert " over [8, 2048] " in plan.steps[0].note
    K.add_vector_bias[4](x, torch.zeros(64), torch.zeros_like(x), 256, 64, 32)
    plan = K.add_vector_bias.last_plan
    assert plan.pattern == "elementwise:program" and plan.steps[0].note.endswith("pitches [64, 0, 64] from [0, 0] to 0")
    # a tile that is a window of a wider matrix cannot be walked as one row
    @asc2.jit
    def windowed(x_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress):
        x_gm, out_gm = asc2.tensor(x_ptr, [64, 128]), asc2.tensor(out_ptr, [64, 128])
        t = asc2.load(x_gm, [64, 64], offsets=[0, 64])
        asc2.store(t / asc2.reduce_max(t), out_gm, offsets=[0, 64])
    with pytest.raises(NotImplementedError):
        windowed[1](torch.zeros(64, 128), torch.zeros(64, 128))


def test_copy_of_tiles_of_types_the_programs_do_not_compute_on(monkeypatch):
    monkeypatch.setenv("DRY_RUN", "1")
    import asc2_scripts as K
    x = torch.zeros(64, 256, dtype=torch.int8)
    K.copy_window[4](x, torch.zeros(64, 512, dtype=torch.int8), 64, 256, 512, 128, 64, 32, 8)
    plan = K.copy_window.last_plan
    assert plan.pattern == "copy" and plan.reads == {0} and plan.writes == {1} and plan.partial_writes == {1}
    (step, ) = plan.steps                                     # the eight row blocks continue each other
    assert step.fn_name == "asc_cuda_copy_2d" and step.note == "[64, 128] int8 from 64 to 32"
    built = step.build({0: 1 << 20, 1: 2 << 20}, None)
    assert [a.value for a in built[:6]] == [(2 << 20) + 32, (1 << 20) + 64, 64, 128, 512, 256]
    d = torch.zeros(64, 128, dtype=torch.float64)
    K.copy_window[4](d, torch.zeros_like(d), 64, 128, 128, 128, 0, 0, 8)
    plan = K.copy_window.last_plan                            # whole matrices: one contiguous move, a full write
    assert plan.steps[0].note == "[8, 1024] float64 from 0 to 0" and not plan.partial_writes
    # a float32 copy stays with the elementwise program
    f = torch.zeros(64, 128)
    K.copy_window[4](f, torch.zeros_like(f), 64, 128, 128, 128, 0, 0, 8)
    assert K.copy_window.last_plan.pattern == "elementwise:program"


def test_atomic_accumulation_of_row_reductions(monkeypatch):
    monkeypatch.setenv("DRY_RUN", "1")
    import asc2_scripts as K
    K.split_row_reduce[4](torch.zeros(64, 2048), torch.zeros(64), 64, 2048, 256, asc2.reduce_sum, asc2.atomic_add)
    plan = K.split_row_reduce.last_plan
    assert plan.pattern == "atomic:add" and len(plan.steps) == 8 and plan.reads == {0, 1} and plan.writes == {1}
    assert all(s.fn_name == "asc_cuda_row_program" for s in plan.steps)
    # x, x, MUL, ROW_SUM, the row's element of the target, ADD: one stored element per row
    assert list(plan.steps[0].build({0: 0, 1: 0}, None)[0]) == [0, 0, 4, 59, 0, 2]


def test_statistics_down_the_columns_plan_reductions_into_temporaries_then_one_program(monkeypatch):
    monkeypatch.setenv("DRY_RUN", "1")
    import asc2_scripts as K
    x = torch.zeros(4 * 64, 256)
    K.column_softmax[2](x, torch.zeros_like(x), 4, 64, 256)
    plan = K.column_softmax.last_plan
    assert plan.pattern == "column:statistics" and plan.reads == {0} and plan.writes == {1}
    assert plan.temps == {"tmp0": 4 * 64 * 256 * 4, "tmp1": 4 * 64 * 256 * 4}
    # per tile: the maximum (a loaded fp32 tile: the reduction kernel), the sum of exp(x - max) (a column program
    # that reads the maximum back as a broadcast row), the quotient (an elementwise program with two broadcast rows)
    assert [s.fn_name for s in plan.steps] == ["asc_cuda_reduce_f32"] * 4 + ["asc_cuda_col_program"] * 4 + \
        ["asc_cuda_eltwise_program_2d"] * 4
    K.column_standardise[2](x.half(), torch.zeros_like(x).half(), 4, 64, 256, 1e-5)
    plan = K.column_standardise.last_plan
    assert plan.pattern == "column:statistics" and len(plan.temps) == 2
    assert [s.fn_name for s in plan.steps] == ["asc_cuda_col_program"] * 8 + ["asc_cuda_eltwise_program_2d"] * 4


def test_explain_lists_the_library_calls_of_a_launch(monkeypatch, capsys):
    monkeypatch.setenv("DRY_RUN", "1")
    import asc2_scripts as K
    x = torch.zeros(4 * 64, 256)
    K.column_softmax[2](x, torch.zeros_like(x), 4, 64, 256, print_ir_before_all=True)     # the reference's option
    err = capsys.readouterr().err
    assert "kernel 'column_softmax' -> column:statistics: 12 call(s)" in err and "temporary tmp0: 262144 bytes" in err
    text = K.column_softmax.explain()
    assert text.splitlines()[3].strip() == "asc_cuda_reduce_f32: max axis 0 of [64, 256] at (0, 0) -> [0, +256)"


def test_device_arguments_that_share_a_buffer():
    """An output argument may be the buffer of an input argument only for kernels that read an element (or its row)
    before they write it; overlapping views and GEMM / attention / reduction outputs over their inputs are refused."""
    from asc.codegen.matcher import Plan
    from asc.runtime.launcher import Launcher
    from asc.runtime.memory_handle import TorchCudaTensorArgument as Dev
    buf = torch.zeros(4096)
    x, y, shifted, other = Dev(buf[:2048]), Dev(buf[:2048]), Dev(buf[1024:3072]), Dev(torch.zeros(2048))

    def plan(pattern, reads, writes):
        p = Plan(pattern)
        p.reads.update(reads)
        p.writes.update(writes)
        return p
    check = Launcher._check_device_aliasing
    for pattern in ("elementwise:vadd", "elementwise:program", "row:program", "softmax", "rms_norm"):
        check(plan(pattern, {0, 1}, {2}), {0: x, 1: other, 2: y})                 # x += other
    check(plan("matmul", {0, 1}, {2}), {0: x, 1: x, 2: other})                     # inputs may alias each other
    check(plan("matmul", {0}, {2}), {0: other, 1: y, 2: y})                        # argument 1 is not used by the plan
    for pattern in ("matmul", "matmul+program", "attention", "reduce:sum", "copy", "atomic:add", "elementwise:program+matmul"):
        with pytest.raises(ValueError, match="overlap in device memory"):
            check(plan(pattern, {0, 1}, {2}), {0: x, 1: other, 2: y})
    with pytest.raises(ValueError, match="overlap in device memory"):              # a shifted view: never
        check(plan("elementwise:program", {0}, {1}), {0: x, 1: shifted})
    with pytest.raises(ValueError, match="overlap in device memory"):              # two outputs in one buffer
        check(plan("elementwise:program", {0}, {1, 2}), {0: other, 1: x, 2: y})


def test_attention_stored_into_its_own_keys_is_refused():
    """Every query tile reads all keys and values of its head while other tiles already store: O may be Q's tensor
    (a tile reads its own queries before it stores), not K's or V's."""
    def make(out_name):
        @asc2.jit
        def attn(q_ptr: asc.GlobalAddress, k_ptr: asc.GlobalAddress, v_ptr: asc.GlobalAddress):
            gm = {n: asc2.tensor(p, [512, 128]) for n, p in (("q", q_ptr), ("k", k_ptr), ("v", v_ptr))}
            for t in range(asc2.block_idx(), 4, asc2.block_num()):
                q = asc2.load(gm["q"], [128, 128], offsets=[t * 128, 0])
                k = asc2.load(gm["k"], [512, 128], offsets=[0, 0])
                v = asc2.load(gm["v"], [512, 128], offsets=[0, 0])
                p = asc2.softmax(asc2.matmul(q, k, trans_b=True) * 0.125).to(asc.float16)
                asc2.store(asc2.matmul(p, v).to(asc.float16), gm[out_name], offsets=[t * 128, 0])
        return attn
    x = torch.zeros(512, 128, dtype=torch.float16)
    attn = make("q")
    attn[4](x, x.clone(), x.clone())
    assert attn.last_plan.pattern == "attention" and attn.last_plan.writes == {0}
    for name in ("k", "v"):
        with pytest.raises(NotImplementedError, match="attention stored into its own K or V"):
            make(name)[4](x, x.clone(), x.clone())


def test_per_row_results_of_one_row_tiles_arrive_as_scalar_stores():
    """reduce(...) of a [1, cols] tile has one element, which asc2.store records as a scalar store: still one value
    per row of a row program, and the 64 one-row tiles merge into one call."""
    x = torch.zeros(64, 512)
    K.row_losses[8](x, x, torch.zeros(64), torch.zeros(64), 64, 512)
    plan = K.row_losses.last_plan
    assert plan.pattern == "row:program+row:program" and [s.fn_name for s in plan.steps] == ["asc_cuda_row_program"] * 2
    assert all(" over [64, 512] " in s.note for s in plan.steps) and plan.reads == {0, 1} and plan.writes == {2, 3}


def test_8_bit_tensors_are_loaded_compared_and_stored_not_computed_on():
    n = 5000
    # the kernels compute on 32- and 16-bit types: 8-bit tensors are widened into (narrowed out of) int32 temporaries
    K.quantise_int8[4](torch.zeros(n), torch.zeros(n, dtype=torch.int8), 8.0, n, 512)
    plan = K.quantise_int8.last_plan
    assert plan.pattern == "elementwise:program" and plan.temps == {"wide1": 4 * n} and not plan.partial_writes
    assert [s.fn_name for s in plan.steps] == ["asc_cuda_eltwise_program", "asc_cuda_convert_bytes"]
    assert plan.steps[0].note.endswith("over [0, 5000)") and plan.reads == {0} and plan.writes == {1}
    K.quantise_int8[4](torch.zeros(n), torch.zeros(n, dtype=torch.int8), 8.0, n - 1000, 512)       # part of the output only
    plan = K.quantise_int8.last_plan
    assert [s.fn_name for s in plan.steps] == ["asc_cuda_convert_bytes", "asc_cuda_eltwise_program", "asc_cuda_convert_bytes"]
    assert plan.partial_writes == {1}
    K.dequantise_int8[4](torch.zeros(n, dtype=torch.int8), torch.zeros(n, dtype=torch.uint8), torch.zeros(n), 0.125, n, 512)
    plan = K.dequantise_int8.last_plan
    assert [s.fn_name for s in plan.steps] == ["asc_cuda_convert_bytes"] * 2 + ["asc_cuda_eltwise_program"]
    assert plan.pattern == "elementwise:program" and plan.reads == {0, 1} and plan.writes == {2} and plan.pipeline is None

    @asc2.jit
    def add_bytes(a_ptr: asc.GlobalAddress, o_ptr: asc.GlobalAddress, form: asc.ConstExpr[int]):
        a_gm, o_gm = asc2.tensor(a_ptr, [1024]), asc2.tensor(o_ptr, [1024])
        a = asc2.load(a_gm, [1024], offsets=[0])
        if form == 0:
            asc2.store(a + a, o_gm, offsets=[0])                                       # would need a wrap per operation
        elif form == 1:
            asc2.store((a.to(asc.int32) * 3).to(asc.int8), o_gm, offsets=[0])          # computed as int32, low byte stored
        else:
            asc2.store(a, o_gm, offsets=[0])                                           # a move of bytes
    b = torch.zeros(1024, dtype=torch.int8)
    with pytest.raises(NotImplementedError):
        add_bytes[1](b, b.clone(), 0)
    add_bytes[1](b, b.clone(), 1)
    assert add_bytes.last_plan.pattern == "elementwise:program"
    add_bytes[1](b, b.clone(), 2)
    assert add_bytes.last_plan.pattern == "copy"


def test_softmax_of_a_computed_tile_is_spelled_out_as_a_row_program():
    x = torch.zeros(64, 1024)
    K.softmax_with_temperature[8](x, torch.zeros(1, 1024), torch.zeros_like(x), 0.5, 64, 1024, 4)
    plan, step = only_step(K.softmax_with_temperature)
    assert plan.pattern == "row:program" and step.fn_name == "asc_cuda_row_program" and " over [64, 1024] " in step.note
    assert plan.reads == {0, 1} and plan.writes == {2}


def test_ragged_last_tiles_of_kernels_whose_operands_are_addressed_differently():
    """A row count that is no multiple of the tile: the last tile reaches past the tensors, its store is clipped
    and the call is cut to the rows that exist.  An operand that ends before the result would bring zero padding
    into stored elements: refused."""
    x = torch.zeros(100, 64)
    K.add_vector_bias[4](x, torch.zeros(64), torch.zeros_like(x), 100, 64, 32)
    assert only_step(K.add_vector_bias)[1].note == "3 ops over [100, 64] pitches [64, 0, 64] from [0, 0] to 0"
    x = torch.zeros(100, 1000)
    K.softmax_with_temperature[8](x, torch.zeros(1, 1000), torch.zeros_like(x), 0.5, 100, 1000, 8)
    assert " over [100, 1000] " in only_step(K.softmax_with_temperature)[1].note
    K.glu_rows[4](torch.zeros(100, 1024), torch.zeros(100, 512), 100, 512, 8)
    assert " over [100, 512] pitches [1024, 1024, 512] " in only_step(K.glu_rows)[1].note

    @asc2.jit
    def shifted(x_ptr: asc.GlobalAddress, y_ptr: asc.GlobalAddress, o_ptr: asc.GlobalAddress, n: int, extra: asc.ConstExpr[int],
                tile: asc.ConstExpr[int]):
        x_gm, y_gm, o_gm = asc2.tensor(x_ptr, [n + extra]), asc2.tensor(y_ptr, [n]), asc2.tensor(o_ptr, [n])
        for i in range(asc2.block_idx() * tile, n, asc2.block_num() * tile):
            asc2.store(asc2.load(x_gm, [tile], offsets=[i + extra]) + asc2.load(y_gm, [tile], offsets=[i]), o_gm, offsets=[i])
    shifted[2](torch.zeros(1008), torch.zeros(1000), torch.zeros(1000), 1000, 8, 256)
    assert [s.note for s in shifted.last_plan.steps] == [
        "3 ops over [3, 256] pitches [256, 256, 256] from [8, 0] to 0",
        "3 ops over [1, 232] pitches [256, 256, 256] from [776, 768] to 768"]
    with pytest.raises(NotImplementedError, match="zero padding would be computed on"):
        _short_operand()


def _short_operand():
    @asc2.jit
    def short(x_ptr: asc.GlobalAddress, y_ptr: asc.GlobalAddress, o_ptr: asc.GlobalAddress, n: int, tile: asc.ConstExpr[int]):
        x_gm, y_gm, o_gm = asc2.tensor(x_ptr, [n - 8]), asc2.tensor(y_ptr, [n]), asc2.tensor(o_ptr, [n])
        for i in range(asc2.block_idx() * tile, n, asc2.block_num() * tile):
            asc2.store(asc2.load(x_gm, [tile], offsets=[i]) + asc2.load(y_gm, [tile], offsets=[i]), o_gm, offsets=[i])
    short[2](torch.zeros(992), torch.zeros(1000), torch.zeros(1000), 1000, 256)


def test_empty_tensors_plan_no_calls():
    """A launch over tensors without elements (or whose every tile lies outside): nothing to do, as on the reference,
    where the blocks' loops simply do not run."""
    x = np.zeros(0, np.float32)
    K.vadd[16](x, x, x.copy(), 0, 128, 4)
    assert K.vadd.last_plan.steps == []
    K.add_vector_bias[4](torch.zeros(0, 64), torch.zeros(64), torch.zeros(0, 64), 0, 64, 32)
    assert K.add_vector_bias.last_plan.steps == [] and K.add_vector_bias.last_plan.writes == {2}
    K.row_losses[8](torch.zeros(0, 512), torch.zeros(0, 512), torch.zeros(0), torch.zeros(0), 0, 512)
    assert K.row_losses.last_plan.steps == []
    K.copy_window[4](torch.zeros(0, 64, dtype=torch.int8), torch.zeros(0, 64, dtype=torch.int8), 0, 64, 64, 64, 0, 0, 8)
    assert K.copy_window.last_plan.steps == []
