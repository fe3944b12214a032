"""Row programs on the GPU: asc2 kernels that reduce their own intermediate tiles along the row, against torch,
and the C-ABI entry point against the CPU oracle's evaluation of the same program."""
import ctypes

import numpy as np
import pytest
import torch

import asc
import asc.runtime.config as config
import asc2

import asc2_scripts as K
from oracle import eltwise as E
from pyasc_b200 import capi

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def platform():
    config.set_platform(config.Backend.CUDA, config.Platform.B200, 0)


@pytest.mark.parametrize("rows, cols, block, blocks", [(64, 512, 8, 4), (256, 4096, 4, 16), (32, 8, 8, 2),
                                                       (48, 1000, 2, 3), (100, 512, 8, 4), (5, 1024, 4, 16)])
def test_layer_norm(rows, cols, block, blocks):
    gen = torch.Generator().manual_seed(rows + cols)
    x = torch.randn(rows, cols, generator=gen) * 2 + 1
    gamma, beta = torch.rand(1, cols, generator=gen) + 0.5, torch.randn(1, cols, generator=gen)
    out = torch.zeros_like(x)
    K.layer_norm_rows[blocks](x, gamma, beta, out, rows, cols, block, 1e-5)
    ref = torch.nn.functional.layer_norm(x, (cols, ), gamma[0], beta[0], 1e-5)
    torch.testing.assert_close(out, ref, rtol=1e-4, atol=1e-5)


def test_l1_normalize_and_row_results():
    gen = torch.Generator().manual_seed(9)
    x = torch.randn(96, 2048, generator=gen)
    out = torch.zeros_like(x)
    K.l1_normalize_rows[8](x, out, 96, 2048)
    torch.testing.assert_close(out, x / (x.abs().sum(1, keepdim=True) + 1e-6), rtol=1e-5, atol=1e-7)
    xd = torch.randn(512, 384, device="cuda")
    res = torch.zeros(512, device="cuda")
    K.row_sum_of_squares[16](xd, res, 512, 384, 8)
    torch.testing.assert_close(res, xd.pow(2).sum(1).sqrt() * 0.5 + xd.abs().amax(1), rtol=1e-5, atol=1e-6)


def test_scalar_store_of_reductions_of_a_computed_row():
    x = torch.randn(200, 1024, generator=torch.Generator().manual_seed(12))
    out = torch.zeros(200)
    K.row_norms_scalar[8](x, out, 200, 1024)
    torch.testing.assert_close(out, x.pow(2).sum(1) / 1024 + x.abs().amax(1), rtol=1e-5, atol=1e-6)


def test_losses_per_row_from_one_row_tiles():
    gen = torch.Generator().manual_seed(14)
    x = torch.randn(300, 1000, generator=gen) * 3
    t = torch.softmax(torch.randn(300, 1000, generator=gen), dim=1)
    mse, ce = torch.zeros(300), torch.zeros(300)
    K.row_losses[16](x, t, mse, ce, 300, 1000)
    assert K.row_losses.last_plan.pattern == "row:program+row:program"
    torch.testing.assert_close(mse, (x - t).pow(2).mean(1), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(ce, torch.logsumexp(x, 1) - (x * t).sum(1), rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("rows, cols, rpt", [(64, 1024, 4), (104, 1000, 8), (16, 4096, 1), (100, 1000, 8), (7, 512, 16)])
def test_softmax_of_a_computed_tile(rows, cols, rpt):
    gen = torch.Generator().manual_seed(rows)
    x = torch.randn(rows, cols, generator=gen) * 4
    bias = torch.randn(1, cols, generator=gen)
    out = torch.zeros_like(x)
    K.softmax_with_temperature[8](x, bias, out, 0.7, rows, cols, rpt)
    assert K.softmax_with_temperature.last_plan.pattern == "row:program"
    torch.testing.assert_close(out, torch.softmax(x * 0.7 + bias, dim=1), rtol=1e-5, atol=1e-8)


@pytest.mark.parametrize("rows", [96, 100, 5])
def test_loaded_columns_repeat_along_the_row(rows):
    """Also with a row count that is no multiple of the 8-row tile: the last tile's rows past the end are left out."""
    gen = torch.Generator().manual_seed(13)
    x, scale, bias = torch.randn(rows, 640, generator=gen), torch.randn(rows, generator=gen), torch.randn(rows, generator=gen)
    out = torch.zeros_like(x)
    K.scale_rows[4](x, scale, bias, out, rows, 640, 8)
    assert torch.equal(out, x * scale[:, None] + bias[:, None])


# ------------------------------------------------------------------------------- C ABI
@pytest.fixture(scope="module")
def lib():
    torch.cuda.set_device(0)
    return capi.load()


def f32_word(v: float) -> int:
    return int(torch.tensor([v], dtype=torch.float32).view(torch.int32)[0])


# LOAD x, ROW_MAX, LOAD x, RSUB (x - max), EXP, the same five again, ROW_SUM, DIV, LOAD y, MUL:
# exp(x - max) / sum(exp(x - max)) * y
SOFTMAX_TIMES_Y = ([0, 60, 0, 54, 11, 0, 60, 0, 54, 11, 59, 5, 0, 4],
                   [0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 1, 0])


def run_row_program(lib, ops, args, inputs, out, rows, cols, lds, row_result, expect=0, flags=None):
    n_in = len(inputs)
    ops_arr = (ctypes.c_int32 * len(ops))(*ops)
    args_arr = (ctypes.c_int32 * len(ops))(*args)
    ins = (ctypes.c_void_p * max(1, n_in))(*[t.data_ptr() for t in inputs])
    types = (ctypes.c_int32 * max(1, n_in))(*[{torch.float32: 0, torch.float16: 1}[t.dtype] | (flags[i] if flags else 0)
                                              for i, t in enumerate(inputs)])
    lds_arr = (ctypes.c_int64 * len(lds))(*lds) if lds is not None else None
    rc = lib.asc_cuda_row_program(ops_arr, args_arr, len(ops), ins, types, n_in, ctypes.c_void_p(out.data_ptr()),
                                  {torch.float32: 0, torch.float16: 1}[out.dtype], rows, cols, lds_arr, row_result, None)
    assert rc == expect, f"returned {rc}: {capi.status_string(rc)} {capi.last_cuda_error()}"
    if rc == 0:
        capi.check_device_status(None)


@pytest.mark.parametrize("rows, cols, pad", [(1, 1, 0), (5, 33, 0), (300, 256, 0), (129, 1000, 24), (64, 4096, 0),
                                             (33, 8192, 0), (16384, 4096, 0)])
def test_capi_row_program_against_oracle(lib, rows, cols, pad):
    """Every lane count of the kernel (1 to 32 elements per thread), ragged rows, pitched operands, a broadcast
    row, and a 256 MiB window (beyond L2)."""
    gen = torch.Generator(device="cuda").manual_seed(rows * 3 + cols)
    ld = cols + pad
    xbuf = torch.randn(rows, ld, device="cuda", generator=gen)
    y = torch.rand(cols, device="cuda", generator=gen) + 0.5
    out = torch.full((rows, ld), -3.0, device="cuda")
    ops, args = SOFTMAX_TIMES_Y
    run_row_program(lib, ops, args, [xbuf, y], out, rows, cols, [ld, 0, ld], 0)
    x = xbuf[:, :cols]
    if rows * cols <= (1 << 22):
        ref = E.run_program(ops, args, [x.cpu(), y.cpu().expand(rows, cols)], 0)
        torch.testing.assert_close(out[:, :cols].cpu(), ref, rtol=2e-5, atol=1e-7)
    torch.testing.assert_close(out[:, :cols], torch.softmax(x, 1) * y, rtol=2e-5, atol=1e-7)
    assert pad == 0 or bool((out[:, cols:] == -3.0).all())


@pytest.mark.parametrize("cols", [200, 500, 1000, 2048, 4096, 8192])
def test_capi_row_program_every_stack_depth_and_temporary_count(lib, cols):
    """Stack depths 2 to 8 with 0 to 4 temporaries at every lane count: shared memory from nothing to beyond the
    200 KiB the kernel accepts (status 6), through the 48 KiB above which a launch has to opt in."""
    rows = 24
    gen = torch.Generator().manual_seed(cols)
    x = torch.rand(rows, cols, generator=gen) + 0.5
    xd = x.cuda()
    per_thread = -(-cols // 256)
    lanes = 1
    while lanes < per_thread:
        lanes *= 2
    for depth in range(2, 9):
        for n_tmp in range(0, 5):
            # x, kept in n_tmp slots; then depth loads folded from the top (x * (x + (x * ...))); the slots added; x / row sum
            ops = [0] + [63] * n_tmp + [0] * (depth - 1) + [4 if k % 2 else 2 for k in range(depth - 1)]
            args = [0] + list(range(n_tmp)) + [0] * (2 * (depth - 1))
            for k in range(n_tmp):
                ops += [64, 2]
                args += [k, 0]
            ops += [59, 0, 55]                  # ROW_SUM, LOAD x, RDIV: x / sum
            args += [0, 0, 0]
            smem = (max(depth - 2, 1) + n_tmp) * lanes * 256 * 4
            out = torch.zeros(rows, cols, device="cuda")
            run_row_program(lib, ops, args, [xd], out, rows, cols, None, 0, expect=6 if smem > 200 * 1024 else 0)
            if smem <= 200 * 1024:
                want = E.run_program(ops, args, [x], 0)
                torch.testing.assert_close(out.cpu(), want, rtol=1e-5, atol=1e-30, msg=lambda m: f"depth {depth}, {n_tmp} slots: {m}")


def test_capi_row_result_and_fp16_operands(lib):
    x = torch.randn(1000, 777, device="cuda").half()
    out = torch.zeros(1000, device="cuda")
    # LOAD 0, LOAD 0, MUL, ROW_SUM: sum of squares of fp16 rows, one fp32 value per row
    run_row_program(lib, [0, 0, 4, 59], [0, 0, 0, 0], [x], out, 1000, 777, None, 1)
    torch.testing.assert_close(out, x.float().pow(2).sum(1), rtol=1e-5, atol=1e-5)
    # ROW_MIN / ROW_PROD with an immediate: min(x) * prod(1 + 0 * x) == min(x)
    out2 = torch.zeros(1000, device="cuda")
    run_row_program(lib, [0, 61, 0, 4 | 0x100, 2 | 0x100, 62, 4], [0, 0, 0, f32_word(0.0), f32_word(1.0), 0, 0], [x], out2,
                    1000, 777, None, 1)
    torch.testing.assert_close(out2, x.float().amin(1), rtol=0, atol=0)


def test_capi_temporaries(lib):
    """TEE / TMP: (x - mean) computed once and used three times, as the launcher compiles a layer norm."""
    x = torch.randn(77, 3000, device="cuda") * 3 + 2
    out = torch.zeros_like(x)
    inv_c = f32_word(1.0 / 3000)
    # LOAD x, LOAD x, ROW_SUM, * 1/C, SUB, TEE 0, TMP 0, MUL, ROW_SUM, * 1/C, + eps, RSQRT, TMP 0, MUL
    ops = [0, 0, 59, 4 | 0x100, 3, 63, 64, 4, 59, 4 | 0x100, 2 | 0x100, 16, 64, 4]
    args = [0, 0, 0, inv_c, 0, 0, 0, 0, 0, inv_c, f32_word(1e-5), 0, 0, 0]
    run_row_program(lib, ops, args, [x], out, 77, 3000, None, 0)
    torch.testing.assert_close(out, torch.nn.functional.layer_norm(x, (3000, ), eps=1e-5), rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(out.cpu(), E.run_program(ops, args, [x.cpu()], 0), rtol=1e-4, atol=1e-5)


def test_capi_row_uniform_values(lib):
    """Values that are the same for the whole row (constants, reductions and functions of them) take a
    once-per-row path in the kernel; mixed with per-element operands and a select they must still be exact."""
    x = torch.randn(40, 1500, device="cuda")
    out = torch.zeros_like(x)
    # LOAD x, 0 > x (immediate), CONST 2, SQRT, LOAD x, ROW_MAX, ADD -> u = sqrt(2) + max(x), TEE 0, LOAD x, MUL,
    # TMP 0, WHERE: x < 0 ? x * u : u
    ops = [0, 28 | 0x100, 1, 15, 0, 60, 2, 63, 0, 4, 64, 32]
    args = [0, f32_word(0.0), f32_word(2.0), 0, 0, 0, 0, 0, 0, 0, 0, 0]
    run_row_program(lib, ops, args, [x], out, 40, 1500, None, 0)
    ref = E.run_program(ops, args, [x.cpu()], 0)
    u = torch.sqrt(torch.tensor(2.0)) + x.cpu().amax(1, keepdim=True)
    torch.testing.assert_close(ref, torch.where(x.cpu() < 0, x.cpu() * u, u.expand_as(x.cpu())), rtol=1e-6, atol=1e-6)
    torch.testing.assert_close(out.cpu(), ref, rtol=1e-6, atol=1e-6)


def test_capi_one_element_per_row_inputs(lib):
    """Input type bit 0x200: a column of a matrix (pitch 8) and a contiguous vector, each read once per row."""
    x = torch.randn(300, 777, device="cuda")
    m = torch.randn(300, 8, device="cuda")
    v = torch.randn(300, device="cuda")
    out = torch.zeros_like(x)
    # LOAD x, LOAD column, MUL, LOAD vector, ADD
    run_row_program(lib, [0, 0, 4, 0, 2], [0, 1, 0, 2, 0], [x, m, v], out, 300, 777, [777, 8, 1, 777], 0, flags=[0, 0x200, 0x200])
    assert torch.equal(out, x * m[:, :1] + v[:, None])
    # the elementwise entry point does not know the flag
    ops_arr, args_arr = (ctypes.c_int32 * 1)(0), (ctypes.c_int32 * 1)(0)
    ins, types = (ctypes.c_void_p * 1)(x.data_ptr()), (ctypes.c_int32 * 1)(0x200)
    assert lib.asc_cuda_eltwise_program(ops_arr, args_arr, 1, ins, types, 1, ctypes.c_void_p(out.data_ptr()), 0, 64, None) == 1


def test_capi_row_program_rejections(lib):
    x = torch.zeros(4, 16, device="cuda")
    out = torch.zeros(4, 16, device="cuda")
    run_row_program(lib, [0, 59], [0, 0], [x], out, 4, 8193 * 4, None, 0, expect=6)       # row too long for one SM
    run_row_program(lib, [0, 59], [0, 0], [x], out, 4, 16, [8, 16], 0, expect=1)          # pitch below the row length
    run_row_program(lib, [0, 65], [0, 0], [x], out, 4, 16, None, 0, expect=1)             # no such opcode
    run_row_program(lib, [0, 64, 2], [0, 0, 0], [x], out, 4, 16, None, 0, expect=1)       # temporary read before written
    run_row_program(lib, [0, 63], [0, 4], [x], out, 4, 16, None, 0, expect=1)             # no such temporary slot
    # the elementwise entry point refuses row opcodes
    ops_arr, args_arr = (ctypes.c_int32 * 2)(0, 59), (ctypes.c_int32 * 2)(0, 0)
    ins, types = (ctypes.c_void_p * 1)(x.data_ptr()), (ctypes.c_int32 * 1)(0)
    assert lib.asc_cuda_eltwise_program(ops_arr, args_arr, 2, ins, types, 1, ctypes.c_void_p(out.data_ptr()), 0, 64, None) == 1


def test_golden_fixture_normalisations(golden_dir):
    import os
    import numpy as np
    d = np.load(os.path.join(golden_dir, "normalisation.npz"))
    x, gamma, beta = (torch.from_numpy(d[k]) for k in ("x", "gamma", "beta"))
    eps = float(d["eps"])
    out = torch.zeros_like(x)
    K.rms_norm_rows[2](x, gamma.reshape(1, -1), out, 8, 512, 4, eps)
    torch.testing.assert_close(out, torch.from_numpy(d["rms_norm"]), rtol=1e-5, atol=1e-6)
    out = torch.zeros_like(x)
    K.layer_norm_rows[2](x, gamma.reshape(1, -1), beta.reshape(1, -1), out, 8, 512, 4, eps)
    torch.testing.assert_close(out, torch.from_numpy(d["layer_norm"]), rtol=1e-5, atol=2e-6)


# ------------------------------------------------------------------------------- random programs
def _random_row_program(rng, n_inputs):
    """A random valid row program over fp32 words: arithmetic, comparisons, selects and immediates as in the
    elementwise fuzz, plus row maxima / minima of subexpressions and temporaries (all exact operations, so the
    device must agree with the oracle bit for bit)."""
    binary = [2, 3, 4, 6, 7, 54]
    unary = [8, 9, 10, 24, 25]
    compare = [26, 27, 28, 29, 30, 31]
    code = []
    slots = []

    def const():
        return f32_word(float(np.float32(rng.uniform(-2, 2))))

    def gen(depth):
        kind = int(rng.integers(0, 9)) if depth > 0 else 0
        if kind == 0:
            code.append((0, int(rng.integers(0, n_inputs))))
        elif kind == 1:
            gen(depth - 1)
            code.append((int(rng.choice(unary)), 0))
        elif kind == 2:
            gen(depth - 1)
            gen(depth - 1)
            code.append((int(rng.choice(binary)), 0))
        elif kind == 3:
            gen(depth - 1)
            code.append((int(rng.choice(binary)) | 0x100, const()))
        elif kind == 4:
            gen(depth - 1)
            gen(depth - 1)
            code.append((int(rng.choice(compare)), 0))
            gen(depth - 1)
            gen(depth - 1)
            code.append((32, 0))
        elif kind in (5, 6):
            gen(depth - 1)
            code.append((int(rng.choice([60, 61])), 0))          # ROW_MAX / ROW_MIN
        elif kind == 7 and len(slots) < 4:
            gen(depth - 1)
            slots.append(len(slots))
            code.append((63, slots[-1]))                          # TEE
        elif kind == 8 and slots:
            code.append((64, int(rng.choice(slots))))             # TMP
        else:
            code.append((1, const()))
    gen(4)
    return [c[0] for c in code], [c[1] for c in code]


@pytest.mark.parametrize("seed", range(32))
def test_random_row_programs_bit_exact(lib, seed):
    import numpy as np
    rng = np.random.default_rng(1000 + seed)
    n_inputs = int(rng.integers(1, 4))
    ops, args = _random_row_program(rng, n_inputs)
    depth = peak = 0
    for op in ops:
        code, imm = op & 0xff, bool(op & 0x100)
        depth += 1 if code in (0, 1, 64) else -2 if code == 32 else 0 if imm or code in (8, 9, 10, 24, 25, 60, 61, 63) else -1
        peak = max(peak, depth)
    if len(ops) > 48 or peak > 8:
        pytest.skip("program beyond the documented limits")
    rows = int(rng.choice([1, 3, 70]))
    cols = int(rng.choice([1, 37, 256, 1000, 4096, 5000]))
    gen = torch.Generator().manual_seed(seed)
    inputs = [torch.rand(rows, cols, generator=gen) * 8 - 4 for _ in range(n_inputs)]
    want = E.run_program(ops, args, inputs, 0)
    out = torch.zeros(rows, cols, device="cuda")
    run_row_program(lib, ops, args, [t.cuda() for t in inputs], out, rows, cols, None, 0)
    assert torch.equal(out.cpu(), want), f"{ops} {args}"


@pytest.mark.parametrize("rows, cols", [(64, 512), (256, 4096), (48, 1000), (8, 8192)])
def test_row_programs_built_at_first_use_equal_the_interpreter(rows, cols, monkeypatch):
    """The first launches of a new row program run in the interpreter while nvcc builds the kernel specialised for
    it; the specialised kernel then gives bit-identical results (same arithmetic, same reduction order)."""
    from pyasc_b200 import jit
    if jit.compiler() is None:
        pytest.skip("no nvcc on this machine")
    gen = torch.Generator().manual_seed(rows + cols)
    x = (torch.randn(rows, cols, generator=gen) * 2 + 1).cuda()
    gamma, beta = (torch.rand(1, cols, generator=gen) + 0.5).cuda(), torch.randn(1, cols, generator=gen).cuda()
    lib = capi.load()

    def run():
        out = torch.zeros_like(x)
        K.layer_norm_rows[8](x, gamma, beta, out, rows, cols, 4, 1e-5)
        torch.cuda.synchronize()
        return out

    monkeypatch.setenv("ASC_CUDA_JIT", "0")
    assert lib.asc_cuda_eltwise_set_lanes(0x100) == 0           # the interpreter, whatever is registered already
    try:
        plain = run()
    finally:
        assert lib.asc_cuda_eltwise_set_lanes(0) == 0
    monkeypatch.setenv("ASC_CUDA_JIT", "sync")
    fast = run()
    (step, ) = K.layer_norm_rows.last_plan.steps
    assert jit.request(*step.program), jit.failures()            # registered by the launch itself
    assert torch.equal(fast, plain)
    ref = torch.nn.functional.layer_norm(x, (cols, ), gamma[0], beta[0], 1e-5)
    torch.testing.assert_close(fast, ref, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("op, torch_op", [(asc2.reduce_max, torch.amax), (asc2.reduce_sum, torch.sum)],
                         ids=lambda v: getattr(v, "__name__", ""))
def test_tile_divided_by_a_reduction_of_the_whole_tile(op, torch_op):
    """`x / reduce(x)` on multi-row tiles: each [32, 64] tile is walked as one row of 2048 elements."""
    gen = torch.Generator().manual_seed(5)
    x = torch.rand(256, 64, generator=gen) + 0.5
    out = torch.zeros_like(x)
    K.tile_over_its_own_reduction[4](x, torch.zeros(64), out, 256, 64, 32, op)
    tiles = x.reshape(8, 32 * 64)
    want = (tiles / torch_op(tiles, 1, keepdim=True)).reshape(256, 64)
    torch.testing.assert_close(out, want, rtol=2e-6, atol=0)


@pytest.mark.parametrize("rows", [256, 100, 33, 7])
def test_vector_bias_reshaped_to_a_row(rows):
    """Also with a row count that is no multiple of the 32-row tile: the last tile is cut to the rows that exist."""
    gen = torch.Generator().manual_seed(6)
    x, b = torch.randn(rows, 64, generator=gen), torch.randn(64, generator=gen)
    out = torch.full((rows + 4, 64), 9.0)
    K.add_vector_bias[4](x, b, out[:rows], rows, 64, 32)
    assert torch.equal(out[:rows], x + b) and bool((out[rows:] == 9.0).all())


def test_ragged_last_tiles_with_shifted_and_strided_operands():
    gen = torch.Generator().manual_seed(8)
    x = torch.randn(100, 1024, generator=gen)
    out = torch.zeros(100, 512)
    K.glu_rows[4](x, out, 100, 512, 8)
    torch.testing.assert_close(out, x[:, :512] / (torch.exp(-x[:, 512:]) + 1), rtol=2e-6, atol=1e-6)

    @asc2.jit
    def shifted(x_ptr: asc.GlobalAddress, y_ptr: asc.GlobalAddress, o_ptr: asc.GlobalAddress, n: int, tile: asc.ConstExpr[int]):
        x_gm, y_gm, o_gm = asc2.tensor(x_ptr, [n + 8]), asc2.tensor(y_ptr, [n]), asc2.tensor(o_ptr, [n])
        for i in range(asc2.block_idx() * tile, n, asc2.block_num() * tile):
            asc2.store(asc2.load(x_gm, [tile], offsets=[i + 8]) + asc2.load(y_gm, [tile], offsets=[i]), o_gm, offsets=[i])
    for n in (1000, 5, 256):
        a, b = torch.randn(n + 8, generator=gen), torch.randn(n, generator=gen)
        o = torch.full((n + 3, ), 9.0)
        shifted[2](a, b, o[:n], n, 256)
        assert torch.equal(o[:n], a[8:] + b) and bool((o[n:] == 9.0).all())


@pytest.mark.parametrize("op, atomic, torch_op", [(asc2.reduce_sum, asc2.atomic_add, torch.sum),
                                                  (asc2.reduce_max, asc2.atomic_max, torch.amax),
                                                  (asc2.reduce_min, asc2.atomic_min, torch.amin)],
                         ids=lambda v: getattr(v, "__name__", ""))
def test_row_reductions_split_over_column_blocks_accumulate_atomically(op, atomic, torch_op):
    gen = torch.Generator().manual_seed(8)
    x = torch.randn(64, 2048, generator=gen)
    start = {asc2.atomic_add: 0.5, asc2.atomic_max: 0.0, asc2.atomic_min: 100.0}[atomic]
    out = torch.full((64, ), start)
    K.split_row_reduce[4](x, out, 64, 2048, 256, op, atomic)
    sq = x * x
    if atomic is asc2.atomic_add:
        torch.testing.assert_close(out, sq.sum(1) + start, rtol=1e-5, atol=1e-5)
    elif atomic is asc2.atomic_max:
        assert torch.equal(out, torch.maximum(sq.amax(1), torch.tensor(start)))
    else:
        # the minimum of the per-block minima of x * x, and of the starting value
        assert torch.equal(out, torch.minimum(sq.reshape(64, 8, 256).amin(2).amin(1), torch.tensor(start)))
