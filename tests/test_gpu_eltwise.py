"""The generic elementwise kernel on the GPU: the reference's operation and kernel tests run through
the asc2 surface (python/test/asc2/operations/test_{binary_ops,unary_ops,where}.py,
python/test/asc2/kernels/test_{leaky_relu,gelu}.py: same shapes, distributions, goldens, tolerances),
and the C-ABI entry point itself against the CPU oracle's evaluation of the same program at sizes
beyond L2.  Bit-exact for arithmetic, comparisons, selects and roundings; transcendental functions
within atol 1e-3 of torch's CPU result as in the reference's tests."""
import ctypes

import numpy as np
import pytest
import torch

import asc
import asc.runtime.config as config
import asc2

import asc2_scripts as K
import eltwise_cases as C
from oracle import eltwise as E
from pyasc_b200 import capi

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def select_platform(backend, platform, device_id):
    config.set_platform(backend, platform, device_id)


def check(out, golden):
    assert out.dtype == golden.dtype
    if golden.dtype == torch.float32:
        assert torch.allclose(out, golden, atol=1e-3)
    else:
        assert torch.equal(out, golden)


# ------------------------------------------------------------------------------- asc2 surface
@pytest.mark.parametrize("asc_op, torch_op, fmt, dtype", C.BINARY_CASES, ids=C.ids)
def test_binary_operations(asc_op, torch_op, fmt, dtype):
    launch, golden, _ = C.binary_case(asc_op, torch_op, fmt, dtype)
    check(launch(), golden)


@pytest.mark.parametrize("asc_op, torch_op", C.UNARY_OPS, ids=C.ids)
def test_unary_operations(asc_op, torch_op):
    launch, golden, _ = C.unary_case(asc_op, torch_op)
    check(launch(), golden)


@pytest.mark.parametrize("scalar", [False, True], ids=["tile", "scalar"])
@pytest.mark.parametrize("dtype", C.WHERE_DTYPES, ids=str)
@pytest.mark.parametrize("asc_op, torch_op", C.COMPARE_OPS, ids=C.ids)
def test_where_ops(asc_op, torch_op, dtype, scalar):
    launch, golden, _ = C.where_case(asc_op, torch_op, dtype, scalar)
    torch.testing.assert_close(launch(), golden, rtol=0, atol=0)


def test_leaky_relu():
    launch, golden, _ = C.leaky_relu_case()
    torch.testing.assert_close(launch(), golden)
    assert torch.equal(launch(), golden)          # one rounded multiply and a select: exact in bf16


@pytest.mark.parametrize("approximate", [True, False])
def test_gelu(approximate):
    launch, golden, _ = C.gelu_case(approximate)
    torch.testing.assert_close(launch(), golden, rtol=1e-3, atol=1e-5)


def test_gelu_pinned_pipelined_matches_plain():
    """64 MiB of page-locked input takes the chunked three-stream launch path."""
    gen = torch.Generator().manual_seed(11)
    x = torch.rand((16384, 1024), dtype=torch.float32, generator=gen)
    plain = torch.empty_like(x)
    K.gelu[16](x, plain, 16384, 1024, 1024, False)
    xp, outp = x.pin_memory(), torch.empty_like(x).pin_memory()
    K.gelu[16](xp, outp, 16384, 1024, 1024, False)
    assert torch.equal(outp, plain)
    torch.testing.assert_close(plain, C.gelu_torch(x, False), rtol=1e-3, atol=1e-5)


# ------------------------------------------------------------------------------- C ABI
@pytest.fixture(scope="module")
def lib():
    torch.cuda.set_device(0)
    return capi.load()


def call(lib, ops, args, inputs, out, out_type, n, expect=0):
    ops_a = (ctypes.c_int32 * len(ops))(*ops)
    args_a = (ctypes.c_int32 * len(ops))(*args)
    ins = (ctypes.c_void_p * max(1, len(inputs)))(*[t.data_ptr() for t in inputs])
    code = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2, torch.int32: 3, torch.int16: 4}
    types = (ctypes.c_int32 * max(1, len(inputs)))(*[code[t.dtype] for t in inputs])
    rc = lib.asc_cuda_eltwise_program(ops_a, args_a, len(ops), ins, types, len(inputs),
                                      ctypes.c_void_p(out.data_ptr()), out_type, n, None)
    assert rc == expect, f"returned {rc}: {capi.status_string(rc)} {capi.last_cuda_error()}"
    if rc == 0:
        capi.check_device_status(None)


def fbits(v):
    return int(np.array([v], dtype=np.float32).view(np.int32)[0])


# x * y + 0.25 - max(x, y), every op rounded through the tensor type
def _arith_program(round_op):
    r = [(round_op, 0)] if round_op else []
    prog = [(0, 0), (0, 1), (4, 0)] + r + [(1, fbits(0.25)), (2, 0)] + r + [(0, 0), (0, 1), (6, 0)] + r + [(3, 0)] + r
    return [p[0] for p in prog], [p[1] for p in prog]


@pytest.mark.parametrize("dtype, round_op, out_type", [(torch.float32, None, 0), (torch.float16, 33, 1),
                                                       (torch.bfloat16, 34, 2)], ids=str)
@pytest.mark.parametrize("n, offset", [(1, 0), (5, 0), (4099, 0), (4099, 1), ((1 << 25) + 3, 0), ((1 << 22) + 1, 3)])
def test_program_arithmetic_bit_exact(lib, dtype, round_op, out_type, n, offset):
    """Sizes around the group-of-four path and its tail, beyond L2 (2 x 128 MiB fp32 in, 128 MiB out),
    and bases that are not aligned to four elements (scalar path)."""
    gen = torch.Generator().manual_seed(n + offset)
    x = (torch.rand(n + offset, generator=gen) * 8 - 4).to(dtype)
    y = (torch.rand(n + offset, generator=gen) * 8 - 4).to(dtype)
    xd, yd = x.cuda(), y.cuda()
    out = torch.zeros(n + offset + 1, dtype=dtype, device="cuda")
    ops, args = _arith_program(round_op)
    call(lib, ops, args, [xd[offset:], yd[offset:]], out[offset:], out_type, n)
    want = E.run_program(ops, args, [x[offset:], y[offset:]], out_type)
    got = out.cpu()
    assert torch.equal(got[offset:offset + n], want)
    assert got[offset + n] == 0 and bool((got[:offset] == 0).all())        # nothing written outside [0, n)


def test_program_integer_ops_wrap_like_torch(lib):
    gen = torch.Generator().manual_seed(3)
    x = torch.randint(-2**31, 2**31 - 1, (100003, ), dtype=torch.int64, generator=gen).to(torch.int32)
    y = torch.randint(-2**31, 2**31 - 1, (100003, ), dtype=torch.int64, generator=gen).to(torch.int32)
    # (x + y) * 3 - min(x, y), then >> 2, then where(x > y, that, -that)
    prog = [(0, 0), (0, 1), (35, 0), (1, 3), (37, 0), (0, 0), (0, 1), (39, 0), (36, 0), (1, 2), (41, 0)]
    body_ops, body_args = [p[0] for p in prog], [p[1] for p in prog]
    ops = [0, 0, 44] + body_ops + body_ops + [48, 32]
    args = [0, 1, 0] + body_args + body_args + [0, 0]
    out = torch.zeros(100003, dtype=torch.int32, device="cuda")
    call(lib, ops, args, [x.cuda(), y.cuda()], out, 3, 100003)
    assert torch.equal(out.cpu(), E.run_program(ops, args, [x, y], 3))
    # int16: wrap after the multiply
    a = torch.randint(-2**15, 2**15 - 1, (4100, ), dtype=torch.int32, generator=gen).to(torch.int16)
    ops16, args16 = [0, 1, 37, 53], [0, 7, 0, 0]
    out16 = torch.zeros(4100, dtype=torch.int16, device="cuda")
    call(lib, ops16, args16, [a.cuda()], out16, 4, 4100)
    assert torch.equal(out16.cpu(), a * 7)


@pytest.mark.parametrize("n, offset", [(4099, 0), (4096, 3), ((1 << 20) + 8, 0), (7, 1), (0, 0)])
def test_bytes_widened_to_words_and_back(lib, n, offset):
    """asc_cuda_convert_bytes: int8 / uint8 -> int32 (sign / zero extension) and int32 -> its low byte, at aligned
    and misaligned byte addresses, writing nothing outside the range."""
    gen = torch.Generator().manual_seed(n + 1)
    s8 = torch.randint(-128, 128, (n + offset, ), generator=gen).to(torch.int8).cuda()
    u8 = torch.randint(0, 256, (n + offset, ), generator=gen).to(torch.uint8).cuda()
    words = torch.randint(-2**31, 2**31 - 1, (n, ), dtype=torch.int64, generator=gen).to(torch.int32).cuda()
    P = lambda t: ctypes.c_void_p(t.data_ptr())
    for src, mode in ((s8, 0), (u8, 1)):
        out = torch.full((n + 1, ), 77, dtype=torch.int32, device="cuda")
        assert lib.asc_cuda_convert_bytes(P(out), P(src[offset:]), n, mode, None) == 0
        assert torch.equal(out[:n], src[offset:].to(torch.int32)) and int(out[n]) == 77
    for dtype in (torch.int8, torch.uint8):
        out = torch.full((n + offset + 1, ), 77, dtype=dtype, device="cuda")
        assert lib.asc_cuda_convert_bytes(P(out[offset:]), P(words), n, 2, None) == 0
        assert torch.equal(out[offset:offset + n], words.to(dtype)) and int(out[offset + n]) == 77 and bool((out[:offset] == 77).all())
    capi.check_device_status(None)
    if n:
        assert lib.asc_cuda_convert_bytes(P(words), P(s8), n, 3, None) == 1                 # no such mode
        assert lib.asc_cuda_convert_bytes(ctypes.c_void_p(words.data_ptr() + 2), P(s8), 1, 0, None) == 2     # misaligned words


def test_program_max_min_relu_propagate_nan(lib):
    """torch.maximum / minimum / relu return NaN when an operand is NaN (fmaxf would return the other operand);
    the same holds for a maximum reduced along the rows of a row program."""
    gen = torch.Generator().manual_seed(9)
    x = torch.randn(4099, generator=gen)
    y = torch.randn(4099, generator=gen)
    x[::7] = float("nan")
    y[3::11] = float("nan")
    xd, yd = x.cuda(), y.cuda()
    out = torch.zeros_like(xd)
    for ops, args, ins, cpu_ins in (([0, 0, 6], [0, 1, 0], [xd, yd], [x, y]), ([0, 0, 7], [0, 1, 0], [xd, yd], [x, y]),
                                    ([0, 10], [0, 0], [xd], [x]), ([0, 6 | 0x100], [0, fbits(0.5)], [xd], [x])):
        call(lib, ops, args, ins, out, 0, 4099)
        want = E.run_program(ops, args, cpu_ins, 0)
        got = out.cpu()
        assert torch.equal(got.isnan(), want.isnan()) and bool(want.isnan().any())
        assert torch.equal(got[~want.isnan()], want[~want.isnan()])


def test_program_transcendentals_close_to_cpu(lib):
    gen = torch.Generator().manual_seed(5)
    x = torch.rand(1 << 20, generator=gen) * 4 + 0.5
    xd = x.cuda()
    out = torch.empty_like(xd)
    for op in range(11, 24):
        call(lib, [0, op], [0, 0], [xd], out, 0, x.numel())
        want = E.run_program([0, op], [0, 0], [x], 0)
        torch.testing.assert_close(out.cpu(), want, rtol=2e-6, atol=1e-6, msg=lambda m: f"opcode {op}: {m}")


IMM = 0x100


@pytest.mark.parametrize("name, dtype, out_type, ops, imms", [
    ("leaky_relu", torch.float32, 0, [0, 31 | IMM, 0, 0, 4 | IMM, 32], {1: 0.0, 4: 0.1}),
    ("leaky_relu", torch.float16, 1, [0, 31 | IMM, 0, 0, 4 | IMM, 33, 32], {1: 0.0, 4: 0.1}),
    ("leaky_relu", torch.bfloat16, 2, [0, 31 | IMM, 0, 0, 4 | IMM, 34, 32], {1: 0.0, 4: 0.1}),
    ("gelu_erf", torch.float32, 0, [0, 0, 4 | IMM, 23, 2 | IMM, 4, 4 | IMM], {2: 0.5 ** 0.5, 4: 1.0, 6: 0.5}),
    ("gelu_tanh", torch.float32, 0, [0, 0, 4, 4 | IMM, 2 | IMM, 0, 4, 11, 2 | IMM, 0, 55, 0, 54],
     {3: 0.0713548, 4: 1.5957691, 8: 1.0}),
    ("sigmoid", torch.float32, 0, [0, 8, 11, 2 | IMM, 5 | IMM], {3: 1.0, 4: 1.0}),
    ("silu", torch.float32, 0, [0, 0, 8, 11, 2 | IMM, 5], {4: 1.0}),
], ids=lambda v: str(v) if isinstance(v, (str, torch.dtype)) else "")
def test_compiled_programs_equal_the_interpreter(lib, name, dtype, out_type, ops, imms):
    """The programs that have a compile-time specialised kernel must give bit-identical results in both
    executors (same per-op arithmetic), at a ragged size beyond L2, and agree with the CPU oracle."""
    n = (1 << 25) + 1029
    gen = torch.Generator().manual_seed(17)
    x = (torch.rand(n, generator=gen) * 6 - 3).to(dtype)
    xd = x.cuda()
    args = [fbits(imms[k]) if k in imms else 0 for k in range(len(ops))]
    if dtype != torch.float32:                       # scalars take the tile's type
        args = [fbits(float(torch.tensor(imms[k]).to(dtype))) if k in imms else 0 for k in range(len(ops))]
    compiled = torch.zeros(n, dtype=dtype, device="cuda")
    interpreted = torch.zeros(n, dtype=dtype, device="cuda")
    before = capi.launch_count()
    call(lib, ops, args, [xd], compiled, out_type, n)
    try:
        lib.asc_cuda_eltwise_set_lanes(0x100)        # interpreter only
        call(lib, ops, args, [xd], interpreted, out_type, n)
    finally:
        lib.asc_cuda_eltwise_set_lanes(0)
    assert capi.launch_count() == before + 2
    assert torch.equal(compiled, interpreted)
    want = E.run_program(ops, args, [x], out_type)
    if name == "leaky_relu":
        assert torch.equal(compiled.cpu(), want)
    else:
        torch.testing.assert_close(compiled.cpu(), want, rtol=1e-5, atol=1e-6)


def test_program_immediates_and_swapped_forms(lib):
    gen = torch.Generator().manual_seed(23)
    x = torch.rand(70001, generator=gen) * 4 - 2
    y = torch.rand(70001, generator=gen) * 4 + 1
    xd, yd = x.cuda(), y.cuda()
    out = torch.empty_like(xd)
    # (3 - x) / y  as  LOAD x, SUB|IMM 3, LOAD y, DIV ;  (x - 3) as RSUB|IMM ; y / x as [x, y] RDIV
    for ops, args, want in [
        ([0, 3 | IMM, 0, 5], [0, fbits(3.0), 1, 0], (3.0 - x) / y),
        ([0, 54 | IMM], [0, fbits(3.0)], x - 3.0),
        ([0, 0, 55], [0, 1, 0], y / x),
        ([0, 0, 54], [0, 1, 0], y - x),
        ([0, 30 | IMM], [0, fbits(0.5)], (0.5 < x).float()),
    ]:
        call(lib, ops, args, [xd, yd], out, 0, 70001)
        assert torch.equal(out.cpu(), want), ops
        assert torch.equal(E.run_program(ops, args, [x, y], 0), want), ops
    xi = torch.randint(-1000, 1000, (70001, ), dtype=torch.int32, generator=gen)
    oi = torch.zeros(70001, dtype=torch.int32, device="cuda")
    for ops, args, want in [([0, 57 | IMM], [0, 3], xi << 3), ([0, 58 | IMM], [0, 2], xi >> 2),
                            ([0, 56 | IMM], [0, 7], xi - 7), ([0, 36 | IMM], [0, 7], 7 - xi)]:
        call(lib, ops, args, [xi.cuda()], oi, 3, 70001)
        assert torch.equal(oi.cpu(), want), ops
        assert torch.equal(E.run_program(ops, args, [xi], 3), want), ops
    call(lib, [0, 11 | IMM], [0, 0], [xd], out, 0, 16, expect=1)             # immediate on a unary opcode


def test_program_rejects_malformed_programs(lib):
    x = torch.zeros(16, device="cuda")
    out = torch.zeros(16, device="cuda")
    call(lib, [0, 2], [0, 0], [x], out, 0, 16, expect=1)                     # ADD with one operand
    call(lib, [0, 0], [0, 0], [x], out, 0, 16, expect=1)                     # two values left
    call(lib, [0], [1], [x], out, 0, 16, expect=1)                           # LOAD of a missing input
    call(lib, [0, 99], [0, 0], [x], out, 0, 16, expect=1)                    # unknown opcode
    call(lib, [0] * 9 + [2] * 8, [0] * 17, [x], out, 0, 16, expect=6)        # stack deeper than 8
    call(lib, [0] * 8 + [2] * 7, [0] * 15, [x], out, 0, 16)                  # exactly 8 is fine
    assert torch.equal(out.cpu(), torch.zeros(16))
    call(lib, [0], [0], [x], out, 0, 0)                                      # n == 0: nothing to do
    half = torch.zeros(17, dtype=torch.float16, device="cuda")
    bad = ctypes.c_void_p(half.data_ptr() + 1)
    ops_a, args_a = (ctypes.c_int32 * 1)(0), (ctypes.c_int32 * 1)(0)
    ins, types = (ctypes.c_void_p * 1)(bad), (ctypes.c_int32 * 1)(1)
    assert lib.asc_cuda_eltwise_program(ops_a, args_a, 1, ins, types, 1, ctypes.c_void_p(out.data_ptr()), 0, 8, None) == 2


def test_golden_fixture(golden_dir):
    import os
    d = np.load(os.path.join(golden_dir, "elementwise_reduce.npz"))
    x = torch.from_numpy(d["gelu_x"])
    out = torch.empty_like(x)
    for approximate, key in ((False, "gelu_erf"), (True, "gelu_tanh")):
        K.gelu[16](x, out, 8, 1024, 1024, approximate)
        torch.testing.assert_close(out, torch.from_numpy(d[key]), rtol=1e-3, atol=1e-5)
    xl = torch.from_numpy(d["leaky_x"]).view(torch.bfloat16)
    ol = torch.empty_like(xl)
    K.leaky_relu[16](xl, torch.tensor(float(d["leaky_alpha"]), dtype=torch.bfloat16), ol, 8192, 128, 4)
    assert torch.equal(ol, torch.from_numpy(d["leaky_out"]).view(torch.bfloat16))


# ------------------------------------------------------------------------------- random programs
def _random_program(rng, n_inputs, round_op):
    """A random valid postfix program over fp32 stack words: arithmetic, comparisons, selects, immediates and
    swapped forms, every result rounded through `round_op` when the tensors are 16-bit."""
    binary = [2, 3, 4, 6, 7, 54]
    unary = [8, 9, 10, 24, 25]
    compare = [26, 27, 28, 29, 30, 31]
    code = []

    def rounded():
        if round_op:
            code.append((round_op, 0))

    def const():
        return fbits(float(np.float32(rng.uniform(-2, 2)))) if not round_op else \
            fbits(float(torch.tensor(rng.uniform(-2, 2)).to(torch.float16 if round_op == 33 else torch.bfloat16)))

    def gen(depth):
        kind = rng.integers(0, 6) if depth > 0 else 0
        if kind == 0:
            code.append((0, int(rng.integers(0, n_inputs))))
        elif kind == 1:
            gen(depth - 1)
            code.append((int(rng.choice(unary)), 0))
            rounded()
        elif kind == 2:
            gen(depth - 1)
            gen(depth - 1)
            code.append((int(rng.choice(binary)), 0))
            rounded()
        elif kind == 3:
            gen(depth - 1)
            code.append((int(rng.choice(binary)) | IMM, const()))
            rounded()
        elif kind == 4:
            gen(depth - 1)
            gen(depth - 1)
            code.append((int(rng.choice(compare)), 0))
            gen(depth - 1)
            gen(depth - 1)
            code.append((32, 0))
        else:
            gen(depth - 1)
            code.append((int(rng.choice(compare)) | IMM, const()))
            gen(depth - 1)
            code.append((1, const()))
            code.append((32, 0))
    gen(3)
    return [c[0] for c in code], [c[1] for c in code]


@pytest.mark.parametrize("seed", range(24))
def test_random_programs_bit_exact_in_every_executor_width(lib, seed):
    rng = np.random.default_rng(seed)
    dtype, out_type, round_op = [(torch.float32, 0, None), (torch.float16, 1, 33), (torch.bfloat16, 2, 34)][seed % 3]
    n_inputs = int(rng.integers(1, 4))
    ops, args = _random_program(rng, n_inputs, round_op)
    depth = peak = 0
    for op in ops:
        code, imm = op & 0xff, bool(op & IMM)
        depth += 1 if code <= 1 else -2 if code == 32 else 0 if imm or code in (8, 9, 10, 24, 25, 33, 34) else -1
        peak = max(peak, depth)
    if len(ops) > 48 or peak > 8:
        pytest.skip("program beyond the documented limits")
    n = int(rng.choice([1, 37, 4096, 70001, (1 << 20) + 5]))
    gen = torch.Generator().manual_seed(seed)
    inputs = [(torch.rand(n, generator=gen) * 8 - 4).to(dtype) for _ in range(n_inputs)]
    dev = [t.cuda() for t in inputs]
    want = E.run_program(ops, args, inputs, out_type)
    try:
        for lanes in (4, 8, 16):
            lib.asc_cuda_eltwise_set_lanes(lanes)
            out = torch.zeros(n + 1, dtype=dtype, device="cuda")
            call(lib, ops, args, dev, out, out_type, n)
            got = out.cpu()
            assert torch.equal(got[:n], want), f"lanes {lanes}: {ops}"
            assert got[n] == 0
    finally:
        lib.asc_cuda_eltwise_set_lanes(0)


# ------------------------------------------------------------------------------- kernels specialised at first use
def _interpreted(lib, fn):
    assert lib.asc_cuda_eltwise_set_lanes(0x100) == 0       # every program through the interpreter
    try:
        return fn()
    finally:
        assert lib.asc_cuda_eltwise_set_lanes(0) == 0


@pytest.mark.parametrize("name, dtype, out_type, ops, args", [
    ("mish", torch.float32, 0, [0, 0, 11, 2 | IMM, 13, 22, 4], [0, 0, 0, fbits(1.0), 0, 0, 0]),
    ("two_inputs", torch.float32, 0, [0, 0, 3, 9, 0, 0, 4, 2, 15, 0, 5], [0, 1, 0, 0, 0, 1, 0, 0, 0, 1, 0]),
    ("half_chain", torch.float16, 1, [0, 0, 4, 33, 0, 2, 33, 10, 33], [0, 1, 0, 0, 0, 0, 0, 0, 0]),
    ("bf16_where", torch.bfloat16, 2, [0, 29 | IMM, 0, 0, 4 | IMM, 34, 0, 2, 34, 32], [0, fbits(0.5), 0, 1, fbits(3.0), 0, 0, 0, 0, 0]),
], ids=lambda v: v if isinstance(v, str) else "")
@pytest.mark.parametrize("n", [4099, (1 << 22) + 5])
def test_programs_built_at_first_use_equal_the_interpreter(lib, name, dtype, out_type, ops, args, n):
    """An expression without a built-in specialised kernel gets one built with nvcc at first use; its results are
    bit-identical to the interpreter's (and the cached library is found again by the second size)."""
    from pyasc_b200 import jit
    if jit.compiler() is None:
        pytest.skip("no nvcc on this machine")
    gen = torch.Generator().manual_seed(n)
    x = (torch.rand(n, generator=gen) * 4 + 0.25).to(dtype).cuda()
    y = (torch.rand(n, generator=gen) * 4 - 2).to(dtype).cuda()
    ins = [x, y][:max(args[k] for k in range(len(ops)) if ops[k] & 0xff == 0) + 1]
    plain = torch.zeros(n, dtype=dtype, device="cuda")
    _interpreted(lib, lambda: call(lib, ops, args, ins, plain, out_type, n))
    assert jit.request(0, jit.program_words(ops, args), wait=True), jit.failures()
    before = capi.launch_count()
    fast = torch.zeros(n, dtype=dtype, device="cuda")
    call(lib, ops, args, ins, fast, out_type, n)
    assert capi.launch_count() == before + 1
    assert torch.equal(fast.view(torch.int16 if dtype != torch.float32 else torch.int32),
                       plain.view(torch.int16 if dtype != torch.float32 else torch.int32))
    want = E.run_program(ops, args, [t.cpu() for t in ins], out_type)
    torch.testing.assert_close(fast.cpu().float(), want.float(), rtol=2e-3, atol=1e-5, equal_nan=True)


def test_in_place_updates_through_asc2():
    """An operand taken from the stored tensor at the stored window: `y = x + y` with scalar-sized tiles (the
    reference's docs/design/software-pipelining.md:55-66) and a 2-D tile scaled in place by a broadcast row."""
    @asc2.jit()
    def accumulate(x, y, size: int):
        x_gm = asc2.tensor(x, [size])
        y_gm = asc2.tensor(y, [size])
        for i in asc2.range(size, unroll_factor=2, parallel=True):
            x_val = asc2.load(x_gm, [1], offsets=[i])
            y_val = asc2.load(y_gm, [1], offsets=[i])
            asc2.store(x_val + y_val, y_gm, offsets=[i])

    gen = torch.Generator().manual_seed(31)
    x, y = torch.randn(64, generator=gen), torch.randn(64, generator=gen)
    want = x + y
    accumulate[1](x, y, 64)
    assert torch.equal(y, want)

    @asc2.jit
    def scale_rows(m_ptr: asc.GlobalAddress, w_ptr: asc.GlobalAddress, rows: int, cols: asc.ConstExpr[int],
                   rpt: asc.ConstExpr[int]):
        m_gm = asc2.tensor(m_ptr, [rows, cols])
        w = asc2.load(asc2.tensor(w_ptr, [1, cols]), [1, cols], offsets=[0, 0])
        for r in range(asc2.block_idx() * rpt, rows, asc2.block_num() * rpt):
            m = asc2.load(m_gm, [rpt, cols], offsets=[r, 0])
            asc2.store(m * w.broadcast_to(rpt, cols) + 1.0, m_gm, offsets=[r, 0])

    m, w = torch.randn(256, 512, generator=gen), torch.randn(1, 512, generator=gen)
    want = m * w + 1.0
    md = m.cuda()
    scale_rows[8](md, w.cuda(), 256, 512, 8)
    torch.cuda.synchronize()
    assert torch.equal(md.cpu(), want)
