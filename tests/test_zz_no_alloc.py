"""The GEMM entry point that allocates nothing, against the ordinary one.

``asc_cuda_gemm_f16_static_workspace`` serves callers that may not allocate device memory once they are running
(a latency-critical thread that must not block in the allocator, a process whose memory budget is spent at
start-up).  It runs the split-K GEMM with a workspace that is a fixed array inside the library instead of a
per-call allocation.  Every call on a device shares that array and it keeps what the last call left there, so the
test calls it twice in a row, with different operands, and checks both results against ``asc_cuda_gemm_f16``
at the tolerance the other GEMM tests use (atol = rtol = 2e-3 for fp16 results, the K-scaled fp32 bound for fp32).

The file name sorts last on purpose: in a run that stops at the first failure every other test has run by then.
"""
import ctypes

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
    return ctypes.c_void_p(t.data_ptr())


def gemm(lib, name, a, b, out_dtype, flags=0, expect=0):
    m, k = a.shape
    n = b.shape[1]
    c = torch.full((m, n), -7.0, dtype=out_dtype, device="cuda")
    out_code = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}[out_dtype]
    rc = getattr(lib, name)(P(a), P(b), P(c), m, n, k, k, n, n, 0, out_code, flags, None)
    assert rc == expect, f"{name} returned {rc}: {capi.status_string(rc)} {capi.last_cuda_error()}"
    if rc == 0:
        capi.check_device_status(None)
    return c


@pytest.mark.parametrize("m, n, k", [(256, 256, 8192), (100, 520, 4104), (1024, 2048, 512)])
def test_two_calls_in_a_row_match_the_allocating_entry_point(lib, m, n, k):
    for seed, out_dtype, flags in ((k, torch.float16, 1), (k + 1, torch.float32, 0)):
        a, b = G.gemm_f16_inputs(m, n, k, seed=seed)
        ad, bd = a.cuda(), b.cuda()
        got = gemm(lib, "asc_cuda_gemm_f16_static_workspace", ad, bd, out_dtype, flags)
        assert lib.asc_cuda_gemm_set_mode(0x10) == 0            # the ordinary entry point on the tensor core too
        try:
            want = gemm(lib, "asc_cuda_gemm_f16", ad, bd, out_dtype, flags)
        finally:
            assert lib.asc_cuda_gemm_set_mode(0) == 0
        if out_dtype == torch.float16:
            G.assert_half_close(got, want.cpu())
            G.assert_half_close(got, G.gemm_f16(a, b, relu=True))
        else:
            torch.testing.assert_close(got, want, atol=2e-5 * (k ** 0.5) / 8 + 1e-5, rtol=1e-4)


def test_output_beyond_the_fixed_workspace_is_refused(lib):
    a, b = G.gemm_f16_inputs(1024, 2304, 64)                    # 8 x 9 = 72 tiles of 128 x 256 > 64
    c = gemm(lib, "asc_cuda_gemm_f16_static_workspace", a.cuda(), b.cuda(), torch.float16, expect=6)
    assert capi.status_string(6) == "size beyond the documented maximum"
    assert bool((c == -7.0).all())                              # nothing was launched
