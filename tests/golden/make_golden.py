"""Generates the committed golden fixtures under tests/golden/ with the reference's own CPU
expressions (torch / NumPy, see oracle/golden.py for the file:line of each).

Run from the repository root:  python tests/golden/make_golden.py
The reference package itself cannot be imported (its compiled MLIR extension and the CANN toolkit are
absent), so the fixtures come from the torch/NumPy calls its tests make, on the seeds its tests use.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import golden as G  # noqa: E402


def main() -> None:
    torch.set_num_threads(1)  # fixed summation order for the fp32 reductions
    # vector add, NumPy form of python/test/asc2/kernels/test_vadd.py:41-48
    rng = np.random.default_rng(seed=2026)
    x = rng.random(8192, dtype=np.float32) * 10
    y = rng.random(8192, dtype=np.float32) * 10
    z = rng.random(8192, dtype=np.float32) * 10
    np.savez_compressed(os.path.join(HERE, "vadd_8192.npz"), x=x, y=y, z=z, out=x + y, muladd=x * y + z)
    # torch form of README.md:43-53
    tx, ty = G.vadd_inputs(8192)
    np.savez_compressed(os.path.join(HERE, "vadd_torch_8192.npz"), x=tx.numpy(), y=ty.numpy(),
                        out=G.vadd(tx, ty).numpy())
    # softmax: torch.rand like the reference test, and the workload's normal(0,1)
    g = G.gen()
    xs = torch.rand((16, 1024), generator=g)
    xn = G.softmax_input(8, 4096)
    np.savez_compressed(os.path.join(HERE, "softmax.npz"), x_rand=xs.numpy(), out_rand=G.softmax(xs).numpy(),
                        x_randn=xn.numpy(), out_randn=G.softmax(xn).numpy())
    # fp16 matmul 64 x 128 x 256 (python/test/asc2/kernels/test_matmul_tiled.py:44-49) + fixpipe form
    g = G.gen()
    a = torch.rand((64, 128), generator=g).half()
    b = torch.rand((128, 256), generator=g).half()
    a2 = ((torch.rand((64, 128), generator=g) - .5) * 10).half()
    b2 = ((torch.rand((128, 256), generator=g) - .5) * 10).half()
    np.savez_compressed(os.path.join(HERE, "gemm_f16.npz"), a=a.numpy(), b=b.numpy(), c_f32=G.gemm_f32acc(a, b).numpy(),
                        a2=a2.numpy(), b2=b2.numpy(), c2_relu_f16=G.gemm_f16(a2, b2, relu=True).numpy())
    # int8 matmul + dequant
    a8, b8, sa, sb = G.gemm_i8_inputs(96, 144, 160)
    acc = G.gemm_i8_int32_form(a8, b8)
    np.savez_compressed(os.path.join(HERE, "gemm_i8.npz"), a=a8.numpy(), b=b8.numpy(), a_scale=sa.numpy(),
                        b_scale=sb.numpy(), acc=acc.numpy(), deq=G.dequant(acc, sa, sb).numpy())
    # attention 1 x 2 x 256 x 128
    q, k, v = G.attention_inputs(1, 2, 256)
    np.savez_compressed(os.path.join(HERE, "attention.npz"), q=q.numpy(), k=k.numpy(), v=v.numpy(),
                        o=G.attention(q, k, v, False).numpy(), o_causal=G.attention(q, k, v, True).numpy())
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    main()
