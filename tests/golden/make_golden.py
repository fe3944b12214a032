"""Generates the committed golden fixtures under tests/golden/ with the reference's own CPU
expressions (torch / NumPy, see oracle/golden.py for the file:line of each).

Run from the repository root:  python tests/golden/make_golden.py   (--only-elementwise: just elementwise_reduce.npz;
--only-normalisation: just normalisation.npz)
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


def elementwise_and_reduce() -> None:
    """GELU (both forms), bf16 leaky ReLU and the tile reductions, with the torch expressions of
    python/test/asc2/kernels/test_gelu.py:46-50, test_leaky_relu.py:41-46 and
    python/test/asc2/operations/test_reduce_ops.py:62-83."""
    import math
    g = G.gen()
    x = torch.rand((8, 1024), generator=g)
    erf = 0.5 * x * (1 + torch.erf(x / math.sqrt(2)))
    tanh = 0.5 * x * (1 + torch.tanh(math.sqrt(2 / math.pi) * (x + 0.044715 * torch.pow(x, 3))))
    xl = (torch.rand(8192, generator=g) * 10.0 - 5.0).to(torch.bfloat16)
    alpha = torch.tensor(0.1, dtype=torch.bfloat16)
    leaky = torch.where(xl >= 0, xl, xl * alpha)
    xr = torch.randn([64, 32], generator=g) * 2.0
    np.savez_compressed(os.path.join(HERE, "elementwise_reduce.npz"), gelu_x=x.numpy(), gelu_erf=erf.numpy(),
                        gelu_tanh=tanh.numpy(), leaky_x=xl.view(torch.int16).numpy(), leaky_alpha=np.float32(alpha.item()),
                        leaky_out=leaky.view(torch.int16).numpy(), reduce_x=xr.numpy(), sum0=xr.sum(0).numpy(),
                        sum1=xr.sum(1).numpy(), max0=xr.amax(0).numpy(), min1=xr.amin(1).numpy(),
                        prod0=xr.prod(0).numpy())


def normalisation() -> None:
    """RMS norm (the formula of the Ascend C RmsNorm routine asc2.rms_norm lowers to,
    python/asc/language/tile/unary_ops.py:225-237) and a layer norm, computed in float64 and rounded once."""
    g = torch.Generator().manual_seed(G.SEED + 1)
    x = torch.randn((8, 512), generator=g) * 3 + 0.5
    gamma = torch.rand(512, generator=g) + 0.5
    beta = torch.randn(512, generator=g)
    xd, gd, bd = x.double(), gamma.double(), beta.double()
    rms = xd / torch.sqrt(xd.pow(2).mean(1, keepdim=True) + 1e-5) * gd
    ln = (xd - xd.mean(1, keepdim=True)) / torch.sqrt(xd.var(1, unbiased=False, keepdim=True) + 1e-5) * gd + bd
    np.savez_compressed(os.path.join(HERE, "normalisation.npz"), x=x.numpy(), gamma=gamma.numpy(), beta=beta.numpy(),
                        eps=np.float32(1e-5), rms_norm=rms.float().numpy(), layer_norm=ln.float().numpy())


def main() -> None:
    torch.set_num_threads(1)  # fixed summation order for the fp32 reductions
    if "--only-elementwise" in sys.argv:
        elementwise_and_reduce()
        return
    if "--only-normalisation" in sys.argv:
        normalisation()
        return
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
    elementwise_and_reduce()
    normalisation()
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    main()
