"""Dense GEMM, fp16/bf16 operands, fp32 accumulation, 16-bit result.

M/N-blocked like the reference's python/test/asc2/kernels/test_matmul_mnblock.py:17-36, with an inner
K loop of ``matmul_acc`` like test_matmul_tiled.py:17-31 and the down-cast epilogue of
test_matmul_fixpipe.py:17-27, so that it can express K = 8192 (the reference scripts keep the whole K
extent in one tile, which their 64 KB limit caps at K = 256 for 128-row tiles)."""
import asc
import asc2


@asc2.jit
def matmul_fp16_kernel(a_ptr: asc.GlobalAddress, b_ptr: asc.GlobalAddress, c_ptr: asc.GlobalAddress,
                       a_shape: asc.ConstExpr, b_shape: asc.ConstExpr, c_shape: asc.ConstExpr,
                       m_tile: asc.ConstExpr[int], n_tile: asc.ConstExpr[int], k_tile: asc.ConstExpr[int],
                       out_dtype: asc.ConstExpr, relu: asc.ConstExpr[bool]):
    a_gm = asc2.tensor(a_ptr, a_shape)
    b_gm = asc2.tensor(b_ptr, b_shape)
    c_gm = asc2.tensor(c_ptr, c_shape)
    m_tiles = asc.ceildiv(c_shape[0], m_tile)
    n_tiles = asc.ceildiv(c_shape[1], n_tile)
    k_tiles = asc.ceildiv(a_shape[1], k_tile)
    for t in range(asc2.block_idx(), m_tiles * n_tiles, asc2.block_num()):
        m_off = (t // n_tiles) * m_tile
        n_off = (t % n_tiles) * n_tile
        acc = asc2.zeros_acc([m_tile, n_tile], dtype=asc.float32)
        for k in range(k_tiles, unroll_factor=2, parallel=True):
            a = asc2.load(a_gm, [m_tile, k_tile], offsets=[m_off, k * k_tile], location=asc2.TileLocation.L0A)
            b = asc2.load(b_gm, [k_tile, n_tile], offsets=[k * k_tile, n_off], location=asc2.TileLocation.L0B)
            asc2.matmul_acc(a, b, acc)
        if relu:
            acc = asc2.relu(acc)
        asc2.store(acc.to(out_dtype), c_gm, offsets=[m_off, n_off])


_ASC_DTYPE = {"float16": asc.float16, "bfloat16": asc.bfloat16, "float32": asc.float32}


def matmul_fp16_launch(a, b, c, core_num: int = 148, m_tile: int = 128, n_tile: int = 256, k_tile: int = 64,
                       relu: bool = False, stream=None):
    """c = a @ b (optionally ReLU'd), c's dtype selects the epilogue cast."""
    out_dtype = _ASC_DTYPE[str(c.dtype).replace("torch.", "")]
    launch = matmul_fp16_kernel[core_num] if stream is None else matmul_fp16_kernel[core_num, stream]
    launch(a, b, c, tuple(a.shape), tuple(b.shape), tuple(c.shape), m_tile, n_tile, k_tile, out_dtype, relu)
    return c
