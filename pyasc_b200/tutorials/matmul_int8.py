"""Quantised GEMM: int8 x int8 -> int32, and the per-channel dequantised fp16 form
``out = acc * a_scale[row] * b_scale[col]``.

The reference's asc2 ``matmul`` takes floating-point tiles only (python/asc/language/tile/utils.py:134);
int8 operands are an extension of the CUDA platform.  The nearest reference definition is the golden of
python/test/generalization/adv/test_matmul_quant.py:124-138 (``a.int32 @ b.int32`` then a scale)."""
import asc
import asc2


@asc2.jit
def matmul_int8_kernel(a_ptr: asc.GlobalAddress, b_ptr: asc.GlobalAddress, c_ptr: asc.GlobalAddress,
                       a_shape: asc.ConstExpr, b_shape: asc.ConstExpr, c_shape: asc.ConstExpr,
                       m_tile: asc.ConstExpr[int], n_tile: asc.ConstExpr[int], k_tile: asc.ConstExpr[int]):
    a_gm = asc2.tensor(a_ptr, a_shape)
    b_gm = asc2.tensor(b_ptr, b_shape)
    c_gm = asc2.tensor(c_ptr, c_shape)
    n_tiles = asc.ceildiv(c_shape[1], n_tile)
    total = asc.ceildiv(c_shape[0], m_tile) * n_tiles
    k_tiles = asc.ceildiv(a_shape[1], k_tile)
    for t in range(asc2.block_idx(), total, asc2.block_num()):
        m_off = (t // n_tiles) * m_tile
        n_off = (t % n_tiles) * n_tile
        acc = asc2.zeros_acc([m_tile, n_tile], dtype=asc.int32)
        for k in range(k_tiles, unroll_factor=2, parallel=True):
            a = asc2.load(a_gm, [m_tile, k_tile], offsets=[m_off, k * k_tile], location=asc2.TileLocation.L0A)
            b = asc2.load(b_gm, [k_tile, n_tile], offsets=[k * k_tile, n_off], location=asc2.TileLocation.L0B)
            asc2.matmul_acc(a, b, acc)
        asc2.store(acc, c_gm, offsets=[m_off, n_off])


def matmul_int8_launch(a, b, c, core_num: int = 148, m_tile: int = 128, n_tile: int = 256, k_tile: int = 128,
                       stream=None):
    launch = matmul_int8_kernel[core_num] if stream is None else matmul_int8_kernel[core_num, stream]
    launch(a, b, c, tuple(a.shape), tuple(b.shape), tuple(c.shape), m_tile, n_tile, k_tile)
    return c


@asc2.jit
def matmul_int8_dequant_kernel(a_ptr: asc.GlobalAddress, b_ptr: asc.GlobalAddress, a_scale_ptr: asc.GlobalAddress,
                               b_scale_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, a_shape: asc.ConstExpr,
                               b_shape: asc.ConstExpr, m_tile: asc.ConstExpr[int], n_tile: asc.ConstExpr[int],
                               k_tile: asc.ConstExpr[int]):
    m, n = a_shape[0], b_shape[1]
    a_gm = asc2.tensor(a_ptr, a_shape)
    b_gm = asc2.tensor(b_ptr, b_shape)
    a_scale_gm = asc2.tensor(a_scale_ptr, [m])
    b_scale_gm = asc2.tensor(b_scale_ptr, [n])
    out_gm = asc2.tensor(out_ptr, [m, n])
    n_tiles = asc.ceildiv(n, n_tile)
    total = asc.ceildiv(m, m_tile) * n_tiles
    k_tiles = asc.ceildiv(a_shape[1], k_tile)
    for t in range(asc2.block_idx(), total, asc2.block_num()):
        m_off = (t // n_tiles) * m_tile
        n_off = (t % n_tiles) * n_tile
        acc = asc2.zeros_acc([m_tile, n_tile], dtype=asc.int32)
        for k in range(k_tiles, unroll_factor=2, parallel=True):
            a = asc2.load(a_gm, [m_tile, k_tile], offsets=[m_off, k * k_tile], location=asc2.TileLocation.L0A)
            b = asc2.load(b_gm, [k_tile, n_tile], offsets=[k * k_tile, n_off], location=asc2.TileLocation.L0B)
            asc2.matmul_acc(a, b, acc)
        sa = asc2.load(a_scale_gm, [m_tile], offsets=[m_off]).reshape(m_tile, 1).broadcast_to(m_tile, n_tile)
        sb = asc2.load(b_scale_gm, [n_tile], offsets=[n_off]).reshape(1, n_tile).broadcast_to(m_tile, n_tile)
        out = acc.to(asc.float32) * sa * sb
        asc2.store(out.to(asc.float16), out_gm, offsets=[m_off, n_off])


def matmul_int8_dequant_launch(a, b, a_scale, b_scale, out, core_num: int = 148, m_tile: int = 128, n_tile: int = 256,
                               k_tile: int = 128, stream=None):
    launch = matmul_int8_dequant_kernel[core_num] if stream is None else matmul_int8_dequant_kernel[core_num, stream]
    launch(a, b, a_scale, b_scale, out, tuple(a.shape), tuple(b.shape), m_tile, n_tile, k_tile)
    return out
