"""Leaky ReLU with a run-time slope (python/test/asc2/kernels/test_leaky_relu.py:16-27): a compare, a
scalar multiply and a select over 1-D tiles, fused into one pass over memory on the CUDA platform."""
import asc
import asc2


@asc2.jit
def leaky_relu_kernel(x_ptr: asc.GlobalAddress, alpha: float, out_ptr: asc.GlobalAddress, size: int,
                      tile_size: asc.ConstExpr[int], tile_per_block: asc.ConstExpr[int]):
    x_gm = asc2.tensor(x_ptr, [size])
    out_gm = asc2.tensor(out_ptr, [size])
    base_offset = asc2.block_idx() * tile_size * tile_per_block
    for i in range(tile_per_block, unroll_factor=2, parallel=True):
        tile_offset = base_offset + i * tile_size
        x = asc2.load(x_gm, [tile_size], offsets=[tile_offset])
        out = asc2.where(x >= 0, x, x * alpha)
        asc2.store(out, out_gm, offsets=[tile_offset])


def leaky_relu_launch(x, alpha, out, core_num: int = 16, tile_size: int = 128, stream=None):
    """out = where(x >= 0, x, x * alpha) for a 1-D float32 / float16 / bfloat16 tensor; ``alpha`` is a
    Python float or a zero-dim tensor of x's dtype."""
    size = int(x.numel())
    num_tiles = asc.ceildiv(size, tile_size)
    launch = leaky_relu_kernel[core_num] if stream is None else leaky_relu_kernel[core_num, stream]
    launch(x, alpha, out, size, tile_size, asc.ceildiv(num_tiles, core_num))
    return out
