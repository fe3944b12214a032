"""Vector add, the README kernel of the reference (README.md:29-41; python/test/asc2/kernels/test_vadd.py:16-28)."""
import asc
import asc2


@asc2.jit
def vadd_kernel(x_ptr: asc.GlobalAddress, y_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, size: int,
                tile_size: asc.ConstExpr[int], tile_per_block: asc.ConstExpr[int]):
    x_gm = asc2.tensor(x_ptr, [size])
    y_gm = asc2.tensor(y_ptr, [size])
    out_gm = asc2.tensor(out_ptr, [size])
    base_offset = asc2.block_idx() * tile_size * tile_per_block
    for i in range(tile_per_block):
        tile_offset = base_offset + i * tile_size
        x = asc2.load(x_gm, [tile_size], offsets=[tile_offset])
        y = asc2.load(y_gm, [tile_size], offsets=[tile_offset])
        out = x + y
        asc2.store(out, out_gm, offsets=[tile_offset])


def vadd_launch(x, y, out, core_num: int = 16, tile_size: int = 128, stream=None):
    """out = x + y for 1-D float32 tensors/arrays of equal length (written in place)."""
    size = int(x.numel()) if hasattr(x, "numel") else int(x.size)
    num_tiles = asc.ceildiv(size, tile_size)
    launch = vadd_kernel[core_num] if stream is None else vadd_kernel[core_num, stream]
    launch(x, y, out, size, tile_size, asc.ceildiv(num_tiles, core_num))
    return out
