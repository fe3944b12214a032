"""Row softmax in both forms the reference tests (python/test/asc2/kernels/test_softmax.py:16-27 and
test_softmax_fused.py:16-24)."""
import asc
import asc2


@asc2.jit(vf_fusion=True)
def softmax_kernel(x_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, num_rows: int, num_cols: int,
                   tile_size: asc.ConstExpr[int]):
    x_gm = asc2.tensor(x_ptr, [num_rows, num_cols])
    out_gm = asc2.tensor(out_ptr, [num_rows, num_cols])
    for i in range(asc2.block_idx(), num_rows, asc2.block_num(), parallel=True):
        row = asc2.load(x_gm, [1, tile_size], offsets=[i, 0])
        row_minus_max = row - asc2.reduce_max(row)
        numerator = asc2.exp(row_minus_max)
        denominator = asc2.reduce_sum(numerator)
        out = numerator / denominator
        asc2.store(out, out_gm, offsets=[i, 0])


def softmax_launch(x, out, core_num: int = 16, stream=None):
    num_rows, num_cols = x.shape
    launch = softmax_kernel[core_num] if stream is None else softmax_kernel[core_num, stream]
    launch(x, out, num_rows, num_cols, tile_size=num_cols)
    return out


@asc2.jit
def softmax_fused_kernel(x_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, num_rows: int,
                         num_cols: asc.ConstExpr[int], block_size: asc.ConstExpr[int]):
    x_gm = asc2.tensor(x_ptr, [num_rows, num_cols])
    out_gm = asc2.tensor(out_ptr, [num_rows, num_cols])
    start_rows = asc2.block_idx() * block_size
    rows = asc2.load(x_gm, [block_size, num_cols], offsets=[start_rows, 0])
    out = asc2.softmax(rows)
    asc2.store(out, out_gm, offsets=[start_rows, 0])


def softmax_fused_launch(x, out, core_num: int = 16, stream=None):
    num_rows, num_cols = x.shape
    block_size = (num_rows + core_num - 1) // core_num
    launch = softmax_fused_kernel[core_num] if stream is None else softmax_fused_kernel[core_num, stream]
    launch(x, out, num_rows, num_cols, block_size)
    return out
