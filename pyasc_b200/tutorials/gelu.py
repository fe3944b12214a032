"""GELU over the rows of a matrix, both forms of the reference's kernel test
(python/test/asc2/kernels/test_gelu.py:16-34): the exact erf form and the exp-based rewrite of the
tanh approximation.  The whole expression becomes one pass over memory on the CUDA platform."""
import asc
import asc2


@asc2.jit
def gelu_kernel(x_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, num_rows: asc.ConstExpr,
                num_columns: asc.ConstExpr, tile_size: asc.ConstExpr, approximate: asc.ConstExpr):
    x_gm = asc2.tensor(x_ptr, [num_rows, num_columns])
    out_gm = asc2.tensor(out_ptr, [num_rows, num_columns])
    for i in range(asc2.block_idx(), num_rows, asc2.block_num(), parallel=True):
        row = asc2.load(x_gm, [1, tile_size], offsets=[i, 0])
        if approximate:
            pi = 3.141592653589793238462643383279502884
            k1 = 2 * asc2.sqrt(2 / pi)
            k2 = 2 * asc2.sqrt(2 / pi) * 0.044715
            param = row * (row * row * k2 + k1)
            out = row - row / (asc2.exp(param) + 1)
        else:
            k = asc2.sqrt(0.5)
            out = row * (asc2.erf(row * k) + 1) * 0.5
        asc2.store(out, out_gm, offsets=[i, 0])


def gelu_launch(x, out, approximate: bool = False, core_num: int = 16, stream=None):
    """out = gelu(x) for a 2-D float32 tensor whose rows are whole tiles (written in place)."""
    num_rows, num_columns = x.shape
    launch = gelu_kernel[core_num] if stream is None else gelu_kernel[core_num, stream]
    launch(x, out, num_rows, num_columns, num_columns, approximate)
    return out
