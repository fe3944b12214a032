"""asc2 kernels in the forms the reference's kernel tests exercise
(python/test/asc2/kernels/test_{vadd,vmuladd,softmax,softmax_fused,matmul_tiled,matmul_mnblock,
matmul_fixpipe,matmul_l0c_to_l1}.py), used by the CPU matcher tests and the GPU parity tests.
Written against the public asc / asc2 names only, exactly as a user script would be."""
import asc
import asc2

L0A, L0B, L1 = asc2.TileLocation.L0A, asc2.TileLocation.L0B, asc2.TileLocation.L1


@asc2.jit(always_compile=True)
def vadd(x_ptr: asc.GlobalAddress, y_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, size: int,
         tile_size: asc.ConstExpr[int], tile_per_block: asc.ConstExpr[int]):
    x_gm, y_gm, out_gm = (asc2.tensor(p, [size]) for p in (x_ptr, y_ptr, out_ptr))
    first = asc2.block_idx() * tile_size * tile_per_block
    for i in range(tile_per_block):
        off = first + i * tile_size
        asc2.store(asc2.load(x_gm, [tile_size], offsets=[off]) + asc2.load(y_gm, [tile_size], offsets=[off]),
                   out_gm, offsets=[off])


@asc2.jit(always_compile=True, vf_fusion=True)
def vmuladd(x_ptr: asc.GlobalAddress, y_ptr: asc.GlobalAddress, z_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress,
            size: int, tile_size: asc.ConstExpr[int], tile_per_block: asc.ConstExpr[int],
            buffer_factor: asc.ConstExpr[int]):
    x_gm, y_gm, z_gm, out_gm = (asc2.tensor(p, [size]) for p in (x_ptr, y_ptr, z_ptr, out_ptr))
    first = asc2.block_idx() * tile_size * tile_per_block
    for i in range(tile_per_block, unroll_factor=buffer_factor, parallel=True):
        off = first + i * tile_size
        x = asc2.load(x_gm, [tile_size], offsets=[off])
        y = asc2.load(y_gm, [tile_size], offsets=[off])
        z = asc2.load(z_gm, [tile_size], offsets=[off])
        asc2.store(x * y + z, out_gm, offsets=[off])


@asc2.jit(always_compile=True, vf_fusion=True)
def softmax_rows(x_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, num_rows: int, num_cols: int,
                 tile_size: asc.ConstExpr[int]):
    x_gm = asc2.tensor(x_ptr, [num_rows, num_cols])
    out_gm = asc2.tensor(out_ptr, [num_rows, num_cols])
    for i in range(asc2.block_idx(), num_rows, asc2.block_num(), parallel=True):
        row = asc2.load(x_gm, [1, tile_size], offsets=[i, 0])
        shifted = row - asc2.reduce_max(row)
        e = asc2.exp(shifted)
        asc2.store(e / asc2.reduce_sum(e), out_gm, offsets=[i, 0])


@asc2.jit(always_compile=True)
def softmax_blocks(x_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, num_rows: int, num_cols: asc.ConstExpr[int],
                   block_size: asc.ConstExpr[int]):
    x_gm = asc2.tensor(x_ptr, [num_rows, num_cols])
    out_gm = asc2.tensor(out_ptr, [num_rows, num_cols])
    r0 = asc2.block_idx() * block_size
    asc2.store(asc2.softmax(asc2.load(x_gm, [block_size, num_cols], offsets=[r0, 0])), out_gm, offsets=[r0, 0])


@asc2.jit(always_compile=True)
def matmul_k_tiled(a_ptr: asc.GlobalAddress, b_ptr: asc.GlobalAddress, c_ptr: asc.GlobalAddress,
                   a_shape: asc.ConstExpr, b_shape: asc.ConstExpr, c_shape: asc.ConstExpr, k_tiles: asc.ConstExpr):
    a_gm, b_gm, c_gm = asc2.tensor(a_ptr, a_shape), asc2.tensor(b_ptr, b_shape), asc2.tensor(c_ptr, c_shape)
    acc = asc2.zeros_acc(c_shape, dtype=asc.float32)
    kt = a_shape[1] // k_tiles
    a_l1 = asc2.load(a_gm, a_shape, offsets=[0, 0], location=L1)
    b_l1 = asc2.load(b_gm, b_shape, offsets=[0, 0], location=L1)
    for i in range(k_tiles, unroll_factor=2, parallel=True):
        a_i = asc2.copy(a_l1, [a_shape[0], kt], offsets=[0, i * kt], location=L0A)
        b_i = asc2.copy(b_l1, [kt, b_shape[1]], offsets=[i * kt, 0], location=L0B)
        asc2.matmul_acc(a_i, b_i, acc)
    asc2.store(acc, c_gm, offsets=[0, 0])


@asc2.jit(always_compile=True)
def matmul_mn_blocked(a_ptr: asc.GlobalAddress, b_ptr: asc.GlobalAddress, c_ptr: asc.GlobalAddress,
                      a_shape: asc.ConstExpr, b_shape: asc.ConstExpr, c_shape: asc.ConstExpr,
                      m_tile: asc.ConstExpr[int], m_tiles_per_block: asc.ConstExpr[int], n_tile: asc.ConstExpr[int],
                      n_tiles_per_block: asc.ConstExpr[int]):
    a_gm, b_gm, c_gm = asc2.tensor(a_ptr, a_shape), asc2.tensor(b_ptr, b_shape), asc2.tensor(c_ptr, c_shape)
    block = asc2.block_idx()
    m_per_block = m_tile * m_tiles_per_block
    m_base = (m_per_block * block) % a_shape[0]
    n_base = ((m_per_block * block) // a_shape[0]) * (n_tile * n_tiles_per_block)
    for j in range(n_tiles_per_block):
        n_off = n_base + j * n_tile
        b_j = asc2.load(b_gm, [b_shape[0], n_tile], offsets=[0, n_off], location=L0B)
        for i in range(m_tiles_per_block):
            m_off = m_base + i * m_tile
            a_i = asc2.load(a_gm, [m_tile, a_shape[1]], offsets=[m_off, 0], location=L0A)
            asc2.store(a_i @ b_j, c_gm, offsets=[m_off, n_off])


@asc2.jit(always_compile=True)
def matmul_relu_cast(a_ptr: asc.GlobalAddress, b_ptr: asc.GlobalAddress, c_ptr: asc.GlobalAddress,
                     a_shape: asc.ConstExpr, b_shape: asc.ConstExpr, c_shape: asc.ConstExpr):
    a_gm, b_gm, c_gm = asc2.tensor(a_ptr, a_shape), asc2.tensor(b_ptr, b_shape), asc2.tensor(c_ptr, c_shape)
    a = asc2.load(a_gm, a_shape, offsets=[0, 0], location=L0A)
    b = asc2.load(b_gm, b_shape, offsets=[0, 0], location=L0B)
    c = asc2.relu(a @ b).to(asc.float16)
    asc2.store(c, c_gm, offsets=[0, 0])


@asc2.jit(always_compile=True)
def matmul_chained(a_ptr: asc.GlobalAddress, b_ptr: asc.GlobalAddress, c_ptr: asc.GlobalAddress,
                   a_shape: asc.ConstExpr, b_shape: asc.ConstExpr, c_shape: asc.ConstExpr, dtype: asc.ConstExpr):
    a_gm, b_gm, c_gm = asc2.tensor(a_ptr, a_shape), asc2.tensor(b_ptr, b_shape), asc2.tensor(c_ptr, c_shape)
    a = asc2.load(a_gm, a_shape, offsets=[0, 0], location=L0A)
    b = asc2.load(b_gm, b_shape, offsets=[0, 0], location=L0B)
    c = (a @ b).to(dtype)
    c_l1 = asc2.copy(c, c_shape, offsets=[0, 0], location=L1)
    c_l0a = asc2.copy(c_l1, c_shape, offsets=[0, 0], location=L0A)
    asc2.store(c_l0a @ b, c_gm, offsets=[0, 0])


@asc2.jit(always_compile=True)
def matmul_bias_act(a_ptr: asc.GlobalAddress, b_ptr: asc.GlobalAddress, bias_ptr: asc.GlobalAddress,
                    res_ptr: asc.GlobalAddress, c_ptr: asc.GlobalAddress, m: int, n: asc.ConstExpr[int],
                    k: asc.ConstExpr[int], m_tile: asc.ConstExpr[int], mode: asc.ConstExpr[int],
                    out_dtype: asc.ConstExpr):
    """A linear layer written the way a user of asc2 would: the product, a bias row, then an activation
    (0: none, 1: ReLU, 2: leaky ReLU, 3: tanh-form GELU plus a residual tile), optionally cast for the store."""
    a_gm, b_gm, c_gm = asc2.tensor(a_ptr, [m, k]), asc2.tensor(b_ptr, [k, n]), asc2.tensor(c_ptr, [m, n])
    res_gm = asc2.tensor(res_ptr, [m, n])
    bias = asc2.load(asc2.tensor(bias_ptr, [1, n]), [1, n], offsets=[0, 0])
    for i in range(asc2.block_idx() * m_tile, m, asc2.block_num() * m_tile):
        a = asc2.load(a_gm, [m_tile, k], offsets=[i, 0])
        b = asc2.load(b_gm, [k, n], offsets=[0, 0])
        t = asc2.matmul(a, b) + bias.broadcast_to(m_tile, n)
        if mode == 1:
            t = asc2.relu(t)
        elif mode == 2:
            t = asc2.where(t >= 0, t, t * 0.01)
        elif mode == 3:
            t = t - t / (asc2.exp(t * (t * t * 0.0713548162726 + 1.5957691216057308)) + 1)
            t = t + asc2.load(res_gm, [m_tile, n], offsets=[i, 0])
        if out_dtype != asc.float32:
            t = t.to(out_dtype)
        asc2.store(t, c_gm, offsets=[i, 0])


@asc2.jit(always_compile=True)
def matmul_batched(a_ptr: asc.GlobalAddress, b_ptr: asc.GlobalAddress, c_ptr: asc.GlobalAddress,
                   batch: asc.ConstExpr[int], m: asc.ConstExpr[int], n: asc.ConstExpr[int], k: asc.ConstExpr[int]):
    """A batch of independent products, one per loop iteration: A, B and C are stacks of matrices."""
    a_gm, b_gm, c_gm = asc2.tensor(a_ptr, [batch * m, k]), asc2.tensor(b_ptr, [batch * k, n]), asc2.tensor(c_ptr, [batch * m, n])
    for i in range(asc2.block_idx(), batch, asc2.block_num()):
        a = asc2.load(a_gm, [m, k], offsets=[i * m, 0])
        b = asc2.load(b_gm, [k, n], offsets=[i * k, 0])
        asc2.store(asc2.matmul(a, b), c_gm, offsets=[i * m, 0])


@asc2.jit(always_compile=True)
def matmul_k_tiled_bias_relu(a_ptr: asc.GlobalAddress, b_ptr: asc.GlobalAddress, bias_ptr: asc.GlobalAddress,
                             c_ptr: asc.GlobalAddress, m: asc.ConstExpr[int], n: asc.ConstExpr[int],
                             k: asc.ConstExpr[int], k_tile: asc.ConstExpr[int]):
    """An accumulation over a K loop, then a bias row and a ReLU on the accumulator."""
    a_gm, b_gm, c_gm = asc2.tensor(a_ptr, [m, k]), asc2.tensor(b_ptr, [k, n]), asc2.tensor(c_ptr, [m, n])
    bias = asc2.load(asc2.tensor(bias_ptr, [1, n]), [1, n], offsets=[0, 0])
    acc = asc2.zeros_acc([m, n], dtype=asc.float32)
    for kk in range(0, k, k_tile):
        a = asc2.load(a_gm, [m, k_tile], offsets=[0, kk])
        b = asc2.load(b_gm, [k_tile, n], offsets=[kk, 0])
        asc2.matmul_acc(a, b, acc)
    asc2.store(asc2.relu(acc + bias.broadcast_to(m, n)), c_gm, offsets=[0, 0])


@asc2.jit(always_compile=True)
def linear_mn_tiles(a_ptr: asc.GlobalAddress, b_ptr: asc.GlobalAddress, bias_ptr: asc.GlobalAddress,
                    c_ptr: asc.GlobalAddress, m: int, n: asc.ConstExpr[int], k: asc.ConstExpr[int],
                    m_tile: asc.ConstExpr[int], n_tile: asc.ConstExpr[int], relu: asc.ConstExpr[int],
                    out_dtype: asc.ConstExpr):
    """A linear layer tiled over M and N: every tile adds its own slice of a bias vector (of any floating type,
    widened to fp32) to the product, then an optional ReLU and a cast."""
    a_gm, b_gm, c_gm = asc2.tensor(a_ptr, [m, k]), asc2.tensor(b_ptr, [k, n]), asc2.tensor(c_ptr, [m, n])
    bias_gm = asc2.tensor(bias_ptr, [n])
    n_blocks = asc.ceildiv(n, n_tile)
    for t in range(asc2.block_idx(), asc.ceildiv(m, m_tile) * n_blocks, asc2.block_num()):
        i, j = (t // n_blocks) * m_tile, (t % n_blocks) * n_tile
        a = asc2.load(a_gm, [m_tile, k], offsets=[i, 0])
        b = asc2.load(b_gm, [k, n_tile], offsets=[0, j])
        bias = asc2.load(bias_gm, [n_tile], offsets=[j]).to(asc.float32)
        v = bias.reshape(1, n_tile).broadcast_to(m_tile, n_tile) + asc2.matmul(a, b)
        if relu:
            v = asc2.relu(v)
        if out_dtype != asc.float32:
            v = v.to(out_dtype)
        asc2.store(v, c_gm, offsets=[i, j])


@asc2.jit(always_compile=True)
def matmul_of_computed_operands(a_ptr: asc.GlobalAddress, b_ptr: asc.GlobalAddress, s_ptr: asc.GlobalAddress,
                                c_ptr: asc.GlobalAddress, m: int, k: asc.ConstExpr[int], n: asc.ConstExpr[int],
                                m_tile: asc.ConstExpr[int], k_tile: asc.ConstExpr[int]):
    """Operands prepared on the way to the cube unit: fp32 activations cast to fp16 (after a ReLU), weights scaled
    elementwise by a second matrix; accumulated over a K loop."""
    a_gm, b_gm, s_gm = asc2.tensor(a_ptr, [m, k]), asc2.tensor(b_ptr, [k, n]), asc2.tensor(s_ptr, [k, n])
    c_gm = asc2.tensor(c_ptr, [m, n])
    for i in range(asc2.block_idx() * m_tile, m, asc2.block_num() * m_tile):
        acc = asc2.zeros_acc([m_tile, n], dtype=asc.float32)
        for kk in range(0, k, k_tile):
            a = asc2.relu(asc2.load(a_gm, [m_tile, k_tile], offsets=[i, kk])).to(asc.float16)
            b = asc2.load(b_gm, [k_tile, n], offsets=[kk, 0]) * asc2.load(s_gm, [k_tile, n], offsets=[kk, 0])
            asc2.matmul_acc(a, b, acc)
        asc2.store(acc, c_gm, offsets=[i, 0])


@asc2.jit(always_compile=True)
def row_losses(x_ptr: asc.GlobalAddress, t_ptr: asc.GlobalAddress, mse_ptr: asc.GlobalAddress, ce_ptr: asc.GlobalAddress,
               rows: int, cols: asc.ConstExpr[int]):
    """Two losses per row, one row per iteration (a one-row tile reduced to one element is stored as a scalar):
    the mean squared error, and the cross entropy of the row's logits against a row of target probabilities."""
    x_gm, t_gm = asc2.tensor(x_ptr, [rows, cols]), asc2.tensor(t_ptr, [rows, cols])
    mse_gm, ce_gm = asc2.tensor(mse_ptr, [rows]), asc2.tensor(ce_ptr, [rows])
    for i in range(asc2.block_idx(), rows, asc2.block_num()):
        x = asc2.load(x_gm, [1, cols], offsets=[i, 0])
        t = asc2.load(t_gm, [1, cols], offsets=[i, 0])
        d = x - t
        asc2.store(asc2.reduce_sum(d * d, 1) / cols, mse_gm, offsets=[i])
        mx = asc2.reduce_max(x, 1, keep_dims=True).broadcast_to(1, cols)
        lse = asc2.log(asc2.reduce_sum(asc2.exp(x - mx), 1)) + asc2.reduce_max(x, 1)
        asc2.store(lse - asc2.reduce_sum(x * t, 1), ce_gm, offsets=[i])


@asc2.jit(always_compile=True)
def quantise_int8(x_ptr: asc.GlobalAddress, q_ptr: asc.GlobalAddress, inv_scale: float, n: int, tile: asc.ConstExpr[int]):
    """fp32 -> int8: round half up, clamp to [-128, 127], narrow through int32 (the reference casts between floats
    and integers of one width only, and between integers of any widths)."""
    x_gm, q_gm = asc2.tensor(x_ptr, [n]), asc2.tensor(q_ptr, [n])
    for i in range(asc2.block_idx() * tile, n, asc2.block_num() * tile):
        x = asc2.load(x_gm, [tile], offsets=[i])
        r = asc2.minimum(asc2.maximum(asc2.floor(x * inv_scale + 0.5), -128.0), 127.0)
        asc2.store(r.to(asc.int32).to(asc.int8), q_gm, offsets=[i])


@asc2.jit(always_compile=True)
def dequantise_int8(q_ptr: asc.GlobalAddress, keep_ptr: asc.GlobalAddress, x_ptr: asc.GlobalAddress, scale: float, n: int,
                    tile: asc.ConstExpr[int]):
    """int8 -> fp32 through int32, zeroed where a uint8 keep mask is 0 (unsigned tiles can be compared, not cast)."""
    q_gm, keep_gm, x_gm = asc2.tensor(q_ptr, [n]), asc2.tensor(keep_ptr, [n]), asc2.tensor(x_ptr, [n])
    for i in range(asc2.block_idx() * tile, n, asc2.block_num() * tile):
        q = asc2.load(q_gm, [tile], offsets=[i]).to(asc.int32).to(asc.float32)
        keep = asc2.load(keep_gm, [tile], offsets=[i])
        asc2.store(asc2.where(keep != 0, q * scale, 0.0), x_gm, offsets=[i])


@asc2.jit(always_compile=True)
def softmax_with_temperature(x_ptr: asc.GlobalAddress, bias_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress,
                             inv_t: float, rows: int, cols: asc.ConstExpr[int], rpt: asc.ConstExpr[int]):
    """asc2.softmax of a computed tile: scaled logits plus a bias row."""
    x_gm, out_gm = asc2.tensor(x_ptr, [rows, cols]), asc2.tensor(out_ptr, [rows, cols])
    bias = asc2.load(asc2.tensor(bias_ptr, [1, cols]), [1, cols], offsets=[0, 0])
    for i in range(asc2.block_idx() * rpt, rows, asc2.block_num() * rpt):
        x = asc2.load(x_gm, [rpt, cols], offsets=[i, 0])
        asc2.store(asc2.softmax(x * inv_t + bias.broadcast_to(rpt, cols)), out_gm, offsets=[i, 0])


@asc2.jit(always_compile=True)
def glu_rows(x_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, rows: int, cols: asc.ConstExpr[int],
             rpt: asc.ConstExpr[int]):
    """A gated linear unit: the two halves of every row of x, a * sigmoid(g)."""
    x_gm, out_gm = asc2.tensor(x_ptr, [rows, 2 * cols]), asc2.tensor(out_ptr, [rows, cols])
    for r in range(asc2.block_idx() * rpt, rows, asc2.block_num() * rpt):
        a = asc2.load(x_gm, [rpt, cols], offsets=[r, 0])
        g = asc2.load(x_gm, [rpt, cols], offsets=[r, cols])
        asc2.store(a / (asc2.exp(-g) + 1), out_gm, offsets=[r, 0])


@asc2.jit(always_compile=True)
def tile_over_its_own_reduction(x_ptr: asc.GlobalAddress, b_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress,
                                rows: int, cols: asc.ConstExpr[int], rpt: asc.ConstExpr[int], op: asc.ConstExpr):
    """Every [rpt, cols] tile divided by a reduction of the whole tile, plus a 1-D bias vector reshaped to a row."""
    x_gm, b_gm, out_gm = asc2.tensor(x_ptr, [rows, cols]), asc2.tensor(b_ptr, [cols]), asc2.tensor(out_ptr, [rows, cols])
    for r in range(asc2.block_idx() * rpt, rows, asc2.block_num() * rpt):
        x = asc2.load(x_gm, [rpt, cols], offsets=[r, 0])
        asc2.store(x / op(x), out_gm, offsets=[r, 0])


@asc2.jit(always_compile=True)
def add_vector_bias(x_ptr: asc.GlobalAddress, b_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, rows: int,
                    cols: asc.ConstExpr[int], rpt: asc.ConstExpr[int]):
    x_gm, b_gm, out_gm = asc2.tensor(x_ptr, [rows, cols]), asc2.tensor(b_ptr, [cols]), asc2.tensor(out_ptr, [rows, cols])
    bias = asc2.load(b_gm, [cols], offsets=[0])
    for r in range(asc2.block_idx() * rpt, rows, asc2.block_num() * rpt):
        asc2.store(asc2.load(x_gm, [rpt, cols], offsets=[r, 0]) + bias.reshape(1, cols).broadcast_to(rpt, cols), out_gm,
                   offsets=[r, 0])


@asc2.jit(always_compile=True)
def copy_window(x_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, rows: int, x_cols: asc.ConstExpr[int],
                out_cols: asc.ConstExpr[int], cols: asc.ConstExpr[int], x_col0: asc.ConstExpr[int],
                out_col0: asc.ConstExpr[int], rpt: asc.ConstExpr[int]):
    """Moves a [rows, cols] window of one matrix into a window of another, rpt rows at a time, whatever the type."""
    x_gm, out_gm = asc2.tensor(x_ptr, [rows, x_cols]), asc2.tensor(out_ptr, [rows, out_cols])
    for r in range(asc2.block_idx() * rpt, rows, asc2.block_num() * rpt):
        asc2.store(asc2.load(x_gm, [rpt, cols], offsets=[r, x_col0]), out_gm, offsets=[r, out_col0])


@asc2.jit(always_compile=True)
def split_row_reduce(x_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, rows: asc.ConstExpr[int],
                     cols: asc.ConstExpr[int], col_tile: asc.ConstExpr[int], op: asc.ConstExpr, atomic: asc.ConstExpr):
    """Row reductions split over column blocks: every block reduces its [rows, col_tile] tiles along the rows and
    accumulates the partial results into the output vector with an atomic."""
    x_gm, out_gm = asc2.tensor(x_ptr, [rows, cols]), asc2.tensor(out_ptr, [rows])
    for c in range(asc2.block_idx() * col_tile, cols, asc2.block_num() * col_tile):
        x = asc2.load(x_gm, [rows, col_tile], offsets=[0, c])
        atomic(op(x * x, 1), out_gm, offsets=[0])


@asc2.jit(always_compile=True)
def column_softmax(x_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, tiles: int, rows: asc.ConstExpr[int],
                   cols: asc.ConstExpr[int]):
    """Softmax down the columns of every [rows, cols] tile: reductions along the first axis, repeated over the rows."""
    x_gm, out_gm = asc2.tensor(x_ptr, [tiles * rows, cols]), asc2.tensor(out_ptr, [tiles * rows, cols])
    for t in range(asc2.block_idx(), tiles, asc2.block_num()):
        x = asc2.load(x_gm, [rows, cols], offsets=[t * rows, 0])
        e = asc2.exp(x - asc2.reduce_max(x, 0, keep_dims=True).broadcast_to(rows, cols))
        asc2.store(e / asc2.reduce_sum(e, 0, keep_dims=True).broadcast_to(rows, cols), out_gm, offsets=[t * rows, 0])


@asc2.jit(always_compile=True)
def column_standardise(x_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, tiles: int, rows: asc.ConstExpr[int],
                       cols: asc.ConstExpr[int], eps: float):
    """(x - mean) / sqrt(var + eps) with the statistics taken down the columns of every tile (a batch norm's core)."""
    x_gm, out_gm = asc2.tensor(x_ptr, [tiles * rows, cols]), asc2.tensor(out_ptr, [tiles * rows, cols])
    for t in range(asc2.block_idx(), tiles, asc2.block_num()):
        x = asc2.load(x_gm, [rows, cols], offsets=[t * rows, 0])
        d = x - (asc2.reduce_sum(x, 0, keep_dims=True) * (1.0 / rows)).broadcast_to(rows, cols)
        var = asc2.reduce_sum(d * d, 0, keep_dims=True) * (1.0 / rows)
        asc2.store(d * asc2.rsqrt(var + eps).broadcast_to(rows, cols), out_gm, offsets=[t * rows, 0])


def mn_tiles_per_block(m, n, core_num, m_tile, n_tile, n_tiles_per_block):
    """Host-side tile bookkeeping of the M/N-blocked kernel (even distribution over blocks)."""
    m_tiles, n_tiles = m // m_tile, n // n_tile
    assert m % m_tile == 0 and n % n_tile == 0 and (m_tiles * n_tiles) % core_num == 0
    per_core = (m_tiles * n_tiles) // core_num
    assert n_tiles % n_tiles_per_block == 0 and per_core % n_tiles_per_block == 0
    m_tiles_per_block = per_core // n_tiles_per_block
    assert m_tiles % m_tiles_per_block == 0
    return m_tiles_per_block


# ---- elementwise kernels (python/test/asc2/kernels/test_{leaky_relu,gelu}.py and
# ---- python/test/asc2/operations/test_{binary_ops,unary_ops,where}.py)
@asc2.jit(always_compile=True)
def leaky_relu(x_ptr: asc.GlobalAddress, alpha: float, out_ptr: asc.GlobalAddress, size: int,
               tile_size: asc.ConstExpr[int], tile_per_block: asc.ConstExpr[int]):
    x_gm = asc2.tensor(x_ptr, [size])
    out_gm = asc2.tensor(out_ptr, [size])
    base_offset = asc2.block_idx() * tile_size * tile_per_block
    for i in range(tile_per_block, unroll_factor=2, parallel=True):
        tile_offset = base_offset + i * tile_size
        x = asc2.load(x_gm, [tile_size], offsets=[tile_offset])
        out = asc2.where(x >= 0, x, x * alpha)
        asc2.store(out, out_gm, offsets=[tile_offset])


@asc2.jit(always_compile=True)
def gelu(x_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, num_rows: asc.ConstExpr, num_columns: asc.ConstExpr,
         tile_size: asc.ConstExpr, approximate: asc.ConstExpr):
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


VV, VS, SV = "VV", "VS", "SV"


@asc2.jit(always_compile=True)
def binary_op(x_ptr, y_ptr, z_ptr, block_length: asc.ConstExpr, fmt: asc.ConstExpr, op: asc.ConstExpr) -> None:
    if fmt == VV:
        xt = asc2.load(asc2.tensor(x_ptr, [32]), [block_length], offsets=[0])
        yt = asc2.load(asc2.tensor(y_ptr, [32]), [block_length], offsets=[0])
    elif fmt == VS:
        xt = asc2.load(asc2.tensor(x_ptr, [32]), [block_length], offsets=[0])
        yt = y_ptr
    elif fmt == SV:
        xt = x_ptr
        yt = asc2.load(asc2.tensor(y_ptr, [32]), [block_length], offsets=[0])
    zt = op(xt, yt)
    asc2.store(zt, asc2.tensor(z_ptr, [32]), offsets=[0])


@asc2.jit(always_compile=True)
def unary_op(x_ptr: asc.GlobalAddress, z_ptr: asc.GlobalAddress, block_length: asc.ConstExpr, op: asc.ConstExpr) -> None:
    xt = asc2.load(asc2.tensor(x_ptr, [32]), [block_length], offsets=[0])
    zt = op(xt)
    asc2.store(zt, asc2.tensor(z_ptr, [32]), offsets=[0])


WHERE_SIZE = 32


@asc2.jit(always_compile=True)
def where_op(x_ptr: asc.GlobalAddress, y_ptr: asc.GlobalAddress, z_ptr: asc.GlobalAddress, op: asc.ConstExpr):
    x = asc2.tensor(x_ptr, [WHERE_SIZE])
    y = asc2.tensor(y_ptr, [WHERE_SIZE])
    z = asc2.tensor(z_ptr, [WHERE_SIZE])
    xt = asc2.load(x, [WHERE_SIZE], offsets=[0])
    yt = asc2.load(y, [WHERE_SIZE], offsets=[0])
    zt = asc2.where(op(xt, yt), xt, yt)
    asc2.store(zt, z, offsets=[0])


@asc2.jit(always_compile=True)
def where_scalar_op(x_ptr: asc.GlobalAddress, scalar, z_ptr: asc.GlobalAddress, op: asc.ConstExpr):
    x = asc2.tensor(x_ptr, [WHERE_SIZE])
    z = asc2.tensor(z_ptr, [WHERE_SIZE])
    xt = asc2.load(x, [WHERE_SIZE], offsets=[0])
    zt = asc2.where(op(xt, scalar), asc.number(0.0, x_ptr.dtype), asc.number(1.0, x_ptr.dtype))
    asc2.store(zt, z, offsets=[0])


# ---- reductions and the softmax op (python/test/asc2/operations/test_{reduce_ops,softmax}.py)
@asc2.jit(always_compile=True)
def reduce_axis(input_ptr: asc.GlobalAddress, output_ptr: asc.GlobalAddress, reduce_dim: asc.ConstExpr,
                input_shape: asc.ConstExpr, input_offsets: asc.ConstExpr, output_shape: asc.ConstExpr,
                output_offsets: asc.ConstExpr, op: asc.ConstExpr, keep_dims: asc.ConstExpr) -> None:
    g_input = asc2.tensor(input_ptr, input_shape)
    g_output = asc2.tensor(output_ptr, output_shape)
    input = asc2.load(g_input, input_shape, offsets=input_offsets)
    output = op(input, reduce_dim, keep_dims=keep_dims)
    asc2.store(output, g_output, offsets=output_offsets)


@asc2.jit(always_compile=True)
def reduce_all(input_ptr: asc.GlobalAddress, output_ptr: asc.GlobalAddress, input_shape: asc.ConstExpr,
               input_offsets: asc.ConstExpr, output_shape: asc.ConstExpr, output_offsets: asc.ConstExpr,
               op: asc.ConstExpr) -> None:
    g_input = asc2.tensor(input_ptr, input_shape)
    g_output = asc2.tensor(output_ptr, output_shape)
    input = asc2.load(g_input, input_shape, offsets=input_offsets)
    scalar = op(input)
    output = asc2.full(output_shape, scalar, dtype=input.dtype)
    asc2.store(output, g_output, offsets=output_offsets)


@asc2.jit(always_compile=True)
def reduce_tile(x_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, size: int, tile_size: asc.ConstExpr[int]):
    x_gm = asc2.tensor(x_ptr, [size])
    out_gm = asc2.tensor(out_ptr, [1])
    tile = asc2.load(x_gm, [tile_size], offsets=[0])
    max_val = asc2.reduce_max(tile)
    result = asc2.full([1], max_val, dtype=tile.dtype)
    asc2.store(result, out_gm, offsets=[0])


@asc2.jit(always_compile=True)
def row_sums(x_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, num_rows: int, num_cols: asc.ConstExpr[int],
             rows_per_tile: asc.ConstExpr[int]):
    """Each block walks row tiles and stores their row sums: the tiles merge into one call."""
    x_gm = asc2.tensor(x_ptr, [num_rows, num_cols])
    out_gm = asc2.tensor(out_ptr, [num_rows])
    for i in range(asc2.block_idx() * rows_per_tile, num_rows, asc2.block_num() * rows_per_tile):
        tile = asc2.load(x_gm, [rows_per_tile, num_cols], offsets=[i, 0])
        asc2.store(asc2.reduce_sum(tile, 1), out_gm, offsets=[i])


@asc2.jit(always_compile=True)
def softmax_1d(dst_ptr, src_ptr, length: asc.ConstExpr) -> None:
    dst = asc2.tensor(dst_ptr, [length])
    src = asc2.tensor(src_ptr, [length])
    src_tile = asc2.load(src, shape=[length], offsets=[0])
    dst_tile = asc2.softmax(src_tile)
    asc2.store(dst_tile, dst, offsets=[0])
    asc2.store(src_tile, src, offsets=[0])


@asc2.jit(always_compile=True)
def softmax_2d(dst_ptr, src_ptr, shape: asc.ConstExpr) -> None:
    dst = asc2.tensor(dst_ptr, shape)
    src = asc2.tensor(src_ptr, shape)
    src_tile = asc2.load(src, shape=shape, offsets=[0, 0])
    dst_tile = asc2.softmax(src_tile)
    asc2.store(dst_tile, dst, offsets=[0, 0])
    asc2.store(src_tile, src, offsets=[0, 0])


# ---- loads and stores of tiles anywhere in a tensor (python/test/asc2/operations/test_memory_ops.py)
@asc2.jit(always_compile=True)
def add_static(x_ptr, y_ptr, z_ptr, tensor_shape: asc.ConstExpr, tile_shape: asc.ConstExpr, tile_id: asc.ConstExpr,
               offsets: asc.ConstExpr) -> None:
    xt = asc2.load(asc2.tensor(x_ptr, tensor_shape), tile_shape, tile_id=tile_id, offsets=offsets)
    yt = asc2.load(asc2.tensor(y_ptr, tensor_shape), tile_shape, tile_id=tile_id, offsets=offsets)
    zt = xt + yt
    asc2.store(zt, asc2.tensor(z_ptr, tensor_shape), tile_id=tile_id, offsets=offsets)


@asc2.jit(always_compile=True)
def add_dynamic_1d(x_ptr, y_ptr, z_ptr, ts0, tile_shape: asc.ConstExpr, tile_id: asc.ConstExpr,
                   offsets: asc.ConstExpr) -> None:
    xt = asc2.load(asc2.tensor(x_ptr, [ts0]), tile_shape, tile_id=tile_id, offsets=offsets)
    yt = asc2.load(asc2.tensor(y_ptr, [ts0]), tile_shape, tile_id=tile_id, offsets=offsets)
    zt = xt + yt
    asc2.store(zt, asc2.tensor(z_ptr, [ts0]), tile_id=tile_id, offsets=offsets)


@asc2.jit(always_compile=True)
def add_dynamic_2d(x_ptr, y_ptr, z_ptr, ts0, ts1, tile_shape: asc.ConstExpr, tile_id: asc.ConstExpr,
                   offsets: asc.ConstExpr) -> None:
    xt = asc2.load(asc2.tensor(x_ptr, [ts0, ts1]), tile_shape, tile_id=tile_id, offsets=offsets)
    yt = asc2.load(asc2.tensor(y_ptr, [ts0, ts1]), tile_shape, tile_id=tile_id, offsets=offsets)
    zt = xt + yt
    asc2.store(zt, asc2.tensor(z_ptr, [ts0, ts1]), tile_id=tile_id, offsets=offsets)


@asc2.jit(always_compile=True)
def add_scalar(x_ptr, y_ptr, z_ptr, tensor_shape: asc.ConstExpr, offsets: asc.ConstExpr) -> None:
    xt = asc2.load(asc2.tensor(x_ptr, tensor_shape), offsets=offsets)
    yt = asc2.load(asc2.tensor(y_ptr, tensor_shape), offsets=offsets)
    zt = xt + yt
    asc2.store(zt, asc2.tensor(z_ptr, tensor_shape), offsets=offsets)


@asc2.jit(always_compile=True)
def copy_1elem(x_ptr, y_ptr, tensor_shape: asc.ConstExpr, offsets: asc.ConstExpr):
    x = asc2.tensor(x_ptr, tensor_shape)
    s = asc2.load(x, offsets=offsets)
    y = asc2.tensor(y_ptr, tensor_shape)
    asc2.store(asc2.full([1], s), y, offsets=offsets)


@asc2.jit(always_compile=True)
def scale_2d_tiles(x_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, rows: int, cols: int, alpha: float,
                   tile_r: asc.ConstExpr[int], tile_c: asc.ConstExpr[int]):
    """Blocks walk the 2-D tile grid of a matrix (tile_id addressing); edge tiles are ragged."""
    x_gm = asc2.tensor(x_ptr, [rows, cols])
    out_gm = asc2.tensor(out_ptr, [rows, cols])
    tiles_c = asc.ceildiv(cols, tile_c)
    num_tiles = asc.ceildiv(rows, tile_r) * tiles_c
    for t in range(asc2.block_idx(), num_tiles, asc2.block_num()):
        tile = asc2.load(x_gm, [tile_r, tile_c], tile_id=[t // tiles_c, t % tiles_c])
        asc2.store(asc2.tanh(tile * alpha), out_gm, tile_id=[t // tiles_c, t % tiles_c])


# ---- shape operations and atomics (python/test/asc2/operations/test_{shape_ops,atomic_ops}.py)
@asc2.jit(always_compile=True)
def shape_op(x_ptr, z_ptr, input_shape: asc.ConstExpr, output_shape: asc.ConstExpr, in_offsets: asc.ConstExpr,
             out_offsets: asc.ConstExpr, op: asc.ConstExpr, op_param: asc.ConstExpr) -> None:
    xt = asc2.load(asc2.tensor(x_ptr, input_shape), input_shape, offsets=in_offsets)
    zt = op(xt, *op_param)
    asc2.store(zt, asc2.tensor(z_ptr, output_shape), offsets=out_offsets)


@asc2.jit(always_compile=True)
def broadcast_dup(out_ptr, shape: asc.ConstExpr, offsets: asc.ConstExpr):
    out_tensor = asc2.tensor(out_ptr, shape)
    out = asc2.full([1], 777, out_tensor.dtype).broadcast_to(*out_tensor.shape)
    asc2.store(out, out_tensor, offsets=offsets)


@asc2.jit(always_compile=True)
def atomic_op(x_ptr: asc.GlobalAddress, z_ptr: asc.GlobalAddress, tensor_shape: asc.ConstExpr, tile_length: asc.ConstExpr,
              op: asc.ConstExpr):
    offset_x = asc.get_block_idx() * tile_length
    xt = asc2.load(asc2.tensor(x_ptr, tensor_shape), [tile_length], offsets=[offset_x])
    xt += asc2.full_like(xt, 10)
    op(xt, asc2.tensor(z_ptr, [tile_length]), offsets=[0])


@asc2.jit(always_compile=True)
def add_row_bias(x_ptr: asc.GlobalAddress, b_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, rows: int,
                 cols: asc.ConstExpr[int], rows_per_tile: asc.ConstExpr[int]):
    """out = relu(x + bias) with one bias row broadcast over the rows of every tile."""
    x_gm = asc2.tensor(x_ptr, [rows, cols])
    out_gm = asc2.tensor(out_ptr, [rows, cols])
    bias = asc2.load(asc2.tensor(b_ptr, [1, cols]), [1, cols], offsets=[0, 0])
    for i in range(asc2.block_idx() * rows_per_tile, rows, asc2.block_num() * rows_per_tile):
        x = asc2.load(x_gm, [rows_per_tile, cols], offsets=[i, 0])
        asc2.store(asc2.relu(x + asc2.broadcast_to(bias, rows_per_tile, cols)), out_gm, offsets=[i, 0])


# ---- RMS normalisation (asc2.rms_norm, python/asc/language/tile/unary_ops.py:225-237)
@asc2.jit
def rms_norm_rows(x_ptr: asc.GlobalAddress, gamma_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, num_rows: int,
                  num_cols: asc.ConstExpr[int], block_size: asc.ConstExpr[int], epsilon: float):
    x_gm = asc2.tensor(x_ptr, [num_rows, num_cols])
    out_gm = asc2.tensor(out_ptr, [num_rows, num_cols])
    gamma = asc2.load(asc2.tensor(gamma_ptr, [1, num_cols]), [1, num_cols], offsets=[0, 0])
    for r0 in asc2.range(asc2.block_idx() * block_size, num_rows, asc2.block_num() * block_size):
        x = asc2.load(x_gm, [block_size, num_cols], offsets=[r0, 0])
        asc2.store(asc2.rms_norm(x, gamma, epsilon), out_gm, offsets=[r0, 0])


@asc2.jit
def rms_norm_1d(x_ptr: asc.GlobalAddress, gamma_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress,
                length: asc.ConstExpr[int]):
    x = asc2.load(asc2.tensor(x_ptr, [length]), [length], offsets=[0])
    gamma = asc2.load(asc2.tensor(gamma_ptr, [length]), [length], offsets=[0])
    asc2.store(asc2.rms_norm(x, gamma, 1e-6), asc2.tensor(out_ptr, [length]), offsets=[0])


# ---- concat (asc2.concat, python/asc/language/tile/creation_ops.py:56-72): tiles joined along the first dimension
@asc2.jit
def concat_rows(a_ptr: asc.GlobalAddress, b_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, rows_a: asc.ConstExpr[int],
                rows_b: asc.ConstExpr[int], cols: asc.ConstExpr[int], blocks_rows: asc.ConstExpr[int]):
    """Every block joins ``blocks_rows`` rows of a (doubled) with the matching rows of b and stores them as one tile."""
    a_gm = asc2.tensor(a_ptr, [rows_a, cols])
    b_gm = asc2.tensor(b_ptr, [rows_b, cols])
    out_gm = asc2.tensor(out_ptr, [rows_a + rows_b, cols])
    i = asc2.block_idx() * blocks_rows
    a = asc2.load(a_gm, [blocks_rows, cols], offsets=[i, 0])
    b = asc2.load(b_gm, [blocks_rows, cols], offsets=[i, 0])
    asc2.store(asc2.concat(a * 2, b), out_gm, offsets=[2 * i, 0])


@asc2.jit
def concat_1d(a_ptr: asc.GlobalAddress, b_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, n: asc.ConstExpr[int]):
    a = asc2.load(asc2.tensor(a_ptr, [n]), [n], offsets=[0])
    b = asc2.load(asc2.tensor(b_ptr, [n]), [n], offsets=[0])
    asc2.store(asc2.concat(a, asc2.concat(b, a + b)), asc2.tensor(out_ptr, [3 * n]), offsets=[0])


# ---- expressions that reduce their own intermediate tiles along the row (row programs)
@asc2.jit
def layer_norm_rows(x_ptr: asc.GlobalAddress, gamma_ptr: asc.GlobalAddress, beta_ptr: asc.GlobalAddress,
                    out_ptr: asc.GlobalAddress, num_rows: int, num_cols: asc.ConstExpr[int],
                    block_size: asc.ConstExpr[int], epsilon: float):
    x_gm = asc2.tensor(x_ptr, [num_rows, num_cols])
    out_gm = asc2.tensor(out_ptr, [num_rows, num_cols])
    gamma = asc2.load(asc2.tensor(gamma_ptr, [1, num_cols]), [1, num_cols], offsets=[0, 0])
    beta = asc2.load(asc2.tensor(beta_ptr, [1, num_cols]), [1, num_cols], offsets=[0, 0])
    for r0 in asc2.range(asc2.block_idx() * block_size, num_rows, asc2.block_num() * block_size):
        x = asc2.load(x_gm, [block_size, num_cols], offsets=[r0, 0])
        mean = (asc2.reduce_sum(x, 1) / num_cols).reshape(block_size, 1).broadcast_to(block_size, num_cols)
        xc = x - mean
        var = (asc2.reduce_sum(xc * xc, 1, keep_dims=True) / num_cols).broadcast_to(block_size, num_cols)
        y = xc * asc2.rsqrt(var + epsilon)
        asc2.store(y * gamma.broadcast_to(block_size, num_cols) + beta.broadcast_to(block_size, num_cols), out_gm,
                   offsets=[r0, 0])


@asc2.jit
def l1_normalize_rows(x_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, num_rows: int, num_cols: asc.ConstExpr[int]):
    x_gm = asc2.tensor(x_ptr, [num_rows, num_cols])
    out_gm = asc2.tensor(out_ptr, [num_rows, num_cols])
    for i in asc2.range(asc2.block_idx(), num_rows, asc2.block_num()):
        row = asc2.load(x_gm, [1, num_cols], offsets=[i, 0])
        asc2.store(row / (asc2.reduce_sum(asc2.abs(row)) + 1e-6), out_gm, offsets=[i, 0])


@asc2.jit
def row_sum_of_squares(x_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, num_rows: int, num_cols: asc.ConstExpr[int],
                       block_size: asc.ConstExpr[int]):
    x_gm = asc2.tensor(x_ptr, [num_rows, num_cols])
    out_gm = asc2.tensor(out_ptr, [num_rows])
    for r0 in asc2.range(asc2.block_idx() * block_size, num_rows, asc2.block_num() * block_size):
        x = asc2.load(x_gm, [block_size, num_cols], offsets=[r0, 0])
        asc2.store(asc2.sqrt(asc2.reduce_sum(x * x, 1)) * 0.5 + asc2.reduce_max(asc2.abs(x), 1), out_gm, offsets=[r0])


@asc2.jit
def row_norms_scalar(x_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress, num_rows: int, num_cols: asc.ConstExpr[int]):
    """One scalar per row, stored the way the reference stores scalars: through a one-element tile."""
    x_gm = asc2.tensor(x_ptr, [num_rows, num_cols])
    out_gm = asc2.tensor(out_ptr, [num_rows])
    for i in asc2.range(asc2.block_idx(), num_rows, asc2.block_num()):
        row = asc2.load(x_gm, [1, num_cols], offsets=[i, 0])
        energy = asc2.reduce_sum(row * row) / num_cols + asc2.reduce_max(asc2.abs(row))
        asc2.store(asc2.full([1], energy, dtype=row.dtype), out_gm, offsets=[i])


@asc2.jit
def scale_rows(x_ptr: asc.GlobalAddress, scale_ptr: asc.GlobalAddress, bias_ptr: asc.GlobalAddress, out_ptr: asc.GlobalAddress,
               num_rows: int, num_cols: asc.ConstExpr[int], block_size: asc.ConstExpr[int]):
    """out[r, c] = x[r, c] * scale[r] + bias[r]: loaded [rows] vectors, each element repeated along its row."""
    x_gm = asc2.tensor(x_ptr, [num_rows, num_cols])
    out_gm = asc2.tensor(out_ptr, [num_rows, num_cols])
    scale_gm = asc2.tensor(scale_ptr, [num_rows])
    bias_gm = asc2.tensor(bias_ptr, [num_rows])
    for r0 in asc2.range(asc2.block_idx() * block_size, num_rows, asc2.block_num() * block_size):
        x = asc2.load(x_gm, [block_size, num_cols], offsets=[r0, 0])
        scale = asc2.load(scale_gm, [block_size], offsets=[r0]).reshape(block_size, 1).broadcast_to(block_size, num_cols)
        bias = asc2.expand_dims(asc2.load(bias_gm, [block_size], offsets=[r0]), 1).broadcast_to(block_size, num_cols)
        asc2.store(x * scale + bias, out_gm, offsets=[r0, 0])
