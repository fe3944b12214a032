"""Attention forward, ``softmax(scale * Q K^T [+ causal mask]) V``, per 128-row query tile.

The reference has no attention kernel.  The script states the math on tiles with two extensions of
the CUDA platform — ``asc2.matmul(q, k, trans_b=True)`` and ``asc2.causal_mask`` — and the platform
runs it as one fused flash-attention kernel (the [q_tile, seq] score tile never exists in memory)."""
import asc
import asc2


@asc2.jit
def attention_kernel(q_ptr: asc.GlobalAddress, k_ptr: asc.GlobalAddress, v_ptr: asc.GlobalAddress,
                     o_ptr: asc.GlobalAddress, scale: float, heads: asc.ConstExpr[int], seq: asc.ConstExpr[int],
                     head_dim: asc.ConstExpr[int], q_tile: asc.ConstExpr[int], causal: asc.ConstExpr[bool],
                     dtype: asc.ConstExpr):
    rows = heads * seq
    q_gm = asc2.tensor(q_ptr, [rows, head_dim])
    k_gm = asc2.tensor(k_ptr, [rows, head_dim])
    v_gm = asc2.tensor(v_ptr, [rows, head_dim])
    o_gm = asc2.tensor(o_ptr, [rows, head_dim])
    tiles_per_head = seq // q_tile
    for t in range(asc2.block_idx(), heads * tiles_per_head, asc2.block_num()):
        head_row = (t // tiles_per_head) * seq
        q_off = (t % tiles_per_head) * q_tile
        q = asc2.load(q_gm, [q_tile, head_dim], offsets=[head_row + q_off, 0], location=asc2.TileLocation.L0A)
        k = asc2.load(k_gm, [seq, head_dim], offsets=[head_row, 0], location=asc2.TileLocation.L0B)
        v = asc2.load(v_gm, [seq, head_dim], offsets=[head_row, 0], location=asc2.TileLocation.L0B)
        s = asc2.matmul(q, k, trans_b=True) * scale
        if causal:
            s = asc2.causal_mask(s, q_off, 0)
        p = asc2.softmax(s).to(dtype)
        o = asc2.matmul(p, v).to(dtype)
        asc2.store(o, o_gm, offsets=[head_row + q_off, 0])


_ASC_DTYPE = {"float16": asc.float16, "bfloat16": asc.bfloat16}


def attention_launch(q, k, v, o, causal: bool = False, scale=None, core_num: int = 148, q_tile: int = 128,
                     stream=None):
    """q, k, v, o: contiguous [batch, heads, seq, head_dim] fp16/bf16 tensors; o is written in place."""
    batch, heads, seq, head_dim = q.shape
    if scale is None:
        scale = float(head_dim) ** -0.5
    q_tile = min(q_tile, seq)
    dtype = _ASC_DTYPE[str(q.dtype).replace("torch.", "")]
    launch = attention_kernel[core_num] if stream is None else attention_kernel[core_num, stream]
    launch(q, k, v, o, float(scale), batch * heads, seq, head_dim, q_tile, bool(causal), dtype)
    return o
