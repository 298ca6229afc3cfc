"""Dense attention for the warm-up steps and skipped layers of the schedule.

Mirrors ``full_attention`` of ``dfsattn/fullattention.py:60-153`` for the mode
the processors use (``"flash"``: varlen attention with cu_seqlens = [0, valid,
L]).  It is the block-sparse kernel with every key block listed -- one
back-end, no flash-attn dependency.
"""
from . import engine, ops


def full_attention(q, k, v, mode="flash", drop_rate=0, attn_mask=None, causal=False, cu_seqlens_q=None,
                   cu_seqlens_kv=None, max_seqlen_q=None, max_seqlen_kv=None, batch_size=1, out_row_map=None,
                   token_major_out=False, out_shards=None, out_head0=0):
    """q, k, v: [1, H, L, D] -> [1, H, L, D] (same layout as the sparse operator).

    Two additions for the fused processor path: ``out_row_map`` (int32 [L]) stores the result of
    query row i at row out_row_map[i] -- dense attention does not care about the key order, so
    inputs that were written in a permuted token order only need their rows put back -- and
    ``token_major_out`` keeps the result as [L, H, D] memory behind the [1, H, L, D] shape."""
    if mode != "flash":
        raise ValueError(f"full_attention mode={mode!r}: only 'flash' (dense varlen) is built for B200")
    if causal or drop_rate:
        raise ValueError("dense attention here is non-causal and without dropout")
    out_dtype = q.dtype
    L = q.shape[2]
    ops._need_cuda(q, k, v)
    ops.poll_status(q.device)   # raises if a kernel of an earlier call gave up on a wait
    qh, kh, vh = engine.prepare_inputs(q, k, v)
    valid = engine.valid_length(cu_seqlens_kv if cu_seqlens_kv is not None else cu_seqlens_q, L)
    out = engine.run_attention(qh, kh, vh, None, out_row_map, valid, token_major=token_major_out,
                               out_shards=out_shards, out_head0=out_head0)
    if out_shards is not None:   # scattered to sequence shards on several GPUs (ops.ShardTable)
        return None
    return engine.as_reference_layout(out, token_major_out).to(out_dtype)
