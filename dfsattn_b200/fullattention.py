"""Dense attention for the warm-up steps and skipped layers of the schedule.

Mirrors ``full_attention`` of ``dfsattn/fullattention.py:60-153`` for the mode
the processors use (``"flash"``: varlen attention with cu_seqlens = [0, valid,
L]).  It is the block-sparse kernel with every key block listed -- one
back-end, no flash-attn dependency.
"""
import torch

from . import engine, ops


def full_attention(q, k, v, mode="flash", drop_rate=0, attn_mask=None, causal=False, cu_seqlens_q=None,
                   cu_seqlens_kv=None, max_seqlen_q=None, max_seqlen_kv=None, batch_size=1):
    """q, k, v: [1, H, L, D] -> [1, H, L, D] (same layout as the sparse operator)."""
    if mode != "flash":
        raise ValueError(f"full_attention mode={mode!r}: only 'flash' (dense varlen) is built for B200")
    if causal or drop_rate:
        raise ValueError("dense attention here is non-causal and without dropout")
    out_dtype = q.dtype
    L = q.shape[2]
    qh, kh, vh = engine.prepare_inputs(q, k, v)
    valid = engine.valid_length(cu_seqlens_kv if cu_seqlens_kv is not None else cu_seqlens_q, L)
    out = engine.run_attention(qh, kh, vh, None, None, valid)
    return out.unsqueeze(0).to(out_dtype)
