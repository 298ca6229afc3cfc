"""Processor-side glue of the fused pre-attention kernel (``dfs_qkv_prepare``).

The reference processors turn the Q/K/V projections into attention inputs with a chain of
separate passes (transpose + contiguous, RMSNorm, rotary embedding: ``dfsattn/replace_hyvideo.py:
243-290``, ``dfsattn/replace_wan.py:154-215``) and the operator then gathers all three into the
Hilbert order (``dfsattn/attention_hyvideo.py:1034-1036``).  Here the projections are read once and
Q, K, V are written once, already normalised, rotated, head-major and permuted.

A call is eligible when it is what the kernel covers: one batch, bf16 CUDA activations, head size 64
or 128, norm modules that are plain RMSNorms (``weight`` + ``eps``; over D or over H*D), rotary
tables given as (cos, sin) or complex frequencies.  Everything else takes the processors' unfused
path, which mirrors the reference line by line; both are the CUDA product, neither is a fallback to
other code.
"""
from typing import Optional, Tuple

import torch

from . import engine, ops

_table_cache = {}


def eligible(hidden_states: torch.Tensor, heads: int, width: int, max_batch: int = 1) -> bool:
    return (hidden_states.is_cuda and hidden_states.dtype == torch.bfloat16
            and 1 <= hidden_states.shape[0] <= max_batch
            and width % heads == 0 and width // heads in (64, 128))


def norm_params(module, heads: int, width: int):
    """(weight bf16, eps, across_heads) of an RMSNorm module, (None, 0, False) for no module;
    raises TypeError for a module the kernel does not cover."""
    if module is None:
        return None, 0.0, None
    weight = getattr(module, "weight", None)
    eps = getattr(module, "eps", None)
    if weight is None or getattr(module, "bias", None) is not None:
        raise TypeError("norm module without weight, or with a bias")
    if eps is None:  # torch.nn.RMSNorm(eps=None) uses the machine epsilon of the input type
        eps = torch.finfo(torch.bfloat16).eps
    if weight.numel() == width // heads:
        across = False
    elif weight.numel() == width:
        across = True
    else:
        raise TypeError("norm weight is neither per head nor over all heads")
    return weight.detach().to(torch.bfloat16).contiguous(), float(eps), across


def _cached_tables(sources, device, build):
    """Tables converted from `sources` (a tuple of tensors), cached per source tensors: an entry
    keeps references to its sources (their addresses cannot be reused while it lives) and is valid
    only for the very same, unmodified tensor objects."""
    key = tuple(id(t) for t in sources) + (str(device),)
    versions = tuple(int(t._version) for t in sources)
    hit = _table_cache.get(key)
    if hit is not None and all(a is b for a, b in zip(hit[0], sources)) and hit[1] == versions:
        return hit[2]
    tables = build()
    if len(_table_cache) >= 8:
        _table_cache.clear()
    _table_cache[key] = (tuple(sources), versions, tables)
    return tables


def rope_tables(rotary, device) -> Optional[Tuple[torch.Tensor, torch.Tensor]]:
    """fp32 2-D (cos, sin) tables from (cos, sin) [S, D] (HunyuanVideo) or complex frequencies
    [1, 1, S, D/2] / a (real, imag) pair (Wan).  Conversions are cached per source tensor."""
    if rotary is None:
        return None
    if isinstance(rotary, torch.Tensor):
        if not rotary.is_complex():
            raise TypeError("a single rotary tensor must be complex")

        def split():
            flat = rotary.reshape(-1, rotary.shape[-1])
            return (flat.real.to(device=device, dtype=torch.float32).contiguous(),
                    flat.imag.to(device=device, dtype=torch.float32).contiguous())
        return _cached_tables((rotary,), device, split)
    cos, sin = rotary
    return _cached_tables((cos, sin), device, lambda: tuple(
        t.reshape(-1, t.shape[-1]).to(device=device, dtype=torch.float32).contiguous() for t in (cos, sin)))


def token_perm(video_perm, seq_len: int, video_len: int, device):
    """int32 device permutation [seq_len] (video part permuted, text tail in place) or None."""
    perm, _inv = engine._perm_cache.get(video_perm, seq_len, video_len, device)
    return perm


def prepare(proj_q, proj_k, proj_v, heads: int, norm_q, norm_k, rotary, rope_rows: int, perm,
            out=None, out_row0: int = 0, out_len: Optional[int] = None):
    """Projections [1, rows, H*D] -> (q, k, v) bf16 [H, out_len, D] through ``ops.qkv_prepare``."""
    width = proj_q.shape[-1]
    gq, eq, aq = norm_params(norm_q, heads, width)
    gk, ek, ak = norm_params(norm_k, heads, width)
    if aq is not None and ak is not None and aq != ak:
        raise TypeError("Q and K norms of different kinds")
    across = bool(aq if aq is not None else ak)
    tabs = rope_tables(rotary, proj_q.device)
    cos, sin = tabs if tabs is not None else (None, None)
    if cos is not None and cos.shape[0] < rope_rows:
        raise TypeError("rotary table shorter than the rotated part of the sequence")
    srcs = [t.reshape(-1, width) for t in (proj_q, proj_k, proj_v)]
    srcs = [t if t.is_contiguous() else t.contiguous() for t in srcs]
    return ops.qkv_prepare(*srcs, heads, gamma_q=gq, gamma_k=gk, eps_q=eq, eps_k=ek, norm_across_heads=across,
                           cos=cos, sin=sin, rope_rows=rope_rows if cos is not None else None, perm=perm,
                           out=out, out_row0=out_row0, out_len=out_len)
