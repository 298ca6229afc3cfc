"""DFS attention operator for Wan2.1 self-attention (video tokens only).

Same public surface as ``dfsattn/attention_wan.py`` of the reference for the
native path.  Differences from the HunyuanVideo operator, all following the
reference: no text tail and no forced-dense blocks (plain top-k over every key
block, :248-253); zero padding only at the end of the sequence (:176-189); the
mask cache key has no sparsity term (:147-154), so a mask computed at a refresh
step is reused by the second classifier-free-guidance pass and by every later
step until the next refresh; ``dfs_attention`` doubles ``skip_steps`` and
``cache_interval`` because the processor's counter advances twice per
denoising step (:792-798).
"""
from typing import Any, Dict, Optional, Tuple

import torch

from . import attention_hyvideo as _hy
from .attention_hyvideo import _compute_cache_schedule  # noqa: F401  (same schedule function)

_dfs_attention_instances: Dict[int, "DFS_Attention"] = {}


class DFS_Attention(_hy.DFS_Attention):
    _cached_metadata: Dict[Tuple[Any, ...], Dict[str, Any]] = {}
    density_records: Dict[int, Dict[int, float]] = {}
    sparsity_records: Dict[int, Dict[int, Dict[str, Any]]] = {}
    execution_tile_records: Dict[int, Dict[int, Dict[str, Any]]] = {}
    record_density: bool = False
    mask_output_dir: Optional[str] = None
    timing_recorder = _hy.DFS_Attention.timing_recorder  # one recorder for both model families
    flavor = "wan"

    def __init__(self, step_idx: int, layer_idx: int, sparse_ratio: float = 0.5, cache_flag: bool = True,
                 video_perm: Optional[torch.Tensor] = None, block_size: int = 128, q_tile_size: int = 32,
                 k_tile_size: int = 32, sparse_execution: str = "native", hybrid_threshold: int = 8):
        super().__init__(step_idx, layer_idx, sparse_ratio, cache_flag, 0, video_perm, block_size,
                         q_tile_size, k_tile_size, sparse_execution, hybrid_threshold)

    def _mask_cache_key(self) -> Tuple[Any, ...]:
        return (self.layer_idx, self.sparse_execution, self.block_size, self.q_tile_size, self.k_tile_size)

    def _video_len(self, seq_len: int) -> int:
        return seq_len

    @classmethod
    def clear_cache(cls):
        cls._cached_metadata.clear()
        cls.density_records.clear()
        cls.sparsity_records.clear()
        cls.execution_tile_records.clear()


def dfs_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, step_idx: int = 0, skip_steps: int = 12,
                  cache_interval: int = 12, layer_idx: int = 0, sparsity: float = 0.25,
                  sparsity_dcrt: float = 0.1, tile_size: int = 32, block_size: int = 128,
                  video_perm: Optional[torch.Tensor] = None, cache_flag: bool = True,
                  record_density: bool = False, cu_seqlens_q=None, cu_seqlens_kv=None, max_seqlen_q=None,
                  max_seqlen_kv=None, sparse_execution: str = "native", hybrid_threshold: int = 8,
                  prepermuted: bool = False, token_major_out: bool = False, out_shards=None, out_head0: int = 0,
                  **unsupported) -> torch.Tensor:
    """q, k, v: [1, H, L, D] raster video tokens.  ``step_idx`` is the processor's
    call counter (two calls per denoising step under classifier-free guidance)."""
    for name in unsupported:
        if not name.startswith("flashinfer64_"):
            raise TypeError(f"dfs_attention() got an unexpected keyword argument {name!r}")
    _hy._reject_unsupported(sparse_execution, "topk", None, 0, block_size, tile_size)
    inst = _dfs_attention_instances.get(layer_idx)
    if inst is None:
        inst = DFS_Attention(step_idx, layer_idx, sparsity, cache_flag, video_perm, block_size, tile_size,
                             tile_size, sparse_execution, hybrid_threshold)
        _dfs_attention_instances[layer_idx] = inst
    inst.step_idx = step_idx
    is_cache_step, current = _compute_cache_schedule(step_idx, skip_steps * 2, cache_interval * 2, sparsity,
                                                     sparsity_dcrt)
    inst.sparse_ratio = current
    inst.cache_flag = cache_flag and is_cache_step
    inst.sparse_execution = sparse_execution
    inst.hybrid_threshold = hybrid_threshold
    if record_density and not DFS_Attention.record_density:
        DFS_Attention.set_record_density(True)
    return inst.forward(q=q, k=k, v=v, attn_mask=None, causal=False, drop_rate=0.0, cu_seqlens_q=cu_seqlens_q,
                        cu_seqlens_kv=cu_seqlens_kv, max_seqlen_q=max_seqlen_q, max_seqlen_kv=max_seqlen_kv,
                        batch_size=q.shape[0], prepermuted=prepermuted, token_major_out=token_major_out,
                        out_shards=out_shards, out_head0=out_head0)
