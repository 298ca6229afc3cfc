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
from . import engine, ops
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

    def forward_pair(self, q, k, v, passes, cu_seqlens_q=None, prepermuted: bool = False,
                     token_major_out: bool = False) -> torch.Tensor:
        """Two passes [2, H, L, D] through the cache logic of ``forward`` one after the other
        (``passes``: (step_idx, cache_flag, sparse_ratio) of each), with one gather launch and,
        when both passes end up with the same lists, one attention launch for both."""
        if q.shape[0] != 2 or len(passes) != 2:
            raise ValueError("forward_pair takes exactly two passes")
        _hy._reject_unsupported(self.sparse_execution, self.selector_mode, self.block_top_p, self.token_top_k,
                                self.block_size, self.q_tile_size)
        out_dtype, device = q.dtype, q.device
        ops._need_cuda(q, k, v)
        ops.poll_status(device)   # raises if a kernel of an earlier call gave up on a wait
        _, H, L, D = q.shape
        if engine.valid_length(cu_seqlens_q, L) != L:
            raise ValueError("a padded tail is not supported for a batched pair")
        qh, kh, vh = engine.prepare_inputs(*(t.reshape(1, 2 * H, L, D) for t in (q, k, v)))
        perm, _inv = engine._perm_cache.get(self.video_perm, L, L, device)
        if perm is not None and not prepermuted:
            qp, kp, vp = ops.permute_qkv(qh, kh, vh, perm)
        else:
            qp, kp, vp = qh, kh, vh
        cls = type(self)
        rec = cls.timing_recorder
        chosen = []
        for b, (step, flag, ratio) in enumerate(passes):
            self.step_idx, self.cache_flag, self.sparse_ratio = step, flag, ratio
            entry = cls._cached_metadata.get(self._mask_cache_key())
            lists = entry["block_lists"] if entry is not None else None
            if lists is None or self.cache_flag:
                t_topk = rec.start(device)
                lists = self._compute_block_lists(qp[b * H:(b + 1) * H], kp[b * H:(b + 1) * H], ratio)
                rec.stop(t_topk, phase="topk_mask", step_idx=step, layer_idx=self.layer_idx, device=device)
                if self.cache_flag:
                    cls._cached_metadata[self._mask_cache_key()] = {"block_lists": lists}
                if (cls.mask_output_dir is not None and cls.mask_layer_interval > 0
                        and self.layer_idx % cls.mask_layer_interval == 0):
                    self._export_mask(lists)
            if cls.record_density:
                self._record_density(lists, L)
            chosen.append(lists)
        t_att = rec.start(device)
        if chosen[0] is chosen[1]:
            out = ops.block_sparse_fwd(qp, kp, vp, chosen[0].idx, chosen[0].cnt, out_row_map=perm,
                                       token_major=token_major_out, batch=2)
        else:   # no entry to share (cache_flag off everywhere): each pass has its own lists
            out = torch.empty((2, L, H, D) if token_major_out else (2, H, L, D), dtype=torch.bfloat16,
                              device=device)
            for b, lists in enumerate(chosen):
                ops.block_sparse_fwd(qp[b * H:(b + 1) * H], kp[b * H:(b + 1) * H], vp[b * H:(b + 1) * H],
                                     lists.idx, lists.cnt, out_row_map=perm, token_major=token_major_out,
                                     out=out[b])
        rec.stop(t_att, phase="attention_execution", step_idx=passes[0][0], layer_idx=self.layer_idx,
                 device=device)
        return (out.permute(0, 2, 1, 3) if token_major_out else out).to(out_dtype)


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


def dfs_attention_cfg_pair(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, step_idx: int = 0,
                           skip_steps: int = 12, cache_interval: int = 12, layer_idx: int = 0,
                           sparsity: float = 0.25, sparsity_dcrt: float = 0.1, tile_size: int = 32,
                           block_size: int = 128, video_perm: Optional[torch.Tensor] = None,
                           cache_flag: bool = True, record_density: bool = False, cu_seqlens_q=None,
                           cu_seqlens_kv=None, max_seqlen_q=None, max_seqlen_kv=None,
                           sparse_execution: str = "native", hybrid_threshold: int = 8,
                           prepermuted: bool = False, token_major_out: bool = False,
                           **unsupported) -> torch.Tensor:
    """Both classifier-free-guidance passes of one denoising step in one call.

    q, k, v: [2, H, L, D]; element 0 is the pass the processor would see at counter ``step_idx``,
    element 1 the pass at ``step_idx + 1``.  The result, the mask cache and the density records are
    what ``dfs_attention(q[0:1], ..., step_idx)`` followed by ``dfs_attention(q[1:2], ...,
    step_idx + 1)`` leave behind -- the reference can only run the passes that way, its operator
    refuses a batch (dfsattn/attention_wan.py:219) -- but the Hilbert gather is one launch over
    both elements, scoring and selection run only where the reference's cache logic would run them
    (at a refresh step: once, on element 0; element 1 finds the entry element 0 stored, because the
    Wan cache key has no step or sparsity term, :147-154), and the attention is one launch in which
    both elements read the same index lists.  Returns [2, H, L, D]."""
    for name in unsupported:
        if not name.startswith("flashinfer64_"):
            raise TypeError(f"dfs_attention_cfg_pair() got an unexpected keyword argument {name!r}")
    _hy._reject_unsupported(sparse_execution, "topk", None, 0, block_size, tile_size)
    if q.dim() != 4 or q.shape[0] != 2 or k.shape != q.shape or v.shape != q.shape:
        raise ValueError("dfs_attention_cfg_pair takes q, k, v of one shape [2, H, L, D]")
    inst = _dfs_attention_instances.get(layer_idx)
    if inst is None:
        inst = DFS_Attention(step_idx, layer_idx, sparsity, cache_flag, video_perm, block_size, tile_size,
                             tile_size, sparse_execution, hybrid_threshold)
        _dfs_attention_instances[layer_idx] = inst
    inst.sparse_execution = sparse_execution
    inst.hybrid_threshold = hybrid_threshold
    if record_density and not DFS_Attention.record_density:
        DFS_Attention.set_record_density(True)
    passes = []
    for s in (step_idx, step_idx + 1):
        is_cache_step, current = _compute_cache_schedule(s, skip_steps * 2, cache_interval * 2, sparsity,
                                                         sparsity_dcrt)
        passes.append((s, cache_flag and is_cache_step, current))
    return inst.forward_pair(q, k, v, passes, cu_seqlens_q=cu_seqlens_q, prepermuted=prepermuted,
                             token_major_out=token_major_out)
