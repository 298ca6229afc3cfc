"""DFS attention operator for HunyuanVideo joint video+text sequences.

Same public surface as ``dfsattn/attention_hyvideo.py`` of the reference for
the native top-k path: ``_compute_cache_schedule`` (:40-65), ``DFS_Attention``
(:94; cache key :196-208, forward :1090-1286, class controls :1288-1334,
:1492-1740) and ``dfs_attention`` (:1743-1982).  The PyTorch gathers, pooled
scoring, ``torch.topk`` and the third-party block-sparse kernel are replaced by
calls into libdfs_b200.so; masks are kept as device-resident index lists.
``selector_mode="kp"`` (:481-489, :211-302: fine top-p over the 16 x 16-token
tiles inside the chosen blocks) adds one 64-bit tile map per list entry, which
the same attention kernel applies to its scores.
Knobs of the reference's other backends are accepted and rejected with
``ValueError`` -- there is no dispatch and no fallback.
"""
import os
from typing import Any, Dict, Optional, Tuple

import numpy as np
import torch
import torch.nn as nn

from . import engine, ops
from .engine import BlockLists
from .timing import AttentionTimingRecorder

_dfs_attention_instances: Dict[int, "DFS_Attention"] = {}


def _compute_cache_schedule(step_idx: int, skip_steps: int, cache_interval: int, sparsity: float,
                            sparsity_dcrt: float) -> Tuple[bool, float]:
    """(refresh this step?, sparsity in force); evaluated by dfs_cache_schedule."""
    return ops.cache_schedule(step_idx, skip_steps, cache_interval, sparsity, sparsity_dcrt)


def _reject_unsupported(sparse_execution, selector_mode, block_top_p, token_top_k, block_size, tile_size,
                        fine_top_p=None, kp_allowed=False):
    if sparse_execution != "native":
        raise ValueError(f"sparse_execution={sparse_execution!r}: only 'native' is built for B200")
    if selector_mode == "kp" and kp_allowed:
        if tile_size != 16 or block_size != 128:
            raise ValueError("kp mode requires 128x128 coarse blocks and 16x16 sub-blocks")
        if fine_top_p is None or not fine_top_p > 0:
            raise ValueError("kp mode needs fine_top_p > 0")
    elif selector_mode != "topk":
        raise ValueError(f"selector_mode={selector_mode!r}: 'topk' (both operators) and 'kp' (HunyuanVideo "
                         "operator) are built for B200")
    if block_top_p is not None:
        raise ValueError("block_top_p is not supported (top-k selection only)")
    if token_top_k:
        raise ValueError("token_top_k > 0 (residual tokens) is not supported")
    if block_size != 128:
        raise ValueError("block_size must be 128")
    if tile_size not in (16, 32, 64):
        raise ValueError("tile_size must be 16, 32 or 64")


class DFS_Attention(nn.Module):
    _cached_metadata: Dict[Tuple[Any, ...], Dict[str, Any]] = {}
    mask_output_dir: Optional[str] = None
    mask_head_indices: Optional[Tuple[int, ...]] = (0,)
    mask_layer_interval: int = 15
    mask_save_bool: bool = False
    record_density: bool = False
    density_records: Dict[int, Dict[int, float]] = {}
    sparsity_records: Dict[int, Dict[int, Dict[str, Any]]] = {}
    timing_recorder = AttentionTimingRecorder()
    flavor = "hyvideo"

    def __init__(self, step_idx: int, layer_idx: int, sparse_ratio: float = 0.5, cache_flag: bool = True,
                 video_len: int = 0, video_perm: Optional[torch.Tensor] = None, block_size: int = 128,
                 q_tile_size: int = 32, k_tile_size: int = 32, sparse_execution: str = "native",
                 hybrid_threshold: int = 8, block_top_p: Optional[float] = None, token_top_k: int = 0,
                 residual_candidate_blocks: int = 4, selector_mode: str = "topk", fine_top_p: float = 0.9):
        super().__init__()
        self.step_idx = step_idx
        self.layer_idx = layer_idx
        self.sparse_ratio = sparse_ratio
        self.cache_flag = cache_flag
        self.video_len = video_len
        self.video_perm = video_perm
        self.block_size = block_size
        self.q_tile_size = q_tile_size
        self.k_tile_size = k_tile_size
        self.sparse_execution = sparse_execution
        self.hybrid_threshold = hybrid_threshold
        self.block_top_p = block_top_p
        self.token_top_k = token_top_k
        self.residual_candidate_blocks = residual_candidate_blocks
        self.selector_mode = selector_mode
        self.fine_top_p = fine_top_p

    # -- cache identity: one entry per layer AND sparsity level (:196-208) ----
    def _mask_cache_key(self) -> Tuple[Any, ...]:
        return (self.layer_idx, self.block_size, self.q_tile_size, self.k_tile_size, self.sparse_ratio,
                self.block_top_p, self.token_top_k, self.residual_candidate_blocks, self.selector_mode,
                self.fine_top_p)

    def _video_len(self, seq_len: int) -> int:
        return self.video_len if self.video_len else seq_len

    def _compute_block_lists(self, q_perm, k_perm, sparse_ratio: float) -> BlockLists:
        """Score + select on permuted [H,L,D] (reference: _compute_block_mask, :388-519)."""
        if self.q_tile_size != self.k_tile_size:
            raise ValueError("q_tile_size and k_tile_size must be equal")
        return engine.compute_block_lists(q_perm, k_perm, self._video_len(q_perm.shape[1]), sparse_ratio,
                                          self.flavor, tile=self.q_tile_size,
                                          fine_top_p=self.fine_top_p if self.selector_mode == "kp" else None)

    def forward(self, q, k, v, attn_mask=None, causal: bool = False, drop_rate: float = 0.0,
                cu_seqlens_q=None, cu_seqlens_kv=None, max_seqlen_q=None, max_seqlen_kv=None,
                batch_size: int = 1, prepermuted: bool = False, token_major_out: bool = False,
                out_shards=None, out_head0: int = 0) -> torch.Tensor:
        """Reference signature plus two switches of the fused processor path: ``prepermuted`` says
        q, k, v already are in the permuted token order (written so by ``ops.qkv_prepare``), and
        ``token_major_out`` stores the result as [L, H, D] memory behind the usual [1, H, L, D]
        shape.  ``out_shards`` (an ``ops.ShardTable``) scatters the result to sequence shards on
        several GPUs instead of returning it (see ``parallel.SequenceShardExchange``)."""
        if causal or drop_rate != 0.0 or attn_mask is not None:
            raise ValueError("the B200 DFS path is non-causal, without dropout or an extra token mask")
        assert batch_size == 1 and q.shape[0] == 1, \
            "DFS Attention with block sparse currently supports batch size 1."
        _reject_unsupported(self.sparse_execution, self.selector_mode, self.block_top_p, self.token_top_k,
                            self.block_size, self.q_tile_size, self.fine_top_p, kp_allowed=self.flavor == "hyvideo")
        out_dtype = q.dtype
        device = q.device
        ops._need_cuda(q, k, v)
        ops.poll_status(device)   # raises if a kernel of an earlier call gave up on a wait
        seq_len = q.shape[2]
        video_len = self._video_len(seq_len)
        rec = DFS_Attention.timing_recorder
        qh, kh, vh = engine.prepare_inputs(q, k, v)
        perm, _inv = engine._perm_cache.get(self.video_perm, seq_len, video_len, device)
        if perm is not None and not prepermuted:
            qp, kp, vp = ops.permute_qkv(qh, kh, vh, perm)
        else:
            qp, kp, vp = qh, kh, vh

        cls = type(self)
        entry = cls._cached_metadata.get(self._mask_cache_key())
        lists: Optional[BlockLists] = entry["block_lists"] if entry is not None else None
        mask_recomputed = False
        if lists is None or self.cache_flag:
            t_sel = rec.start(device)
            t_topk = rec.start(device)
            lists = self._compute_block_lists(qp, kp, self.sparse_ratio)
            rec.stop(t_topk, phase="topk_mask", step_idx=self.step_idx, layer_idx=self.layer_idx, device=device)
            mask_recomputed = True
            if self.cache_flag:
                if self.selector_mode == "kp":
                    # as the reference (:1166-1178): only the current schedule entry of a layer is kept
                    for key in [kk for kk in cls._cached_metadata
                                if kk[0] == self.layer_idx and kk != self._mask_cache_key()]:
                        del cls._cached_metadata[key]
                cls._cached_metadata[self._mask_cache_key()] = {"block_lists": lists}
            rec.stop(t_sel, phase="topk_routing", step_idx=self.step_idx, layer_idx=self.layer_idx,
                     device=device)

        if (mask_recomputed and cls.mask_output_dir is not None and cls.mask_layer_interval > 0
                and self.layer_idx % cls.mask_layer_interval == 0):
            self._export_mask(lists)

        if cls.record_density:
            self._record_density(lists, seq_len)

        t_att = rec.start(device)
        valid = engine.valid_length(cu_seqlens_q, seq_len)
        out = engine.run_attention(qp, kp, vp, lists, perm, valid, token_major=token_major_out,
                                   out_shards=out_shards, out_head0=out_head0)
        rec.stop(t_att, phase="attention_execution", step_idx=self.step_idx, layer_idx=self.layer_idx,
                 device=device)
        if out_shards is not None:
            return None
        return engine.as_reference_layout(out, token_major_out).to(out_dtype)

    def _record_density(self, lists: BlockLists, seq_len: int) -> None:
        cls = type(self)
        if lists.fine is not None:
            # kp: density of the 16 x 16-token mask (the reference counts with logical_block_size 16, :1243)
            pairs = lists.fine_pair_count(seq_len)
        else:
            pairs = ops.interaction_count(lists.idx, lists.cnt, lists.idx.shape[0], seq_len, self.block_size)
        total = lists.idx.shape[0] * seq_len * seq_len
        cls.density_records.setdefault(self.step_idx, {})[self.layer_idx] = pairs / total
        cls.sparsity_records.setdefault(self.step_idx, {})[self.layer_idx] = {
            "block_density": pairs / total, "realized_block_sparsity": 1.0 - pairs / total,
            "residual_token_interactions": 0.0, "final_density": pairs / total,
            "final_hybrid_sparsity": 1.0 - pairs / total,
        }

    def _export_mask(self, lists: BlockLists) -> None:
        """Headless replacement of the PNG heat-maps: one .npy bool mask per head."""
        cls = type(self)
        os.makedirs(cls.mask_output_dir, exist_ok=True)
        mask = lists.to_bool_mask().cpu().numpy()
        heads = range(mask.shape[0]) if cls.mask_head_indices is None else cls.mask_head_indices
        for h in heads:
            if 0 <= h < mask.shape[0]:
                np.save(os.path.join(cls.mask_output_dir,
                                     f"step{self.step_idx:03d}_layer{self.layer_idx:03d}_head{h:02d}.npy"),
                        mask[h])

    # -- class-level controls ----------------------------------------------------
    @classmethod
    def clear_cache(cls):
        cls._cached_metadata.clear()
        cls.density_records.clear()
        cls.sparsity_records.clear()

    @classmethod
    def configure_mask_export(cls, output_dir: Optional[str], head_indices: Optional[Tuple[int, ...]] = (0,),
                              layer_interval: int = 15, save_bool: bool = False):
        if layer_interval < 1:
            raise ValueError("layer_interval must be at least 1")
        cls.mask_output_dir = output_dir
        cls.mask_head_indices = head_indices
        cls.mask_layer_interval = layer_interval
        cls.mask_save_bool = bool(save_bool)

    @classmethod
    def set_record_density(cls, enabled: bool):
        cls.record_density = bool(enabled)
        if not cls.record_density:
            cls.density_records.clear()
            cls.sparsity_records.clear()

    @classmethod
    def set_record_timing(cls, enabled: bool):
        cls.timing_recorder.reset(bool(enabled))

    @classmethod
    def dump_timing_records(cls, output_path: str, extra_totals: Optional[Dict[str, float]] = None):
        return cls.timing_recorder.dump_csv(output_path, extra_totals=extra_totals)

    @classmethod
    def get_density_records(cls) -> Dict[int, Dict[int, float]]:
        return cls.density_records

    @classmethod
    def dump_density_records(cls, output_path: Optional[str] = None) -> Optional[str]:
        if not cls.density_records:
            return None
        if output_path is not None:
            os.makedirs(os.path.dirname(output_path) or ".", exist_ok=True)
            with open(output_path, "w") as f:
                f.write("step_idx,layer_idx,density\n")
                for step in sorted(cls.density_records):
                    for layer, d in sorted(cls.density_records[step].items()):
                        f.write(f"{step},{layer},{d}\n")
        return output_path

    @classmethod
    def get_cache_info(cls) -> Dict:
        return {
            "num_cached_steps": len(cls._cached_metadata),
            "cached_steps": list(cls._cached_metadata.keys()),
            "total_cached_layers": sum(len(v) for v in cls._cached_metadata.values()),
        }


def dfs_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, step_idx: int = 0, skip_steps: int = 12,
                  cache_interval: int = 12, layer_idx: int = 0, sparsity: float = 0.25,
                  sparsity_dcrt: float = 0.1, tile_size: int = 32, block_size: int = 128, video_len: int = 0,
                  video_perm: Optional[torch.Tensor] = None, cache_flag: bool = True,
                  record_density: bool = False, cu_seqlens_q=None, cu_seqlens_kv=None, max_seqlen_q=None,
                  max_seqlen_kv=None, sparse_execution: str = "native", hybrid_threshold: int = 8,
                  block_top_p: Optional[float] = None, token_top_k: int = 0, residual_candidate_blocks: int = 4,
                  selector_mode: str = "topk", fine_top_p: float = 0.9, prepermuted: bool = False,
                  token_major_out: bool = False, out_shards=None, out_head0: int = 0,
                  **unsupported) -> torch.Tensor:
    """q, k, v: [1, H, L, D] (raster video tokens, then text).  Returns [1, H, L, D].

    Keyword arguments of the reference's other back-ends (``flashinfer64_*``)
    are accepted for call compatibility and ignored, as they are by the
    reference's native branch.
    """
    for name in unsupported:
        if not name.startswith("flashinfer64_"):
            raise TypeError(f"dfs_attention() got an unexpected keyword argument {name!r}")
    _reject_unsupported(sparse_execution, selector_mode, block_top_p, token_top_k, block_size, tile_size,
                        fine_top_p, kp_allowed=True)
    inst = _dfs_attention_instances.get(layer_idx)
    if inst is None:
        inst = DFS_Attention(step_idx, layer_idx, sparsity, cache_flag, video_len, video_perm, block_size,
                             tile_size, tile_size, sparse_execution, hybrid_threshold, block_top_p, token_top_k,
                             residual_candidate_blocks, selector_mode, fine_top_p)
        _dfs_attention_instances[layer_idx] = inst
    inst.step_idx = step_idx
    is_cache_step, current = _compute_cache_schedule(step_idx, skip_steps, cache_interval, sparsity,
                                                     sparsity_dcrt)
    inst.sparse_ratio = current
    inst.cache_flag = cache_flag and is_cache_step
    inst.sparse_execution = sparse_execution
    inst.hybrid_threshold = hybrid_threshold
    inst.block_top_p = block_top_p
    inst.token_top_k = token_top_k
    inst.residual_candidate_blocks = residual_candidate_blocks
    inst.selector_mode = selector_mode
    inst.fine_top_p = fine_top_p
    if record_density and not DFS_Attention.record_density:
        DFS_Attention.set_record_density(True)
    return inst.forward(q=q, k=k, v=v, attn_mask=None, causal=False, drop_rate=0.0, cu_seqlens_q=cu_seqlens_q,
                        cu_seqlens_kv=cu_seqlens_kv, max_seqlen_q=max_seqlen_q, max_seqlen_kv=max_seqlen_kv,
                        batch_size=q.shape[0], prepermuted=prepermuted, token_major_out=token_major_out,
                        out_shards=out_shards, out_head0=out_head0)
