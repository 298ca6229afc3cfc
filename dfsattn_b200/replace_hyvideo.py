"""HunyuanVideo attention processor with B200 DFS sparse attention.

Drop-in for ``HunyuanVideo_DFSAttn_Processor2_0`` of
``dfsattn/replace_hyvideo.py:31-464``: same constructor argument order, same
``__call__`` signature and return arity, same dense/sparse gating per step and
layer (:314-325) and the same self-advancing step counter (:460-462).  The
``attn`` argument is a diffusers ``Attention`` module (or anything exposing the
same projections); diffusers itself is not imported.
"""
from typing import Optional

import torch

from . import fused_qkv
from .attention_hyvideo import DFS_Attention, dfs_attention
from .fullattention import full_attention


def apply_rotary_emb(x: torch.Tensor, freqs_cis) -> torch.Tensor:
    """Rotary embedding with real (cos, sin) tables of shape [S, D] on x [B, H, S, D];
    pairs are adjacent elements (the convention HunyuanVideo uses in diffusers)."""
    cos, sin = freqs_cis
    cos = cos[None, None].to(x.device)
    sin = sin[None, None].to(x.device)
    x_real, x_imag = x.reshape(*x.shape[:-1], -1, 2).unbind(-1)
    x_rot = torch.stack([-x_imag, x_real], dim=-1).flatten(3)
    return (x.float() * cos + x_rot.float() * sin).to(x.dtype)


class HunyuanVideo_DFSAttn_Processor2_0:
    def __init__(self, mode, sparsity, tile_size, block_size, video_len, video_perm, processor_id, skip_layers,
                 skip_steps, cache_interval, sparsity_dcrt, cache_flag, dense_interval=0, rest_steps=0,
                 skip_steps2=0, record_density=False, sparse_execution="native", hybrid_threshold=8,
                 block_top_p=None, token_top_k=0, residual_candidate_blocks=4, selector_mode="topk",
                 fine_top_p=0.9, **other_backend_knobs):
        if mode not in ("dfs", "flash"):
            raise ValueError(f"mode={mode!r}: the B200 build has 'dfs' and 'flash' (dense)")
        if mode == "dfs":
            if sparse_execution != "native":
                raise ValueError(f"sparse_execution={sparse_execution!r}: only 'native' is built for B200")
            if selector_mode not in ("topk", "kp") or block_top_p is not None or token_top_k:
                raise ValueError("the B200 build has the top-k block selector and its kp refinement "
                                 "(fine top-p inside the chosen blocks)")
            if block_size != 128 or tile_size not in (16, 32, 64):
                raise ValueError("block_size must be 128 and tile_size 16, 32 or 64")
            if selector_mode == "kp" and tile_size != 16:
                raise ValueError("kp mode requires 128x128 coarse blocks and 16x16 sub-blocks")
        for name in other_backend_knobs:
            if not (name.startswith("flashinfer64_") or name.startswith("attention_debug_")):
                raise TypeError(f"unexpected keyword argument {name!r}")
        self.mode = mode
        self.sparsity = sparsity
        self.tile_size = tile_size
        self.block_size = block_size
        self.video_len = video_len
        self.video_perm = video_perm
        self.step_idx = 0
        self.layer_idx = processor_id
        self.skip_layers = skip_layers
        self.skip_steps = skip_steps
        self.cache_interval = cache_interval
        self.sparsity_dcrt = sparsity_dcrt
        self.cache_flag = cache_flag
        self.dense_interval = dense_interval
        self.rest_steps = rest_steps
        self.skip_steps2 = skip_steps2
        self.record_density = record_density
        self.sparse_execution = sparse_execution
        self.hybrid_threshold = hybrid_threshold
        self.block_top_p = block_top_p
        self.token_top_k = token_top_k
        self.residual_candidate_blocks = residual_candidate_blocks
        self.selector_mode = selector_mode
        self.fine_top_p = fine_top_p
        self.num_inference_steps = 50  # the reference hard-codes the wrap-around (:461)

    def get_cu_max_seqlen(self, attention_mask, device):
        valid = int(attention_mask.sum())
        total = attention_mask.numel()
        cu = torch.tensor([0, valid, total], dtype=torch.int32)  # host copy: no second sync downstream
        return cu, cu, total, total

    def _is_sparse_call(self) -> bool:
        if self.mode != "dfs":
            return False
        phase_rest_end = self.skip_steps + self.rest_steps
        phase_sparse2_start = phase_rest_end + self.skip_steps2
        in_sparse = (self.skip_steps <= self.step_idx < phase_rest_end) or self.step_idx >= phase_sparse2_start
        periodic_dense = (self.dense_interval > 0 and self.step_idx >= self.skip_steps
                          and (self.step_idx - self.skip_steps + 1) % self.dense_interval == 0)
        return self.layer_idx not in self.skip_layers and in_sparse and not periodic_dense

    # One pass from the projections to permuted, normalised, rotated Q/K/V and a token-major
    # attention result (no transpose before the output projection).  Class-wide switch; calls the
    # fused kernel does not cover take the unfused path below.
    fused_prepare = True

    def _fused_qkv(self, attn, hidden_states, encoder_hidden_states, image_rotary_emb, single_stream):
        """(q, k, v [1,H,L,D] in permuted token order, perm) or None when the call is not eligible."""
        width = attn.to_q.out_features if hasattr(attn.to_q, "out_features") else None
        if width is None or not fused_qkv.eligible(hidden_states, attn.heads, width):
            return None
        heads = attn.heads
        double_stream = getattr(attn, "add_q_proj", None) is not None and encoder_hidden_states is not None
        n_main = hidden_states.shape[1]
        n_text = encoder_hidden_states.shape[1] if double_stream else 0
        seq_len = n_main + n_text
        text_in_main = encoder_hidden_states.shape[1] if single_stream else 0
        video_len = n_main - text_in_main                                 # rows that get the rotation
        perm_video_len = self.video_len if self.video_len else seq_len    # as the operator builds its permutation
        if perm_video_len > seq_len or (double_stream and perm_video_len > n_main):
            return None
        try:
            perm = fused_qkv.token_perm(self.video_perm, seq_len, perm_video_len, hidden_states.device) \
                if self.video_perm is not None else None
            main_perm = perm[:n_main] if (perm is not None and double_stream) else perm
            out = fused_qkv.prepare(attn.to_q(hidden_states), attn.to_k(hidden_states), attn.to_v(hidden_states),
                                    heads, getattr(attn, "norm_q", None), getattr(attn, "norm_k", None),
                                    image_rotary_emb, video_len, main_perm, out_row0=0, out_len=seq_len)
            if double_stream:
                fused_qkv.prepare(attn.add_q_proj(encoder_hidden_states), attn.add_k_proj(encoder_hidden_states),
                                  attn.add_v_proj(encoder_hidden_states), heads,
                                  getattr(attn, "norm_added_q", None), getattr(attn, "norm_added_k", None),
                                  None, 0, None, out=out, out_row0=n_main, out_len=seq_len)
        except TypeError:
            return None
        return tuple(t.unsqueeze(0) for t in out), perm

    def __call__(self, attn, hidden_states: torch.Tensor, encoder_hidden_states: Optional[torch.Tensor] = None,
                 attention_mask: Optional[torch.Tensor] = None, image_rotary_emb=None):
        single_stream = getattr(attn, "add_q_proj", None) is None and encoder_hidden_states is not None
        if single_stream:
            hidden_states = torch.cat([hidden_states, encoder_hidden_states], dim=1)

        fused = self._fused_qkv(attn, hidden_states, encoder_hidden_states, image_rotary_emb, single_stream) \
            if self.fused_prepare else None
        self.last_call_fused = fused is not None   # for tests and logs: which path this call took
        if fused is not None:
            (query, key, value), perm = fused
            return self._attend_and_project(attn, query, key, value, encoder_hidden_states, attention_mask,
                                            prepermuted=True, perm=perm)

        query = attn.to_q(hidden_states).unflatten(2, (attn.heads, -1)).transpose(1, 2).contiguous()
        key = attn.to_k(hidden_states).unflatten(2, (attn.heads, -1)).transpose(1, 2).contiguous()
        value = attn.to_v(hidden_states).unflatten(2, (attn.heads, -1)).transpose(1, 2).contiguous()
        if getattr(attn, "norm_q", None) is not None:
            query = attn.norm_q(query)
        if getattr(attn, "norm_k", None) is not None:
            key = attn.norm_k(key)

        if image_rotary_emb is not None:
            if single_stream:  # text is the last text_len tokens and is not rotated
                t = encoder_hidden_states.shape[1]
                query = torch.cat([apply_rotary_emb(query[:, :, :-t], image_rotary_emb), query[:, :, -t:]], dim=2)
                key = torch.cat([apply_rotary_emb(key[:, :, :-t], image_rotary_emb), key[:, :, -t:]], dim=2)
            else:
                query = apply_rotary_emb(query, image_rotary_emb)
                key = apply_rotary_emb(key, image_rotary_emb)

        if getattr(attn, "add_q_proj", None) is not None and encoder_hidden_states is not None:
            eq = attn.add_q_proj(encoder_hidden_states).unflatten(2, (attn.heads, -1)).transpose(1, 2)
            ek = attn.add_k_proj(encoder_hidden_states).unflatten(2, (attn.heads, -1)).transpose(1, 2)
            ev = attn.add_v_proj(encoder_hidden_states).unflatten(2, (attn.heads, -1)).transpose(1, 2)
            if getattr(attn, "norm_added_q", None) is not None:
                eq = attn.norm_added_q(eq)
            if getattr(attn, "norm_added_k", None) is not None:
                ek = attn.norm_added_k(ek)
            query = torch.cat([query, eq], dim=2)
            key = torch.cat([key, ek], dim=2)
            value = torch.cat([value, ev], dim=2)
        return self._attend_and_project(attn, query, key, value, encoder_hidden_states, attention_mask)

    def _attend_and_project(self, attn, query, key, value, encoder_hidden_states, attention_mask,
                            prepermuted: bool = False, perm=None):
        """Steps 5 and 6 of the reference processor (replace_hyvideo.py:314-464).  With
        ``prepermuted`` the inputs are in the permuted token order and the result comes back
        token-major, so the transpose below is a view."""
        if attention_mask is not None:
            cu_q, cu_kv, max_q, max_kv = self.get_cu_max_seqlen(attention_mask, query.device)
        else:
            cu_q = cu_kv = None
            max_q = max_kv = query.shape[2]

        rec = DFS_Attention.timing_recorder
        if self._is_sparse_call():
            hidden_states = dfs_attention(
                query, key, value, step_idx=self.step_idx, skip_steps=self.skip_steps,
                cache_interval=self.cache_interval, layer_idx=self.layer_idx, sparsity=self.sparsity,
                sparsity_dcrt=self.sparsity_dcrt, tile_size=self.tile_size, block_size=self.block_size,
                video_len=self.video_len, video_perm=self.video_perm, cache_flag=self.cache_flag,
                record_density=self.record_density, cu_seqlens_q=cu_q, cu_seqlens_kv=cu_kv,
                max_seqlen_q=max_q, max_seqlen_kv=max_kv, sparse_execution=self.sparse_execution,
                hybrid_threshold=self.hybrid_threshold, block_top_p=self.block_top_p,
                token_top_k=self.token_top_k, residual_candidate_blocks=self.residual_candidate_blocks,
                selector_mode=self.selector_mode, fine_top_p=self.fine_top_p, prepermuted=prepermuted,
                token_major_out=prepermuted)
        else:
            t0 = rec.start(query.device)
            hidden_states = full_attention(query, key, value, mode="flash", drop_rate=0.0, attn_mask=None,
                                           causal=False, cu_seqlens_q=cu_q, cu_seqlens_kv=cu_kv,
                                           max_seqlen_q=max_q, max_seqlen_kv=max_kv, batch_size=query.shape[0],
                                           out_row_map=perm if prepermuted else None,
                                           token_major_out=prepermuted)
            rec.stop(t0, phase="attention_execution", step_idx=self.step_idx, layer_idx=self.layer_idx,
                     device=query.device)

        hidden_states = hidden_states.transpose(1, 2).flatten(2, 3).to(query.dtype)
        if encoder_hidden_states is not None:
            t = encoder_hidden_states.shape[1]
            hidden_states, encoder_hidden_states = hidden_states[:, :-t], hidden_states[:, -t:]
            if getattr(attn, "to_out", None) is not None:
                hidden_states = attn.to_out[0](hidden_states)
                hidden_states = attn.to_out[1](hidden_states)
            if getattr(attn, "to_add_out", None) is not None:
                encoder_hidden_states = attn.to_add_out(encoder_hidden_states)

        self.step_idx += 1
        if self.step_idx == self.num_inference_steps:
            self.step_idx = 0
        return hidden_states, encoder_hidden_states
