"""Wan2.1 attention processor with B200 DFS sparse attention.

Drop-in for ``Wan_DFSAttn_Processor2_0`` of ``dfsattn/replace_wan.py:79-324``:
same constructor argument order and ``__call__`` signature.  Self-attention
(``cross_flag=False``) runs sparse when the gate (:252-301) says so; the call
counter advances twice per denoising step (classifier-free guidance) and wraps
at 100 (:320-323).  Cross-attention (``cross_flag=True``) is always dense and
uses PyTorch SDPA because its key length differs from its query length.

One addition: a self-attention call with a batch of TWO is taken as both
guidance passes of one denoising step (conditional first), counts as two calls
and runs as one gather and one attention launch with shared index lists
(``attention_wan.dfs_attention_cfg_pair``); the reference's operator refuses a
batch (dfsattn/attention_wan.py:219), so its callers run the passes one by one.
"""
from typing import Optional

import torch
import torch.nn.functional as F

from . import fused_qkv
from .attention_wan import dfs_attention, dfs_attention_cfg_pair
from .fullattention import full_attention


def apply_rotary_emb_complex(x: torch.Tensor, freqs: torch.Tensor) -> torch.Tensor:
    """x [B,H,S,D] rotated by complex frequencies [1,1,S,D/2] (replace_wan.py:211-215)."""
    xc = torch.view_as_complex(x.to(torch.float64).unflatten(3, (-1, 2)))
    return torch.view_as_real(xc * freqs).flatten(3, 4).type_as(x)


class Wan_DFSAttn_Processor2_0:
    def __init__(self, mode, sparsity, tile_size, block_size, video_perm, processor_id, skip_layers, skip_steps,
                 cache_interval, sparsity_dcrt, cache_flag, cross_flag, dense_step_idx=-1, dense_interval=0,
                 rest_steps=0, skip_steps2=0, record_density=False, sparse_execution="native",
                 hybrid_threshold=8, **other_backend_knobs):
        if mode not in ("dfs", "flash"):
            raise ValueError(f"mode={mode!r}: the B200 build has 'dfs' and 'flash' (dense)")
        if mode == "dfs" and not cross_flag:
            if sparse_execution != "native":
                raise ValueError(f"sparse_execution={sparse_execution!r}: only 'native' is built for B200")
            if block_size != 128 or tile_size not in (16, 32, 64):
                raise ValueError("block_size must be 128 and tile_size 16, 32 or 64")
        for name in other_backend_knobs:
            if not name.startswith("flashinfer64_"):
                raise TypeError(f"unexpected keyword argument {name!r}")
        self.mode = mode
        self.sparsity = sparsity
        self.tile_size = tile_size
        self.block_size = block_size
        self.video_perm = video_perm
        self.step_idx = 0
        self.layer_idx = processor_id
        self.skip_layers = skip_layers
        self.skip_steps = skip_steps
        self.cache_interval = cache_interval
        self.sparsity_dcrt = sparsity_dcrt
        self.cache_flag = cache_flag
        self.cross_flag = cross_flag
        self.dense_step_idx = dense_step_idx
        self.dense_interval = dense_interval
        self.rest_steps = rest_steps
        self.skip_steps2 = skip_steps2
        self.record_density = record_density
        self.sparse_execution = sparse_execution
        self.hybrid_threshold = hybrid_threshold
        self.num_inference_steps = 50

    def _gate(self) -> str:
        """'sparse' or 'dense' for this call (replace_wan.py:252-301)."""
        if self.mode != "dfs" or self.cross_flag:
            return "dense"
        real_step = self.step_idx // 2
        phase_rest_end = self.skip_steps + self.rest_steps
        in_sparse = (self.skip_steps <= real_step < phase_rest_end) or \
            real_step >= phase_rest_end + self.skip_steps2
        periodic_dense = (self.dense_interval > 0 and real_step >= self.skip_steps
                          and (real_step - self.skip_steps + 1) % self.dense_interval == 0)
        if self.step_idx == self.dense_step_idx or periodic_dense:
            return "dense"
        if self.layer_idx not in self.skip_layers and in_sparse:
            return "sparse"
        return "dense"

    def _advance(self, calls: int = 1) -> None:
        for _ in range(calls):
            self.step_idx += 1
            if self.step_idx == self.num_inference_steps * 2:
                self.step_idx = 0

    def _dfs_kwargs(self, S_q: int, S_k: int) -> dict:
        return dict(skip_steps=self.skip_steps, cache_interval=self.cache_interval, layer_idx=self.layer_idx,
                    sparsity=self.sparsity, sparsity_dcrt=self.sparsity_dcrt, tile_size=self.tile_size,
                    block_size=self.block_size, video_perm=self.video_perm, cache_flag=self.cache_flag,
                    record_density=self.record_density, max_seqlen_q=S_q, max_seqlen_kv=S_k,
                    sparse_execution=self.sparse_execution, hybrid_threshold=self.hybrid_threshold)

    # A batch of two sparse guidance passes as one gather + one attention launch (True), or as two
    # operator calls one after the other (False); the results are the same bits either way.
    cfg_pair_batch = True

    def _attend_self(self, query, key, value, perm=None, fused: bool = False):
        """Self-attention of one pass ([1, H, S, D]) or of both guidance passes ([2, H, S, D]) per the
        gate; advances the call counter by the batch.  ``fused``: inputs are already in the permuted
        token order ``perm`` and the result is wanted token-major."""
        B, _, S, _ = query.shape
        extra = dict(prepermuted=True, token_major_out=True) if fused else {}
        if B == 2:
            if self.step_idx % 2:
                raise ValueError("a batch of two guidance passes must start at an even call counter")
            first = self._gate()
            self.step_idx += 1
            second = self._gate()
            self.step_idx -= 1
            if self.cfg_pair_batch and first == second == "sparse":
                out = dfs_attention_cfg_pair(query, key, value, step_idx=self.step_idx,
                                             **self._dfs_kwargs(S, S), **extra)
                self._advance(2)
                return out
        elif B != 1:
            raise AssertionError("DFS Attention with block sparse currently supports batch size 1 "
                                 "(or 2: the guidance pair).")
        outs = []
        for b in range(B):
            qb, kb, vb = (t[b:b + 1] for t in (query, key, value))
            if self._gate() == "sparse":
                outs.append(dfs_attention(qb, kb, vb, step_idx=self.step_idx, **self._dfs_kwargs(S, S), **extra))
            elif fused:
                outs.append(full_attention(qb, kb, vb, mode="flash", max_seqlen_q=S, max_seqlen_kv=S,
                                           batch_size=1, out_row_map=perm, token_major_out=True))
            else:
                outs.append(full_attention(qb, kb, vb, mode="flash", max_seqlen_q=S, max_seqlen_kv=S,
                                           batch_size=1))
            self._advance()
        return outs[0] if B == 1 else torch.cat(outs, dim=0)

    # One pass from the projections to permuted, normalised, rotated Q/K/V and a token-major
    # attention result; class-wide switch, self-attention only (cross-attention is not on the path).
    fused_prepare = True

    def _fused_self_attention(self, attn, hidden_states, rotary_emb):
        width = getattr(attn.to_q, "out_features", None)
        if width is None or not fused_qkv.eligible(hidden_states, attn.heads, width, max_batch=2):
            return None
        B, S = hidden_states.shape[0], hidden_states.shape[1]
        try:
            perm = fused_qkv.token_perm(self.video_perm, S, S, hidden_states.device) \
                if self.video_perm is not None else None
            pq, pk, pv = attn.to_q(hidden_states), attn.to_k(hidden_states), attn.to_v(hidden_states)
            H, D = attn.heads, width // attn.heads
            out = tuple(torch.empty((B * H, S, D), dtype=torch.bfloat16, device=hidden_states.device)
                        for _ in range(3))
            for b in range(B):   # one pass per batch element, each filling its heads of the shared buffers
                fused_qkv.prepare(pq[b], pk[b], pv[b], H, getattr(attn, "norm_q", None),
                                  getattr(attn, "norm_k", None), rotary_emb, S, perm,
                                  out=tuple(t[b * H:(b + 1) * H] for t in out))
        except TypeError:
            return None
        query, key, value = (t.view(B, H, S, D) for t in out)
        hidden_states = self._attend_self(query, key, value, perm=perm, fused=True)
        hidden_states = hidden_states.transpose(1, 2).flatten(2, 3).type_as(query)  # a view
        hidden_states = attn.to_out[0](hidden_states)
        hidden_states = attn.to_out[1](hidden_states)
        return hidden_states

    def __call__(self, attn, hidden_states: torch.Tensor, encoder_hidden_states: Optional[torch.Tensor] = None,
                 attention_mask: Optional[torch.Tensor] = None, rotary_emb: Optional[torch.Tensor] = None):
        encoder_hidden_states_img = None
        if getattr(attn, "add_k_proj", None) is not None:
            image_context_length = encoder_hidden_states.shape[1] - 512
            encoder_hidden_states_img = encoder_hidden_states[:, :image_context_length]
            encoder_hidden_states = encoder_hidden_states[:, image_context_length:]
        self_attention = encoder_hidden_states is None
        if encoder_hidden_states is None:
            encoder_hidden_states = hidden_states

        self.last_call_fused = False   # for tests and logs: which path this call took
        if self.fused_prepare and self_attention and attention_mask is None:
            fused = self._fused_self_attention(attn, hidden_states, rotary_emb)
            if fused is not None:
                self.last_call_fused = True
                return fused

        query = attn.to_q(hidden_states)
        key = attn.to_k(encoder_hidden_states)
        value = attn.to_v(encoder_hidden_states)
        if getattr(attn, "norm_q", None) is not None:
            query = attn.norm_q(query)
        if getattr(attn, "norm_k", None) is not None:
            key = attn.norm_k(key)
        query = query.unflatten(2, (attn.heads, -1)).transpose(1, 2).contiguous()
        key = key.unflatten(2, (attn.heads, -1)).transpose(1, 2).contiguous()
        value = value.unflatten(2, (attn.heads, -1)).transpose(1, 2).contiguous()
        if rotary_emb is not None:
            query = apply_rotary_emb_complex(query, rotary_emb)
            key = apply_rotary_emb_complex(key, rotary_emb)

        hidden_states_img = None
        if encoder_hidden_states_img is not None:
            key_img = attn.add_k_proj(encoder_hidden_states_img)
            value_img = attn.add_v_proj(encoder_hidden_states_img)
            if getattr(attn, "norm_added_k", None) is not None:
                key_img = attn.norm_added_k(key_img)
            key_img = key_img.unflatten(2, (attn.heads, -1)).transpose(1, 2)
            value_img = value_img.unflatten(2, (attn.heads, -1)).transpose(1, 2)
            hidden_states_img = F.scaled_dot_product_attention(query, key_img, value_img)
            hidden_states_img = hidden_states_img.transpose(1, 2).flatten(2, 3).type_as(query)

        S_q, S_k = query.shape[2], key.shape[2]
        if self_attention and attention_mask is None:
            hidden_states = self._attend_self(query, key, value)   # advances the counter
            counted = True
        else:
            counted = False
            gate = self._gate()
            if gate == "sparse":
                hidden_states = dfs_attention(query, key, value, step_idx=self.step_idx,
                                              **self._dfs_kwargs(S_q, S_k))
            elif S_q == S_k and attention_mask is None:
                hidden_states = full_attention(query, key, value, mode="flash", max_seqlen_q=S_q,
                                               max_seqlen_kv=S_k, batch_size=query.shape[0])
            else:  # cross-attention: different key length, not part of the DFS path
                hidden_states = F.scaled_dot_product_attention(query, key, value)

        hidden_states = hidden_states.transpose(1, 2).flatten(2, 3).type_as(query)
        if hidden_states_img is not None:
            hidden_states = hidden_states + hidden_states_img
        hidden_states = attn.to_out[0](hidden_states)
        hidden_states = attn.to_out[1](hidden_states)
        if not counted:
            self._advance()
        return hidden_states
