"""Host logic shared by the HunyuanVideo and Wan DFS attention operators.

Device-resident pieces built once and reused: the int32 permutation and its
inverse (the reference rebuilds and re-uploads them on every call,
dfsattn/attention_hyvideo.py:1116-1120), the scoring workspace, and the
per-layer block index lists (the reference caches bool masks,
attention_hyvideo.py:1165-1183).
"""
import math
from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch

from . import ops

BLOCK = ops.BLOCK


@dataclass
class BlockLists:
    """Selected key blocks per (head, query block): ascending lists."""
    idx: torch.Tensor  # int32 [H, Qb, kmax], -1 padded
    cnt: torch.Tensor  # int32 [H, Qb]; -1 = the row attends every key block (nothing listed)
    k_blocks: int
    # "kp" selector only: int64 [H, Qb, kmax], per list entry the 8 x 8 map of attended 16 x 16-token
    # tiles (bit 8 * query tile + key tile); None = whole blocks
    fine: Optional[torch.Tensor] = None

    def clone(self) -> "BlockLists":
        return BlockLists(self.idx.clone(), self.cnt.clone(), self.k_blocks,
                          None if self.fine is None else self.fine.clone())

    def fine_pair_count(self, seq_len: int) -> int:
        """Attended (q, k) token pairs under the tile maps, partial last blocks included, without
        building the 16 x 16 mask: an all-ones map is a whole block (counted with its true row and
        column sizes), any other map belongs to a pair of full 128-token blocks (refined pairs lie
        before the boundary block) and counts 256 pairs per set bit."""
        if self.fine is None:
            raise ValueError("no tile maps")
        H, Qb, kmax = self.idx.shape
        dev = self.idx.device
        valid = self.idx >= 0
        whole = valid & (self.fine == -1)
        size = torch.full((self.k_blocks + 1,), BLOCK, dtype=torch.int64, device=dev)
        size[self.k_blocks - 1] = seq_len - BLOCK * (self.k_blocks - 1)
        size[self.k_blocks] = 0
        cols = size[torch.where(valid, self.idx, torch.full_like(self.idx, self.k_blocks)).long()]
        per_row = torch.where(self.cnt < 0, torch.full_like(self.cnt, seq_len, dtype=torch.int64),
                              (cols * whole).sum(-1))
        pairs = int((size[None, :Qb] * per_row).sum().item())
        lut = torch.tensor([bin(i).count("1") for i in range(256)], dtype=torch.int64, device=dev)
        part = (valid & ~whole)[..., None].expand(-1, -1, -1, 8)
        set_bits = int((lut[self.fine.view(torch.uint8).view(H, Qb, kmax, 8).long()] * part).sum().item())
        return pairs + 256 * set_bits

    def to_fine_mask(self, seq_len: int) -> torch.Tensor:
        """bool [H, ceil(L/16), ceil(L/16)]: the reference's fine mask format
        (dfsattn/attention_hyvideo.py:236-241), for inspection and tests."""
        H, Qb, kmax = self.idx.shape
        if self.fine is None:
            full = self.to_bool_mask().repeat_interleave(8, 1).repeat_interleave(8, 2)
        else:
            shifts = torch.arange(64, device=self.idx.device, dtype=torch.int64)
            tiles = ((self.fine[..., None] >> shifts) & 1).bool().view(H, Qb, kmax, 8, 8)
            tiles = tiles & (self.idx >= 0)[..., None, None]
            dense = torch.zeros((H, Qb, self.k_blocks + 1, 8, 8), dtype=torch.bool, device=self.idx.device)
            safe = torch.where(self.idx >= 0, self.idx, torch.full_like(self.idx, self.k_blocks)).long()
            dense.scatter_(2, safe[..., None, None].expand(-1, -1, -1, 8, 8), tiles)
            full = dense[:, :, : self.k_blocks].permute(0, 1, 3, 2, 4).reshape(H, Qb * 8, self.k_blocks * 8)
        full = full | (self.cnt < 0).repeat_interleave(8, 1)[..., None]
        nf = math.ceil(seq_len / 16)
        return full[:, :nf, :nf]

    def to_bool_mask(self) -> torch.Tensor:
        """bool [H, Qb, Kb] (the reference's mask format)."""
        H, Qb, kmax = self.idx.shape
        mask = torch.zeros((H, Qb, self.k_blocks + 1), dtype=torch.bool, device=self.idx.device)
        safe = torch.where(self.idx >= 0, self.idx, torch.full_like(self.idx, self.k_blocks)).long()
        mask.scatter_(-1, safe, True)
        return mask[..., : self.k_blocks] | (self.cnt < 0)[..., None]

    @staticmethod
    def from_bool_mask(mask: torch.Tensor) -> "BlockLists":
        H, Qb, Kb = mask.shape
        cnt = mask.sum(dim=-1).to(torch.int32)
        kmax = max(int(cnt.max().item()), 1)
        order = torch.argsort((~mask).to(torch.int8), dim=-1, stable=True)[..., :kmax].to(torch.int32)
        pos = torch.arange(kmax, device=mask.device)[None, None, :]
        idx = torch.where(pos < cnt[..., None], order, torch.full_like(order, -1))
        return BlockLists(idx.contiguous(), cnt.contiguous(), Kb)


class PermutationCache:
    """int32 (perm, inverse) on the device per (permutation, lengths, device).

    An entry is found by the identity of the ``video_perm`` tensor (and its version counter); the
    entry holds a reference to that tensor, so its address cannot be handed to another permutation
    while the entry lives.  A tensor that is not known by identity is compared by CONTENT with the
    cached ones of the same length before anything is rebuilt (a caller that builds an equal
    permutation anew for every call still hits).  At most ``max_entries`` entries are kept."""

    def __init__(self, max_entries: int = 16):
        self._cache: Dict[tuple, tuple] = {}
        self.max_entries = max_entries

    def get(self, video_perm: Optional[torch.Tensor], seq_len: int, video_len: int,
            device: torch.device) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor]]:
        if video_perm is None:
            return None, None  # raster order: no gather at all
        shape_key = (int(video_perm.numel()), seq_len, video_len, str(device))
        key = (id(video_perm), int(video_perm._version)) + shape_key
        hit = self._cache.get(key)
        if hit is not None and hit[0] is video_perm:
            return hit[1], hit[2]
        for other_key, (src, perm, inv) in list(self._cache.items()):
            if other_key[2:] == shape_key and src.device == video_perm.device and src.dtype == video_perm.dtype \
                    and src._version == other_key[1] and torch.equal(src, video_perm):
                self._store(key, (video_perm, perm, inv))
                return perm, inv
        if video_perm.numel() != video_len:
            raise ValueError(f"video_perm has {video_perm.numel()} entries, expected video_len={video_len}")
        if seq_len >= 2 ** 31:
            raise ValueError("sequence too long for int32 token indices")
        vp = video_perm.to(device=device, dtype=torch.int64)
        if seq_len > video_len:  # text tokens stay in place at the tail
            perm = torch.cat([vp, torch.arange(video_len, seq_len, device=device, dtype=torch.int64)])
        else:
            perm = vp
        inv = torch.empty_like(perm)
        inv[perm] = torch.arange(seq_len, device=device, dtype=torch.int64)
        out = (perm.to(torch.int32).contiguous(), inv.to(torch.int32).contiguous())
        self._store(key, (video_perm,) + out)
        return out

    def _store(self, key, entry):
        while len(self._cache) >= self.max_entries:
            self._cache.pop(next(iter(self._cache)))
        self._cache[key] = entry

    def clear(self):
        self._cache.clear()


_perm_cache = PermutationCache()
_workspaces: Dict[str, torch.Tensor] = {}


def _workspace(device, nbytes: int) -> torch.Tensor:
    key = str(device)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(nbytes, dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def clear_device_caches():
    _perm_cache.clear()
    _workspaces.clear()


def topk_block_num(sparsity: float, k_blocks: int) -> int:
    """max(1, int(s * Kb)) in float64, as dfsattn/attention_hyvideo.py:432."""
    return max(1, int(float(sparsity) * k_blocks))


def list_budget(seq_len: int, video_len: int, sparsity: float, flavor: str, kp: bool = False):
    """(n_rank, k_select, dense_row_start) of a selection under the reference's budget rules.

    flavor "hyvideo": dfsattn/attention_hyvideo.py:424-443,491-501 (text and
    boundary key blocks use up budget and are always on; rows from the first
    block holding a text token on are dense).  flavor "wan":
    dfsattn/attention_wan.py:248-253 (plain top-k over every key block).
    """
    kb = math.ceil(seq_len / BLOCK)
    kk = topk_block_num(sparsity, kb)
    if flavor == "wan":
        return kb, kk, kb
    dense_start = video_len // BLOCK
    n_text_blocks = max(0, kb - dense_start)
    text_len = seq_len - video_len
    if n_text_blocks > 0:
        n_sel = kk - n_text_blocks
        if n_sel <= 0:
            raise AssertionError("num_video_blocks_to_select must be non-negative")
        n_rank = dense_start
    else:
        n_sel, n_rank = kk, kb
    # the kp selector keeps every row from the boundary block on dense, text or not (:298-301)
    dense_row_start = dense_start if (text_len > 0 or (kp and n_text_blocks > 0)) else kb
    return n_rank, n_sel, dense_row_start


def select_lists(scores: torch.Tensor, seq_len: int, video_len: int, sparsity: float,
                 flavor: str, want_mask: bool = False, kp: bool = False):
    """Index lists from fp32 block scores with the budget of ``list_budget``."""
    n_rank, n_sel, dense_row_start = list_budget(seq_len, video_len, sparsity, flavor, kp)
    return ops.select_topk(scores, q_rows=math.ceil(seq_len / BLOCK), n_rank=n_rank, k_select=n_sel,
                           dense_row_start=dense_row_start, want_mask=want_mask)


def compute_block_lists(q_perm, k_perm, video_len: int, sparsity: float, flavor: str,
                        tile: int = ops.TILE, fine_top_p: Optional[float] = None) -> BlockLists:
    """Scores + selection on permuted [H, L, D] tensors -> BlockLists.  With ``fine_top_p`` (the
    "kp" selector, HunyuanVideo flavour, 16-token tiles) the lists also carry the tile maps of
    ``ops.fine_top_p``; a value >= 1 keeps whole blocks, as the reference does
    (dfsattn/attention_hyvideo.py:266-281)."""
    H, L, D = q_perm.shape
    wan = flavor == "wan"
    kp = fine_top_p is not None
    if kp and (wan or tile != 16):
        raise ValueError("kp mode requires the HunyuanVideo operator, 128x128 coarse blocks and 16x16 sub-blocks")
    need = ops.lib.dfs_score_workspace_bytes(H, L, L if wan else video_len, D, tile, BLOCK, int(wan))
    if need < 0:
        ops.check(int(need), "dfs_score_workspace_bytes")
    ws = _workspace(q_perm.device, int(need))
    scores = ops.block_scores(q_perm, k_perm, L if wan else video_len, wan, tile=tile, workspace=ws)
    idx, cnt, _ = select_lists(scores, L, L if wan else video_len, sparsity, flavor, kp=kp)
    fine = None
    if kp and fine_top_p < 1.0:
        dense_start = video_len // BLOCK
        fine = ops.fine_top_p(ws, H, L, video_len, D, False, idx, cnt, n_rank=dense_start,
                              dense_row_start=dense_start, top_p=fine_top_p, tile=tile)
    return BlockLists(idx, cnt, math.ceil(L / BLOCK), fine)


def _as_heads(x: torch.Tensor) -> torch.Tensor:
    if x.dim() != 4 or x.shape[0] != 1:
        raise AssertionError("DFS Attention with block sparse currently supports batch size 1.")
    return x[0]


def prepare_inputs(q, k, v):
    """[1,H,L,D] (any float dtype, CUDA) -> contiguous bf16 [H,L,D] views/copies."""
    outs = []
    for t in (q, k, v):
        t = _as_heads(t)
        if not t.is_cuda:
            raise ValueError("dfsattn_b200 runs on CUDA tensors only (no CPU fallback)")
        if t.dtype != torch.bfloat16:
            t = t.to(torch.bfloat16)
        outs.append(t.contiguous())
    return outs


def valid_length(cu_seqlens, seq_len: int) -> int:
    """End of the first varlen segment from cu_seqlens = [0, valid, L]
    (dfsattn/replace_hyvideo.py:221-228); None means one segment."""
    if cu_seqlens is None:
        return seq_len
    vals = cu_seqlens.tolist() if isinstance(cu_seqlens, torch.Tensor) else list(cu_seqlens)
    if len(vals) < 2:
        return seq_len
    valid = int(vals[1])
    return seq_len if valid <= 0 or valid > seq_len else valid


def run_attention(qp, kp, vp, lists: Optional[BlockLists], perm_i32, valid_len: int,
                  token_major: bool = False, out_shards=None, out_head0: int = 0) -> torch.Tensor:
    """Block-sparse (or dense when ``lists`` is None) attention on permuted
    bf16 [H,L,D]; returns the un-permuted result, [H,L,D] or, with
    ``token_major``, [L,H,D] (what the output projection reads).

    A padded tail [valid_len, L) forms a second, independent varlen segment
    whose block coordinates restart at zero (block_sparse_attn semantics,
    dfsattn/attention_hyvideo.py:1055,1075-1082); it is a second launch on the
    tail rows with the top-left corner of the same block mask.
    """
    H, L, D = qp.shape
    idx = lists.idx if lists is not None else None
    cnt = lists.cnt if lists is not None else None
    fine = lists.fine if lists is not None else None
    if fine is not None and (out_shards is not None or valid_len < L):
        raise ValueError("tile maps (kp selector) are not combined with sharded output or a padded tail")
    if out_shards is not None:
        # the result is scattered to sequence shards on several GPUs (ops.ShardTable); no local copy
        if valid_len < L:
            raise ValueError("a padded tail is not supported together with sharded output")
        return ops.block_sparse_fwd(qp, kp, vp, idx, cnt, out_row_map=perm_i32, kv_len=valid_len,
                                    out_shards=out_shards, out_head0=out_head0)
    out = ops.block_sparse_fwd(qp, kp, vp, idx, cnt, out_row_map=perm_i32, kv_len=valid_len,
                               token_major=token_major, fine=fine)
    if valid_len < L:
        tail = L - valid_len
        if perm_i32 is not None and not bool((perm_i32[valid_len:] == torch.arange(
                valid_len, L, device=qp.device, dtype=torch.int32)).all()):
            raise ValueError("the padded tail must lie in the un-permuted (text) part of the sequence")
        q2, k2, v2 = (t[:, valid_len:].contiguous() for t in (qp, kp, vp))
        lists2 = None
        if lists is not None:
            nb2 = math.ceil(tail / BLOCK)
            lists2 = BlockLists.from_bool_mask(lists.to_bool_mask()[:, :nb2, :nb2].contiguous())
        o2 = ops.block_sparse_fwd(q2, k2, v2, None if lists2 is None else lists2.idx,
                                  None if lists2 is None else lists2.cnt, kv_len=tail)
        if token_major:
            out[valid_len:] = o2.permute(1, 0, 2)
        else:
            out[:, valid_len:] = o2
    return out


def as_reference_layout(out: torch.Tensor, token_major: bool) -> torch.Tensor:
    """[H,L,D] or token-major [L,H,D] -> the operator's result shape [1,H,L,D].  For a
    token-major buffer this is a view whose ``transpose(1, 2).flatten(2, 3)`` (what the
    processors do next) is again a view: no copy between attention and output projection."""
    return (out.permute(1, 0, 2) if token_major else out).unsqueeze(0)
