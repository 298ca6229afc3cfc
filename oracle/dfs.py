"""Oracle: schedule, scoring, selection and block-sparse attention.

TEST INFRASTRUCTURE ONLY -- a PyTorch-CPU restatement of the reference's
native DFS attention path.  Each function cites the reference lines it follows
(paths relative to the reference repository).  Pinned against the reference's
own functions run on CPU (``tests/golden``) and its schedule table
(``tests/test_flashinfer64_attention.py:122-144``).
"""

import math

import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------- #
# schedule
# --------------------------------------------------------------------------- #
def compute_cache_schedule(step_idx, skip_steps, cache_interval, sparsity, sparsity_dcrt):
    """(is_cache_step, current_sparsity); dfsattn/attention_hyvideo.py:40-65."""
    if cache_interval <= 0:
        raise ValueError("cache_interval must be greater than 0.")
    if step_idx < skip_steps:
        return False, sparsity
    raw = (step_idx - skip_steps) // cache_interval
    if sparsity_dcrt > 0:
        max_valid = max(0, math.ceil(sparsity / sparsity_dcrt) - 1)
    else:
        max_valid = raw
    idx = min(raw, max_valid)
    is_cache_step = raw <= max_valid and (step_idx - skip_steps) % cache_interval == 0
    current = sparsity - idx * sparsity_dcrt
    current = min(1.0, max(0.0, current))
    return is_cache_step, current


# --------------------------------------------------------------------------- #
# permutation
# --------------------------------------------------------------------------- #
def build_permutation(video_perm, seq_len, video_len=None):
    """Full-length permutation and its inverse (int64 tensors).

    dfsattn/attention_hyvideo.py:154-174 (text tokens keep their place at the
    tail) and dfsattn/attention_wan.py:113-125 (video only).  ``video_perm``
    None means raster order (identity).
    """
    if video_perm is None:
        ident = torch.arange(seq_len, dtype=torch.long)
        return ident, ident.clone()
    video_perm = torch.as_tensor(video_perm, dtype=torch.long)
    if video_len is None:
        video_len = video_perm.numel()
    if seq_len > video_len:
        perm = torch.cat([video_perm, torch.arange(video_len, seq_len, dtype=torch.long)])
    else:
        perm = video_perm
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(perm.numel(), dtype=torch.long)
    return perm, inv


# --------------------------------------------------------------------------- #
# scoring
# --------------------------------------------------------------------------- #
def _pool(x, tile):
    b, h, n, d = x.shape
    return x.view(b, h, n // tile, tile, d).mean(dim=3)


def tile_score_hyvideo(q, k, perm, video_len, tile=16, block=128):
    """Softmax-ed pooled tile scores [1,H,Vb*block/tile,Kb*block/tile].

    dfsattn/attention_hyvideo.py:310-385: gather by perm; video part zero-padded
    to a block multiple *between* video and text (:331-351); whole sequence
    zero-padded to Kb*block at the end (:356-365); mean over each tile with the
    zero rows included (:372-381); softmax over all key tiles (:383).
    """
    b, h, L, d = q.shape
    scale = 1.0 / math.sqrt(d)
    text_len = L - video_len
    vb = math.ceil(video_len / block)
    kb = math.ceil(L / block)
    qp = q[:, :, perm, :]
    kp = k[:, :, perm, :]
    vpad = vb * block - video_len
    if vpad > 0:
        zq = torch.zeros((b, h, vpad, d), dtype=q.dtype)
        parts_q = [qp[:, :, :video_len], zq]
        parts_k = [kp[:, :, :video_len], zq.clone()]
        if text_len > 0:
            parts_q.append(qp[:, :, video_len:])
            parts_k.append(kp[:, :, video_len:])
        qp = torch.cat(parts_q, dim=2)
        kp = torch.cat(parts_k, dim=2)
    if qp.shape[2] < kb * block:
        qp = F.pad(qp, (0, 0, 0, kb * block - qp.shape[2]))
    if kp.shape[2] < kb * block:
        kp = F.pad(kp, (0, 0, 0, kb * block - kp.shape[2]))
    qm = _pool(qp[:, :, : vb * block].contiguous(), tile)
    km = _pool(kp.contiguous(), tile)
    return (qm @ km.transpose(-2, -1) * scale).softmax(dim=-1)


def tile_score_wan(q, k, perm, tile=16, block=128):
    """dfsattn/attention_wan.py:157-209: zero pad only at the end; Q and K both
    cover every tile."""
    b, h, L, d = q.shape
    scale = 1.0 / math.sqrt(d)
    kb = math.ceil(L / block)
    qp = q[:, :, perm, :]
    kp = k[:, :, perm, :]
    pad = kb * block - L
    if pad > 0:
        qp = F.pad(qp, (0, 0, 0, pad))
        kp = F.pad(kp, (0, 0, 0, pad))
    qm = _pool(qp.contiguous(), tile)
    km = _pool(kp.contiguous(), tile)
    return (qm @ km.transpose(-2, -1) * scale).softmax(dim=-1)


def _block_sums(score, rows, cols, tpb):
    h = score.shape[1]
    return score.view(1, h, rows, tpb, cols, tpb).sum(dim=(3, 5))


def block_scores_hyvideo(q, k, perm, video_len, tile=16, block=128):
    """Block score sums [1,H,Vb,Kb]; dfsattn/attention_hyvideo.py:419-422."""
    L = q.shape[2]
    s = tile_score_hyvideo(q, k, perm, video_len, tile, block)
    return _block_sums(s, math.ceil(video_len / block), math.ceil(L / block), block // tile)


def block_scores_wan(q, k, perm, tile=16, block=128):
    """Block score sums [1,H,Kb,Kb]; dfsattn/attention_wan.py:243-246."""
    L = q.shape[2]
    kb = math.ceil(L / block)
    s = tile_score_wan(q, k, perm, tile, block)
    return _block_sums(s, kb, kb, block // tile)


# --------------------------------------------------------------------------- #
# selection
# --------------------------------------------------------------------------- #
def select_hyvideo(block_sums, seq_len, video_len, sparsity, block=128):
    """bool mask [H,Kb,Kb] from block sums; dfsattn/attention_hyvideo.py:424-443,
    491-501,517.  Text / boundary key blocks use up part of the budget (:433-436)
    and are forced on for every row (:493-494); rows from the first block that
    holds a text token on are fully dense (:500-501)."""
    h = block_sums.shape[1]
    kb = math.ceil(seq_len / block)
    vb = math.ceil(video_len / block)
    text_len = seq_len - video_len
    dense_start = video_len // block
    n_text_blocks = max(0, kb - dense_start)
    video_mask = torch.zeros((1, h, vb, kb), dtype=torch.bool)
    kk = max(1, int(sparsity * kb))
    if n_text_blocks > 0:
        n_sel = kk - n_text_blocks
        if n_sel <= 0:
            raise AssertionError("num_video_blocks_to_select must be non-negative")
        _, top = torch.topk(block_sums[:, :, :, :dense_start], k=n_sel, dim=-1)
        video_mask.scatter_(-1, top, True)
        video_mask[..., dense_start:] = True
    else:
        _, top = torch.topk(block_sums, k=kk, dim=-1)
        video_mask.scatter_(-1, top, True)
    mask = torch.zeros((1, h, kb, kb), dtype=torch.bool)
    mask[:, :, :vb, :] = video_mask
    if text_len > 0:
        mask[:, :, dense_start:, :] = True
    return mask[0]


def select_wan(block_sums, seq_len, sparsity, block=128):
    """dfsattn/attention_wan.py:248-255: plain top-k over all key blocks."""
    kb = math.ceil(seq_len / block)
    kk = max(1, int(sparsity * kb))
    _, top = torch.topk(block_sums, k=kk, dim=-1)
    mask = torch.zeros(block_sums.shape, dtype=torch.bool)
    mask.scatter_(-1, top, True)
    return mask[0]


def block_mask_hyvideo(q, k, perm, video_len, sparsity, tile=16, block=128):
    """dfsattn/attention_hyvideo.py:388-519 (top-k branch)."""
    sums = block_scores_hyvideo(q, k, perm, video_len, tile, block)
    return select_hyvideo(sums, q.shape[2], video_len, sparsity, block)


def block_mask_wan(q, k, perm, sparsity, tile=16, block=128):
    """dfsattn/attention_wan.py:212-261."""
    sums = block_scores_wan(q, k, perm, tile, block)
    return select_wan(sums, q.shape[2], sparsity, block)


def fine_mask_hyvideo(q, k, perm, video_len, sparsity, fine_top_p, tile=16, block=128):
    """The "kp" selector: bool mask [H, ceil(L/tile), ceil(L/tile)] over tile x tile token squares.

    dfsattn/attention_hyvideo.py:481-489 and :211-302: the coarse top-k choice of video key blocks
    is kept (forced text / boundary columns are not part of it); inside every chosen 128 x 128 pair
    of the region before the first boundary block its 8 x 8 softmax-ed tile scores are ranked
    jointly, largest first, and a tile stays while the scores ranked before it sum to less than
    fine_top_p times the pair's total (:283-293); fine_top_p >= 1 keeps whole pairs (:266-281).
    Columns from the boundary block on are on for every earlier row, and every row from the
    boundary block on is fully on (:298-301) -- also when there is no text."""
    if tile != 16 or block != 128:
        raise ValueError("kp mode requires 128x128 coarse blocks and 16x16 sub-blocks")
    b, h, L, d = q.shape
    tpb = block // tile
    ts = tile_score_hyvideo(q, k, perm, video_len, tile, block)
    vb, kb = math.ceil(video_len / block), math.ceil(L / block)
    sums = _block_sums(ts, vb, kb, tpb)
    dense_start = video_len // block
    n_text_blocks = max(0, kb - dense_start)
    kk = max(1, int(sparsity * kb))
    coarse = torch.zeros((h, vb, kb), dtype=torch.bool)
    if n_text_blocks > 0:
        if kk - n_text_blocks <= 0:
            raise AssertionError("num_video_blocks_to_select must be non-negative")
        top = torch.topk(sums[0, :, :, :dense_start], k=kk - n_text_blocks, dim=-1).indices
    else:
        top = torch.topk(sums[0], k=kk, dim=-1).indices
    coarse.scatter_(-1, top, True)
    nf = math.ceil(L / tile)
    dfs = min(dense_start * tpb, nf)
    fine = torch.zeros((h, nf, nf), dtype=torch.bool)
    for hh in range(h):
        for qb, cb in coarse[hh, :dense_start, :dense_start].nonzero().tolist():
            vals = ts[0, hh, qb * tpb:(qb + 1) * tpb, cb * tpb:(cb + 1) * tpb].reshape(-1).float()
            if fine_top_p >= 1.0:
                keep = torch.ones_like(vals, dtype=torch.bool)
            else:
                order = torch.argsort(vals, descending=True)
                ranked = vals[order]
                keep = torch.zeros_like(vals, dtype=torch.bool)
                keep[order] = (ranked.cumsum(0) - ranked) < ranked.sum() * fine_top_p
            fine[hh, qb * tpb:(qb + 1) * tpb, cb * tpb:(cb + 1) * tpb] = keep.view(tpb, tpb)
    fine[:, :dfs, dfs:] = True
    fine[:, dfs:, :] = True
    return fine


def block_interaction_count(mask, seq_len, block=128):
    """Exact selected (q,k) token pairs; dfsattn/attention_hyvideo.py:521-546."""
    qb, kb = mask.shape[-2:]
    q_last = seq_len - block * (qb - 1)
    k_last = seq_len - block * (kb - 1)
    interior = int(torch.count_nonzero(mask[:, :-1, :-1]))
    last_q = int(torch.count_nonzero(mask[:, -1:, :-1]))
    last_k = int(torch.count_nonzero(mask[:, :-1, -1:]))
    corner = int(torch.count_nonzero(mask[:, -1:, -1:]))
    return (interior * block * block + last_q * q_last * block
            + last_k * block * k_last + corner * q_last * k_last)


def mask_to_index_lists(mask):
    """bool [H,Qb,Kb] -> (idx int32 [H,Qb,kmax] ascending, padded with -1;
    cnt int32 [H,Qb])."""
    h, qb, kb = mask.shape
    cnt = mask.sum(dim=-1).to(torch.int32)
    kmax = int(cnt.max()) if cnt.numel() else 0
    # ascending positions of True entries: sort (not mask) as keys, stable
    order = torch.argsort((~mask).to(torch.int8), dim=-1, stable=True)[..., :kmax]
    idx = order.to(torch.int32)
    pos = torch.arange(kmax)[None, None, :]
    idx = torch.where(pos < cnt[..., None], idx, torch.full_like(idx, -1))
    return idx.contiguous(), cnt.contiguous()


# --------------------------------------------------------------------------- #
# attention
# --------------------------------------------------------------------------- #
def block_sparse_attention(q, k, v, perm, inv_perm, mask, block=128, valid_len=None, q_block_range=None):
    """Block-sparse attention in the permuted order, un-permuted on return.

    Semantics of the native branch, dfsattn/attention_hyvideo.py:1034-1086:
    gather Q,K,V by perm; query token i attends the keys j of its own varlen
    segment with mask[h, i//block, j//block] (block coordinates relative to the
    segment start); softmax scale D**-0.5; inverse gather.  The per-query-block
    loop mirrors the reference's own CPU loop (:850-937, with no residual
    tokens).  Accumulates in fp32 and returns q.dtype.

    ``valid_len``: end of the first varlen segment (cu_seqlens [0, valid, L],
    dfsattn/replace_hyvideo.py:221-228); None means one segment.
    ``q_block_range``: (first, last+1) query blocks to compute (timing samples);
    rows outside stay zero.
    """
    b, h, L, d = q.shape
    assert b == 1
    scale = d ** -0.5
    qp = q[0][:, perm].float()
    kp = k[0][:, perm].float()
    vp = v[0][:, perm].float()
    out = torch.zeros_like(qp)
    segs = [(0, L)] if valid_len is None or valid_len >= L else [(0, valid_len), (valid_len, L)]
    for s0, s1 in segs:
        n = s1 - s0
        for qb in range(math.ceil(n / block)):
            if q_block_range is not None and not (q_block_range[0] <= qb < q_block_range[1]):
                continue
            r0, r1 = s0 + qb * block, min(s0 + (qb + 1) * block, s1)
            for hh in range(h):
                cols = torch.nonzero(mask[hh, qb, : math.ceil(n / block)]).flatten().tolist()
                if not cols:
                    continue
                key_idx = torch.cat([
                    torch.arange(s0 + c * block, min(s0 + (c + 1) * block, s1)) for c in cols])
                s = (qp[hh, r0:r1] @ kp[hh, key_idx].T) * scale
                out[hh, r0:r1] = torch.softmax(s, dim=-1) @ vp[hh, key_idx]
    return out[:, inv_perm].to(q.dtype).unsqueeze(0)


def dense_masked_sdpa(q, k, v, perm, inv_perm, mask, block=128):
    """Dense SDPA with the block mask expanded to tokens (single segment)."""
    L = q.shape[2]
    qp = q[:, :, perm].float()
    kp = k[:, :, perm].float()
    vp = v[:, :, perm].float()
    tok = mask.repeat_interleave(block, dim=-2).repeat_interleave(block, dim=-1)[:, :L, :L]
    o = F.scaled_dot_product_attention(qp, kp, vp, attn_mask=tok[None])
    return o[:, :, inv_perm].to(q.dtype)


def tensor_metrics(left, right):
    """max-abs, mean-abs, relative L2 (compare_attention_debug.py:10-33) + cosine."""
    a = left.float().reshape(-1)
    b = right.float().reshape(-1)
    diff = a - b
    return {
        "max_abs": float(diff.abs().max()),
        "mean_abs": float(diff.abs().mean()),
        "relative_l2": float((diff.dot(diff) / b.dot(b).clamp_min(1e-40)) ** 0.5),
        "cosine": float(a.dot(b) / (a.norm() * b.norm()).clamp_min(1e-40)),
    }
