"""Multi-GPU entry points of the DFS attention path (one process per GPU).

Heads are independent in every stage of the path (scores, top-k lists, mask
cache and attention are all per head), so the primary partitioning is by
head and needs no collective: rank r works on heads [r*H/P, (r+1)*H/P).

Inputs that arrive SEQUENCE-sharded (rank r holds a contiguous range of the L
raster-order tokens for all H heads) are first turned into head shards with one
all-to-all over Q, K and V together (Ulysses-style head/sequence swap), because
the Hilbert permutation, the pooled scoring and the selection are global over
the sequence; the output goes back through one all-to-all.  The collective is
``torch.distributed.all_to_all_single`` (NCCL over NVLink on GPUs, gloo in the
CPU tests); everything a kernel reads has landed in local memory before the
kernel runs.
"""
from typing import List, Tuple

import torch
import torch.distributed as dist


def head_shard(num_heads: int, rank: int, world: int) -> Tuple[int, int]:
    """(first head, head count) of ``rank``; heads must divide evenly."""
    if num_heads % world != 0:
        raise ValueError(f"{num_heads} heads do not split evenly over {world} ranks")
    per = num_heads // world
    return rank * per, per


def seq_shard(seq_len: int, rank: int, world: int) -> Tuple[int, int]:
    """(first token, token count) of ``rank`` for a sequence split into
    ``world`` contiguous chunks of ceil(L/world) tokens (the last may be short)."""
    chunk = -(-seq_len // world)
    start = min(rank * chunk, seq_len)
    return start, min(chunk, seq_len - start)


def seq_to_head_shards(tensors: List[torch.Tensor], seq_len: int, group=None) -> List[torch.Tensor]:
    """[H, L_r, D] sequence shards (one per tensor in ``tensors``, same shape) ->
    [H/P, L, D] head shards, with ONE all-to-all for all of them."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    n = len(tensors)
    H, Lr, D = tensors[0].shape
    _, hp = head_shard(H, rank, world)
    assert Lr == seq_shard(seq_len, rank, world)[1], "local shard length does not match the sequence split"
    # [n, H, Lr, D] -> per destination rank d: [n, hp, Lr, D]
    send = torch.stack(tensors).view(n, world, hp, Lr, D).permute(1, 0, 2, 3, 4).contiguous()
    lens = [seq_shard(seq_len, s, world)[1] for s in range(world)]
    recv = torch.empty(n * hp * seq_len * D, dtype=send.dtype, device=send.device)
    dist.all_to_all_single(recv, send.view(-1), output_split_sizes=[n * hp * l * D for l in lens],
                           input_split_sizes=[n * hp * Lr * D] * world, group=group)
    out = torch.empty((n, hp, seq_len, D), dtype=send.dtype, device=send.device)
    off = pos = 0
    for s in range(world):
        out[:, :, pos:pos + lens[s]] = recv[off:off + n * hp * lens[s] * D].view(n, hp, lens[s], D)
        off += n * hp * lens[s] * D
        pos += lens[s]
    return [out[i] for i in range(n)]


def head_to_seq_shards(x: torch.Tensor, num_heads: int, group=None) -> torch.Tensor:
    """[H/P, L, D] head shard -> [H, L_r, D] sequence shard (inverse swap, one all-to-all)."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    hp, L, D = x.shape
    lens = [seq_shard(L, d, world)[1] for d in range(world)]
    Lr = lens[rank]
    chunks, pos = [], 0
    for d in range(world):
        chunks.append(x[:, pos:pos + lens[d]].reshape(-1))
        pos += lens[d]
    send = torch.cat(chunks)
    recv = torch.empty(world * hp * Lr * D, dtype=x.dtype, device=x.device)
    dist.all_to_all_single(recv, send, output_split_sizes=[hp * Lr * D] * world,
                           input_split_sizes=[hp * l * D for l in lens], group=group)
    return recv.view(world * hp, Lr, D)[:num_heads]


def dfs_attention_sequence_parallel(q, k, v, seq_len: int, attention_fn, group=None):
    """q, k, v: [1, H, L_r, D] sequence shards (raster order).  ``attention_fn`` is
    called as ``attention_fn(q, k, v)`` with [1, H/P, L, D] head shards (e.g. a
    partial of ``dfs_attention``) and must return [1, H/P, L, D].  Returns this
    rank's [1, H, L_r, D] slice of the output."""
    H = q.shape[1]
    qh, kh, vh = seq_to_head_shards([q[0], k[0], v[0]], seq_len, group)
    out = attention_fn(qh[None], kh[None], vh[None])
    return head_to_seq_shards(out[0].contiguous(), H, group)[None]
