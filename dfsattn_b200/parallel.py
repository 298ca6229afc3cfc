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

``SequenceShardExchange`` is the fused form of the same exchange for the GPUs of
one node: the shards live in symmetric (peer-accessible) memory, the Hilbert
gather reads every row straight from the GPU that holds it and the attention
kernel stores every output row straight into the shard of the GPU that owns it
-- the two all-to-alls and their staging copies disappear into the gather and
into the attention epilogue.  Plain loads and stores over NVLink; no multicast.
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


class SequenceShardExchange:
    """Sequence shards of Q, K, V and of the output in symmetric memory, for the fused exchange.

    Every rank constructs one (collectively), writes its tokens into ``inputs()`` and calls
    ``run``; afterwards ``output()`` holds its tokens of the result for all heads.  One barrier
    across the GPUs before the gather (every shard is written) and one after the attention (every
    row has landed); both are stream-ordered kernels of the symmetric-memory handle, so no host
    synchronisation happens.
    """

    def __init__(self, heads: int, seq_len: int, head_dim: int, device, group=None):
        import torch.distributed._symmetric_memory as symm
        from . import ops
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.heads, self.seq_len, self.head_dim = heads, seq_len, head_dim
        self.head0, self.heads_local = head_shard(heads, self.rank, self.world)
        self.chunk = -(-seq_len // self.world)
        self.start, self.rows = seq_shard(seq_len, self.rank, self.world)
        self._in = symm.empty((3, heads, self.chunk, head_dim), dtype=torch.bfloat16, device=device)
        self._out = symm.empty((heads, self.chunk, head_dim), dtype=torch.bfloat16, device=device)
        self._h_in = symm.rendezvous(self._in, self.group)
        self._h_out = symm.rendezvous(self._out, self.group)
        plane = heads * self.chunk * head_dim * 2   # bytes of one of Q, K, V inside a shard
        in_ptrs = list(self._h_in.buffer_ptrs)
        self.in_tabs = [ops.ShardTable([p + t * plane for p in in_ptrs], self.chunk, self.chunk) for t in range(3)]
        self.out_tab = ops.ShardTable(list(self._h_out.buffer_ptrs), self.chunk, self.chunk)

    def inputs(self):
        """(q, k, v) views [H, rows, D] of this rank's shard, to be filled by the producer."""
        return tuple(self._in[t, :, :self.rows] for t in range(3))

    def output(self) -> torch.Tensor:
        """[H, rows, D] view of this rank's tokens of the result."""
        return self._out[:, :self.rows]

    def run(self, attention_fn, perm_i32) -> torch.Tensor:
        """``attention_fn(q, k, v, **kw)`` is a partial of ``dfs_attention`` (or of ``full_attention``
        wrapped likewise) that accepts ``prepermuted``, ``out_shards`` and ``out_head0``; ``perm_i32``
        is the int32 device permutation of the whole sequence it will use (None for raster order)."""
        from . import ops
        self._h_in.barrier(channel=0)
        qp, kp, vp = ops.permute_qkv_sharded(*self.in_tabs, self.head0, self.heads_local, self.seq_len,
                                             self.head_dim, perm_i32, self._in.device)
        attention_fn(qp[None], kp[None], vp[None], prepermuted=True, out_shards=self.out_tab,
                     out_head0=self.head0)
        self._h_out.barrier(channel=0)
        return self.output()
