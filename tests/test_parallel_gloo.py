"""CPU, world_size 2 over gloo: the head partition and the sequence<->head
all-to-all swap of the multi-GPU entry points (no GPU kernels involved)."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, H, L, D, results):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from dfsattn_b200 import parallel
        g = torch.Generator().manual_seed(0)
        full = [torch.randn(H, L, D, generator=g) for _ in range(3)]  # same on every rank
        s0, n = parallel.seq_shard(L, rank, world)
        h0, hp = parallel.head_shard(H, rank, world)
        local = [t[:, s0:s0 + n].contiguous() for t in full]
        heads = parallel.seq_to_head_shards(local, L)
        ok = all(torch.equal(heads[i], full[i][h0:h0 + hp]) for i in range(3))
        # attention stand-in: a function of the full sequence per head (cumulative sum over tokens)
        fake = lambda q, k, v: torch.cumsum(q + 2 * k - v, dim=2)
        out = parallel.dfs_attention_sequence_parallel(local[0][None], local[1][None], local[2][None], L, fake)
        want = torch.cumsum(full[0] + 2 * full[1] - full[2], dim=1)[:, s0:s0 + n]
        ok = ok and torch.equal(out[0], want)
        back = parallel.head_to_seq_shards(full[0][h0:h0 + hp].contiguous(), H)
        ok = ok and torch.equal(back, local[0])
        results[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("H,L,D", [(4, 10, 8), (6, 257, 16)])
def test_sequence_parallel_swap_world2(H, L, D):
    world = 2
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), H, L, D, results), nprocs=world, join=True)
    assert dict(results) == {0: True, 1: True}


def test_partitions_cover_everything():
    sys.path.insert(0, ROOT)
    from dfsattn_b200 import parallel
    for world in (1, 2, 4, 8):
        heads = [parallel.head_shard(24, r, world) for r in range(world)]
        assert sorted(h for s, n in heads for h in range(s, s + n)) == list(range(24))
        toks = [parallel.seq_shard(119056, r, world) for r in range(world)]
        assert sum(n for _, n in toks) == 119056 and toks[0][0] == 0
        assert all(toks[i][0] + toks[i][1] == toks[i + 1][0] for i in range(world - 1))
    with pytest.raises(ValueError):
        parallel.head_shard(24, 0, 5)
