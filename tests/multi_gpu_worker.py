"""Worker of tests/test_gpu_multi.py (one process per GPU, started by torch.distributed.run):
the fused sequence-shard exchange against the all-to-all form and against the single-GPU call."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    from dfsattn_b200 import engine, ops, parallel
    from dfsattn_b200.attention_hyvideo import DFS_Attention, _dfs_attention_instances, dfs_attention
    from dfsattn_b200.fullattention import full_attention
    from dfsattn_b200.order import hilbert3d_perm
    from dfsattn_b200.synthetic import structured_qkv

    grid, text, H, D = (5, 12, 21), 100, 4, 128          # L = 1360: not a multiple of the world size or of 128
    q, k, v = structured_qkv(grid, H, D, text_len=text, dtype=torch.bfloat16, device=dev, seed=0)
    L = q.shape[2]
    video_len = L - text
    vperm = hilbert3d_perm(*grid)
    kw = dict(step_idx=12, skip_steps=12, cache_interval=12, sparsity=0.5, sparsity_dcrt=0.1, tile_size=16,
              block_size=128, video_len=video_len, video_perm=vperm)
    t0, tn = parallel.seq_shard(L, rank, world)
    shards = [t[:, :, t0:t0 + tn].contiguous() for t in (q, k, v)]

    def reset():
        DFS_Attention.clear_cache()
        _dfs_attention_instances.clear()

    # 1. every head on this GPU (the single-GPU answer)
    reset()
    whole = dfs_attention(q, k, v, layer_idx=0, **kw)
    # 2. sequence shards swapped by all-to-alls around head-sharded compute
    reset()
    swapped = parallel.dfs_attention_sequence_parallel(*shards, L, lambda a, b, c: dfs_attention(a, b, c, layer_idx=0, **kw))
    # 3. the fused exchange: gather from and scatter to peer shards inside the kernels
    reset()
    ex = parallel.SequenceShardExchange(H, L, D, dev)
    for dst, src in zip(ex.inputs(), shards):
        dst.copy_(src[0])
    perm_dev, _ = engine._perm_cache.get(vperm, L, video_len, dev)
    for _ in range(2):   # twice: buffers are reused from call to call
        fused = ex.run(lambda a, b, c, **e: dfs_attention(a, b, c, layer_idx=0, **kw, **e), perm_dev).clone()
    # 4. the dense call through the same exchange
    dense = ex.run(lambda a, b, c, prepermuted, out_shards, out_head0: full_attention(
        a, b, c, mode="flash", out_row_map=perm_dev, out_shards=out_shards, out_head0=out_head0), perm_dev).clone()
    torch.cuda.synchronize()
    ops.check_status(dev)
    want = whole[0, :, t0:t0 + tn]
    assert torch.equal(swapped[0], want), "all-to-all form differs from the single-GPU call"
    assert torch.equal(fused, want), "fused exchange differs from the single-GPU call"
    ref = torch.nn.functional.scaled_dot_product_attention(q.float(), k.float(), v.float())[0, :, t0:t0 + tn]
    err = float((dense.float() - ref).abs().max())
    assert err <= 2e-2, err
    dist.barrier()
    if rank == 0:
        print("MULTI_GPU_OK", world, flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
