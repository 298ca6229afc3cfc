"""DFS attention for tensors that live in HOST memory.

``dfs_attention_host`` is the call for a caller whose Q/K/V sit in (pinned) host
buffers: heads are independent on the whole path, so the heads are cut into
groups and the host->device copy of group g+1, the attention of group g and the
device->host copy of group g-1 run concurrently on three CUDA streams (uploads are
queued two groups ahead, into one device staging buffer allocated per call).  Each
group keeps its own mask-cache entry (cache key ``(layer_idx, group)``), so the
refresh / reuse schedule of the operator is unchanged.
"""
from typing import Optional

import torch

from . import attention_hyvideo, attention_wan


def dfs_attention_host(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: Optional[torch.Tensor] = None,
                       head_groups: int = 12, device="cuda", flavor: str = "hyvideo", layer_idx: int = 0,
                       **kwargs) -> torch.Tensor:
    """q, k, v: host tensors [1, H, L, D] (pinned memory makes the copies asynchronous).
    Returns the host tensor ``out`` ([1, H, L, D], pinned if allocated here).  ``kwargs`` are those of
    ``dfs_attention`` (step_idx, skip_steps, cache_interval, sparsity, ..., video_perm)."""
    if q.is_cuda or k.is_cuda or v.is_cuda:
        raise ValueError("dfs_attention_host takes host tensors; use dfs_attention for device tensors")
    fn = attention_hyvideo.dfs_attention if flavor == "hyvideo" else attention_wan.dfs_attention
    dev = torch.device(device)
    H = q.shape[1]
    groups = max(1, min(head_groups, H))
    bounds = [(g * H // groups, (g + 1) * H // groups) for g in range(groups)]
    if out is None:
        out = torch.empty(q.shape, dtype=q.dtype).pin_memory()
    compute = torch.cuda.current_stream(dev)
    copy_in, copy_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    # one device staging buffer for all three tensors: a single allocation per call
    stage = torch.empty((3,) + tuple(q.shape[1:]), dtype=q.dtype, device=dev)
    stage.record_stream(copy_in)
    copy_in.wait_stream(compute)
    uploaded = []

    def upload(g):
        h0, h1 = bounds[g]
        with torch.cuda.stream(copy_in):
            for i, t in enumerate((q, k, v)):
                stage[i, h0:h1].copy_(t[0, h0:h1], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(copy_in)
        uploaded.append(ev)

    # The copy stream always holds the next two uploads; the host does not queue all uploads
    # before the first kernels (issuing a copy costs host time that would delay them).
    for g in range(min(2, groups)):
        upload(g)
    for g, (h0, h1) in enumerate(bounds):
        compute.wait_event(uploaded[g])
        o = fn(stage[0, h0:h1].unsqueeze(0), stage[1, h0:h1].unsqueeze(0), stage[2, h0:h1].unsqueeze(0),
               layer_idx=(layer_idx, g), **kwargs)
        done = torch.cuda.Event()
        done.record(compute)
        if g + 2 < groups:
            upload(g + 2)
        with torch.cuda.stream(copy_out):
            copy_out.wait_event(done)
            o.record_stream(copy_out)
            out[:, h0:h1].copy_(o, non_blocking=True)
    compute.wait_stream(copy_out)
    compute.wait_stream(copy_in)
    return out
