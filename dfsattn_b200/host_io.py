"""DFS attention for tensors that live in HOST memory.

``dfs_attention_host`` is the call for a caller whose Q/K/V sit in (pinned) host
buffers: heads are independent on the whole path, so the heads are cut into
groups and the host->device copy of group g+1, the attention of group g and the
device->host copy of group g-1 run concurrently on three CUDA streams (uploads are
queued two groups ahead, into one device staging buffer allocated per call).  Each
group keeps its own mask-cache entry (cache key ``(layer_idx, group)``), so the
refresh / reuse schedule of the operator is unchanged.  The first three and the
last two groups are single heads when there are enough heads: the first upload and
the last download are the only copies nothing overlaps, so they are kept short.
"""
from typing import Optional

import torch

from . import attention_hyvideo, attention_wan


def group_bounds(heads: int, groups: int, ramp: bool = True):
    """[h0, h1) of each head group: ``groups`` near-equal groups, or, with ``ramp`` and at least 10
    heads and 6 groups, three single heads first (a head is uploaded a little faster than it is
    attended, so the uploads get ahead of the kernels while the groups are small), two single heads
    last, and the rest split evenly in between."""
    groups = max(1, min(int(groups), heads))
    if ramp and heads >= 10 and groups >= 6:
        inner, n = heads - 5, groups - 5
        sizes = [1, 1, 1] + [(i + 1) * inner // n - i * inner // n for i in range(n)] + [1, 1]
    else:
        sizes = [(g + 1) * heads // groups - g * heads // groups for g in range(groups)]
    bounds, h = [], 0
    for sz in sizes:
        bounds.append((h, h + sz))
        h += sz
    return bounds


def dfs_attention_host(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: Optional[torch.Tensor] = None,
                       head_groups: int = 12, device="cuda", flavor: str = "hyvideo", layer_idx: int = 0,
                       ramp: bool = True, **kwargs) -> torch.Tensor:
    """q, k, v: host tensors [1, H, L, D] (pinned memory makes the copies asynchronous).
    Returns the host tensor ``out`` ([1, H, L, D], pinned if allocated here).  ``kwargs`` are those of
    ``dfs_attention`` (step_idx, skip_steps, cache_interval, sparsity, ..., video_perm)."""
    if q.is_cuda or k.is_cuda or v.is_cuda:
        raise ValueError("dfs_attention_host takes host tensors; use dfs_attention for device tensors")
    fn = attention_hyvideo.dfs_attention if flavor == "hyvideo" else attention_wan.dfs_attention
    dev = torch.device(device)
    H = q.shape[1]
    bounds = group_bounds(H, head_groups, ramp)
    groups = len(bounds)
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
