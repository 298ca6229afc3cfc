"""DFS attention for tensors that live in HOST memory.

``dfs_attention_host`` is the call for a caller whose Q/K/V sit in (pinned) host
buffers: heads are independent on the whole path, so the heads are cut into
groups and the host->device copy of group g+1, the attention of group g and the
device->host copy of group g-1 run concurrently on three CUDA streams (uploads are
queued two groups ahead).  The two copy streams and the device staging buffer are
created once per (device, shape) and reused by later calls.  Each
group keeps its own mask-cache entry (cache key ``(layer_idx, group)``), so the
refresh / reuse schedule of the operator is unchanged.  The first three and the
last two groups are single heads when there are enough heads: the first upload and
the last download are the only copies nothing overlaps, so they are kept short.

By default the call returns once the last download has landed (it waits on one
event), so ``out`` can be read and q, k, v reused straight away.  With
``wait=False`` it returns at once and hands back the event to wait on.
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


_resources = {}


def _stream_set(dev: torch.device, shape, dtype):
    """Copy streams and the staging buffer [3, H, L, D] of a (device, shape): made on first use."""
    key = (dev.index if dev.index is not None else torch.cuda.current_device(), tuple(shape), dtype)
    res = _resources.get(key)
    if res is None:
        if len(_resources) >= 4:   # a caller cycling through shapes keeps the four latest
            _resources.pop(next(iter(_resources)))
        res = {"copy_in": torch.cuda.Stream(dev), "copy_out": torch.cuda.Stream(dev),
               "stage": torch.empty((3,) + tuple(shape), dtype=dtype, device=dev)}
        _resources[key] = res
    return res


def release_resources():
    """Drop the cached copy streams and staging buffers."""
    _resources.clear()


def dfs_attention_host(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: Optional[torch.Tensor] = None,
                       head_groups: int = 12, device="cuda", flavor: str = "hyvideo", layer_idx: int = 0,
                       ramp: bool = True, wait: bool = True, **kwargs):
    """q, k, v: host tensors [1, H, L, D] (pinned memory makes the copies asynchronous).
    Returns the host tensor ``out`` ([1, H, L, D], pinned if allocated here); with ``wait=False``
    returns ``(out, event)`` without waiting: ``out`` must not be read, nor q, k, v overwritten,
    before ``event.synchronize()``.  ``kwargs`` are those of ``dfs_attention`` (step_idx, skip_steps,
    cache_interval, sparsity, ..., video_perm)."""
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
    res = _stream_set(dev, q.shape[1:], q.dtype)
    copy_in, copy_out, stage = res["copy_in"], res["copy_out"], res["stage"]
    # the staging buffer is reused: this call's uploads follow whatever the stream did before
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
    landed = torch.cuda.Event()
    landed.record(copy_out)
    compute.wait_stream(copy_out)
    compute.wait_stream(copy_in)
    if not wait:
        return out, landed
    landed.synchronize()
    return out
