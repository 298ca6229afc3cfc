"""Seeded synthetic Q/K/V with the spatial structure of video-latent activations.

Stands in for real HunyuanVideo / Wan activations (model checkpoints are not
available offline).  Per head, Q and K are each a sum of 8 three-dimensional
Fourier modes over the raster (t, y, x) grid -- wavevector components uniform
in [0, pi/4], a random phase, each mode multiplied by an N(0,1) direction in
head space -- plus 0.5*N(0,1) noise.  V ~ N(0,1).  Text tokens (appended after
the video tokens) are N(0,1) for Q, K and V.

The small random parameters (wavevectors, phases, directions) always come from
a CPU generator so that they do not depend on the device; the per-token noise
comes from a generator on the target device.
"""

import math

import torch

NUM_MODES = 8


def _grid_coords(f, h, w, device):
    t = torch.arange(f, device=device, dtype=torch.float32)
    y = torch.arange(h, device=device, dtype=torch.float32)
    x = torch.arange(w, device=device, dtype=torch.float32)
    tt, yy, xx = torch.meshgrid(t, y, x, indexing="ij")
    return torch.stack([tt.reshape(-1), yy.reshape(-1), xx.reshape(-1)], dim=1)  # [V,3] raster


def structured_qkv(grid, heads, dim, text_len=0, dtype=torch.float32, device="cpu", seed=0,
                   head_offset=0, total_heads=None):
    """Return q, k, v of shape [1, heads, f*h*w + text_len, dim].

    ``head_offset`` / ``total_heads``: generate heads [head_offset, head_offset+heads)
    of a ``total_heads``-head tensor, so that a head shard equals the slice of
    the full tensor generated with the same seed.
    """
    f, h, w = grid
    V = f * h * w
    L = V + text_len
    total_heads = heads + head_offset if total_heads is None else total_heads
    device = torch.device(device)
    coords = _grid_coords(f, h, w, device)
    out = [torch.empty((1, heads, L, dim), dtype=dtype, device=device) for _ in range(3)]
    for hh in range(total_heads):
        # one CPU generator per head keeps head shards independent of the shard layout
        cpu_gen = torch.Generator(device="cpu").manual_seed(seed * 1000003 + hh)
        params = []
        for _ in range(2):  # Q then K
            kappa = torch.rand((NUM_MODES, 3), generator=cpu_gen) * (math.pi / 4)
            phase = torch.rand((NUM_MODES,), generator=cpu_gen) * (2 * math.pi)
            dirs = torch.randn((NUM_MODES, dim), generator=cpu_gen)
            params.append((kappa, phase, dirs))
        if hh < head_offset or hh >= head_offset + heads:
            continue
        dev_gen = torch.Generator(device=device).manual_seed(seed * 7919 + 104729 * hh + 1)
        for which, (kappa, phase, dirs) in enumerate(params):
            ang = coords @ kappa.to(device).T + phase.to(device)[None, :]      # [V,8]
            x = torch.cos(ang) @ dirs.to(device)                               # [V,D]
            x = x + 0.5 * torch.randn((V, dim), generator=dev_gen, device=device)
            out[which][0, hh - head_offset, :V] = x.to(dtype)
            if text_len:
                out[which][0, hh - head_offset, V:] = torch.randn(
                    (text_len, dim), generator=dev_gen, device=device).to(dtype)
        out[2][0, hh - head_offset] = torch.randn((L, dim), generator=dev_gen, device=device).to(dtype)
    return out[0], out[1], out[2]


def drift(x, step_seed, decay=0.98, noise=0.2):
    """One denoising-step drift x <- decay*x + noise*N(0,1) (mask-caching trace)."""
    gen = torch.Generator(device=x.device).manual_seed(step_seed)
    n = torch.randn(x.shape, generator=gen, device=x.device, dtype=torch.float32)
    return (decay * x.float() + noise * n).to(x.dtype)
