"""Token orders over the (f, h, w) latent grid.

Mirrors ``dfsattn/utils/order.py`` for the orders the native DFS path uses:
``hilbert3d`` (:206-258) and raster order (``--order org``, no permutation).
The Hilbert order is computed by the library's host entry point
``dfs_hilbert3d_perm``.
"""
from typing import Optional

import torch

from . import ops


def hilbert3d_perm(f: int, h: int, w: int, device="cpu") -> torch.Tensor:
    """int64 [f*h*w]: raster indices (z*h*w + y*w + x) listed in Hilbert order."""
    return ops.hilbert3d_perm(f, h, w).to(device)


def raster_perm(f: int, h: int, w: int, device="cpu") -> Optional[torch.Tensor]:
    """Raster order is the absence of a permutation (``video_perm=None``)."""
    return None


def build_video_perm(order: str, f: int, h: int, w: int, device="cpu") -> Optional[torch.Tensor]:
    if order == "hilbert3d":
        return hilbert3d_perm(f, h, w, device)
    if order in ("org", "raster", None):
        return None
    raise ValueError(f"order={order!r} is not supported by the B200 DFS path (use 'hilbert3d' or 'org')")
