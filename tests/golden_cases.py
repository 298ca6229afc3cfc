"""Shared description of the golden cases (mirrors tests/golden/make_golden.py)."""
import hashlib
import os

import numpy as np
import torch

from dfsattn_b200.synthetic import structured_qkv
from oracle.hilbert import hilbert3d_perm

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
ROW_STRIDE = 5

CASES = {
    "cfg0_4x16x16": dict(grid=(4, 16, 16), text=0, heads=2, dim=64, sparsity=0.3, order="hilbert3d"),
    "hy_text_4x12x20_t100": dict(grid=(4, 12, 20), text=100, heads=2, dim=128, sparsity=0.5, order="hilbert3d"),
    "hy_text_5x11x17_t256": dict(grid=(5, 11, 17), text=256, heads=3, dim=128, sparsity=0.45, order="hilbert3d"),
    "ragged_5x11x17": dict(grid=(5, 11, 17), text=0, heads=2, dim=128, sparsity=0.3, order="hilbert3d"),
    "raster_3x16x16": dict(grid=(3, 16, 16), text=0, heads=2, dim=64, sparsity=0.34, order="raster"),
}


def load(name):
    return np.load(os.path.join(GOLDEN, name + ".npz"))


def inputs(name, seed=0):
    spec = CASES[name]
    f, h, w = spec["grid"]
    q, k, v = structured_qkv(spec["grid"], spec["heads"], spec["dim"], text_len=spec["text"],
                             dtype=torch.float32, device="cpu", seed=seed)
    vperm = torch.from_numpy(hilbert3d_perm(f, h, w)) if spec["order"] == "hilbert3d" else None
    return q, k, v, vperm


def checksum(*tensors):
    m = hashlib.sha256()
    for t in tensors:
        m.update(t.contiguous().numpy().tobytes())
    return m.hexdigest()
