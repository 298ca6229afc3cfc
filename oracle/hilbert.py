"""Oracle: 3-D Hilbert token order.  TEST INFRASTRUCTURE ONLY.

Follows ``dfsattn/utils/order.py:206-258`` for everything around the code
computation (bit count :228-229, coordinate triple ordered [x, y, z] :238-247,
linear index z*h*w + y*w + x :243, argsort of the codes :255-256).

The code computation itself (``hilbert.encode`` at order.py:250) lives in the
third-party package ``numpy-hilbert-curve`` (unpinned ``>=1.0.0``), absent
offline: **parity unpinned**.  What is restated here is the algorithm that
package documents: J. Skilling, "Programming the Hilbert curve", AIP Conf.
Proc. 707 (2004) -- the inverse-undo pass over the axes (most significant bit
first, dimension 0 first), then the bits of all axes interleaved (bit level
major, dimension minor, dimension 0 most significant) and read as a Gray code.
"""

import math

import numpy as np


def hilbert_encode(coords, num_dims, num_bits):
    """Hilbert index of integer points.

    coords: int array [N, num_dims], each entry in [0, 2**num_bits).
    returns: uint64 array [N].
    """
    x = np.array(coords, dtype=np.uint64, copy=True)
    if x.ndim != 2 or x.shape[1] != num_dims:
        raise ValueError("coords must be [N, num_dims]")
    if num_dims * num_bits > 64:
        raise ValueError("num_dims * num_bits must fit in 64 bits")
    one = np.uint64(1)
    # Skilling's "inverse undo": for every bit level from the top down and
    # every axis: if the bit is set invert the lower bits of axis 0, otherwise
    # exchange the lower bits of axis 0 and this axis where they differ.
    for level in range(num_bits - 1, 0, -1):
        q = one << np.uint64(level)
        p = q - one
        for dim in range(num_dims):
            on = (x[:, dim] & q) != 0
            inv = np.where(on, p, np.uint64(0))
            t = np.where(on, np.uint64(0), (x[:, 0] ^ x[:, dim]) & p)
            x[:, 0] ^= inv
            x[:, 0] ^= t
            x[:, dim] ^= t
    # Interleave (level major, axis minor) into one Gray-coded word.
    gray = np.zeros(x.shape[0], dtype=np.uint64)
    for level in range(num_bits - 1, -1, -1):
        for dim in range(num_dims):
            gray = (gray << one) | ((x[:, dim] >> np.uint64(level)) & one)
    # Gray -> binary: prefix XOR from the most significant bit.
    code = gray.copy()
    shift = 1
    total = num_dims * num_bits
    while shift < total:
        code ^= code >> np.uint64(shift)
        shift <<= 1
    return code


def hilbert3d_perm(f, h, w):
    """Permutation (int64 [f*h*w]) listing raster indices in Hilbert order.

    ``tensor[perm]`` re-orders raster tokens (index = z*h*w + y*w + x) along
    the curve.  The curve covers the enclosing 2**b cube; only in-grid points
    are kept, in curve order (order.py:228-256).
    """
    max_dim = max(w, h, f)
    num_bits = max(1, math.ceil(math.log2(max_dim))) if max_dim > 1 else 1
    xs = np.arange(w, dtype=np.int64)
    ys = np.arange(h, dtype=np.int64)
    zs = np.arange(f, dtype=np.int64)
    # enumeration order of the reference: x slowest, then y, then z fastest
    X = np.repeat(xs, h * f)
    Y = np.tile(np.repeat(ys, f), w)
    Z = np.tile(zs, w * h)
    linear = Z * (h * w) + Y * w + X
    codes = hilbert_encode(np.stack([X, Y, Z], axis=1), 3, num_bits).astype(np.int64)
    order = np.argsort(codes, kind="stable")
    return linear[order]
