"""CPU: property pins of the Hilbert order (the reference's third-party code
function is unavailable offline, so these are properties, not golden vectors)."""
import numpy as np
import pytest

from oracle.hilbert import hilbert3d_perm, hilbert_encode
from dfsattn_b200.order import hilbert3d_perm as product_perm, raster_perm


@pytest.mark.parametrize("dims,bits", [(2, 1), (2, 3), (3, 1), (3, 2), (3, 4)])
def test_full_cube_is_a_unit_step_bijection(dims, bits):
    n = 1 << bits
    pts = np.stack(np.meshgrid(*[np.arange(n)] * dims, indexing="ij"), -1).reshape(-1, dims)
    codes = hilbert_encode(pts, dims, bits).astype(np.int64)
    assert sorted(codes.tolist()) == list(range(n ** dims))
    assert codes[(pts == 0).all(1)][0] == 0
    walk = pts[np.argsort(codes)]
    assert (np.abs(np.diff(walk, axis=0)).sum(1) == 1).all()


def test_known_2d_order_one_bit():
    # 2x2: (0,0) -> (0,1) -> (1,1) -> (1,0) with axis 0 most significant
    pts = np.array([[0, 0], [0, 1], [1, 1], [1, 0]])
    assert hilbert_encode(pts, 2, 1).tolist() == [0, 1, 2, 3]


@pytest.mark.parametrize("grid", [(4, 16, 16), (3, 5, 7), (1, 1, 1), (2, 1, 9), (21, 30, 52)])
def test_perm_is_filtered_curve(grid):
    f, h, w = grid
    perm = hilbert3d_perm(f, h, w)
    assert perm.dtype == np.int64 and sorted(perm.tolist()) == list(range(f * h * w))
    # in-grid filtering preserves curve order: codes along perm strictly increase
    bits = max(1, int(np.ceil(np.log2(max(grid))))) if max(grid) > 1 else 1
    z, rem = np.divmod(perm, h * w)
    y, x = np.divmod(rem, w)
    codes = hilbert_encode(np.stack([x, y, z], 1), 3, bits).astype(np.int64)
    assert (np.diff(codes) > 0).all()


@pytest.mark.parametrize("grid", [(4, 16, 16), (3, 5, 7), (33, 45, 80)])
def test_product_builder_equals_oracle(grid):
    np.testing.assert_array_equal(product_perm(*grid).numpy(), hilbert3d_perm(*grid))


def test_power_of_two_cube_neighbours():
    perm = hilbert3d_perm(8, 8, 8)
    z, rem = np.divmod(perm, 64)
    y, x = np.divmod(rem, 8)
    steps = np.abs(np.diff(np.stack([x, y, z], 1), axis=0)).sum(1)
    assert (steps == 1).all()


def test_raster():
    assert raster_perm(2, 3, 4) is None
