"""GPU: the allocation-free scoring entry point (dfs_block_scores_static).

Some callers of this library cannot allocate device memory when they need
block scores -- their memory pool is frozen after start-up, or they run inside
another framework's step where an allocation would stall the device.  For them
the library carries a fixed 32 MiB scratch array; this test checks, through the
C ABI, that the entry point using it returns exactly what the regular entry
point (caller-provided workspace) returns, on two calls in a row with different
inputs (the shared scratch keeps the first call's contents), and that shapes
beyond the fixed size are refused.  The file name sorts last so that a run that
stops at the first failure has already run every other test.
"""
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from dfsattn_b200 import ops as _ops
    return _ops


def _case(seed, H, L, video_len, D, dtype):
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randn(H, L, D, generator=g, device="cuda").to(dtype)
    k = torch.randn(H, L, D, generator=g, device="cuda").to(dtype)
    return q, k, video_len


def test_static_scratch_scores_equal_workspace_scores_twice_in_a_row(ops):
    calls = [
        _case(1, 3, 1191, 935, 128, torch.bfloat16),   # text tail, ragged video part
        _case(2, 2, 4096, 4096, 64, torch.float32),    # different shape: stale scratch must not leak
        _case(3, 3, 1191, 935, 128, torch.bfloat16),   # first shape again, new values
    ]
    for n, (q, k, video_len) in enumerate(calls):
        H, L, D = q.shape
        wan = video_len == L
        want = ops.block_scores(q, k, video_len, wan)
        out = torch.full_like(want, float("nan"))
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        reserved_before = torch.cuda.memory_reserved()
        got = ops.block_scores_static(q, k, video_len, wan, out)
        torch.cuda.synchronize()
        assert got is out
        assert torch.cuda.memory_reserved() == reserved_before   # torch's allocator asked for nothing
        if n > 0:   # the first call may load the kernels' module image; later calls leave the device's free memory alone
            assert torch.cuda.mem_get_info()[0] == free_before
        # same kernels, same inputs: the tolerance of the scoring tests (rtol 2e-4) and in fact bit-equal
        torch.testing.assert_close(got, want, rtol=2e-4, atol=1e-6)
        assert torch.equal(got, want)
        # and against the CPU oracle of the reference's scoring on the same values (inputs are already in
        # the permuted order: identity permutation)
        qc, kc = q.float().cpu()[None], k.float().cpu()[None]
        ident = torch.arange(L)
        ref = (oracle.block_scores_wan(qc, kc, ident) if wan
               else oracle.block_scores_hyvideo(qc, kc, ident, video_len))[0]
        torch.testing.assert_close(got.cpu(), ref, rtol=2e-4, atol=1e-6)


def test_static_scratch_rejects_shapes_beyond_its_size(ops):
    limit = ops.lib.dfs_block_scores_static_max_bytes()
    assert limit == 32 << 20
    H, L, D = 16, 32768, 128
    assert ops.lib.dfs_score_workspace_bytes(H, L, L, D, 16, 128, 1) > limit
    q = torch.zeros(H, L, D, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros(H, L // 128, L // 128, device="cuda")
    with pytest.raises(ValueError, match="32 MiB"):
        ops.block_scores_static(q, q, L, True, out)
