"""CPU: the oracle restatement against fixtures produced by the reference's own code."""
import os
import numpy as np
import pytest
import torch

import oracle
from oracle import dfs as odfs
from golden_cases import CASES, GOLDEN, ROW_STRIDE, checksum, inputs, load


def test_schedule_matches_reference_tables(golden_dir):
    g = np.load(golden_dir + "/schedule.npz")
    i = 0
    while f"params_{i}" in g:
        skip, interval, s, dcrt, steps = g[f"params_{i}"]
        for step in range(int(steps)):
            flag, val = oracle.compute_cache_schedule(step, int(skip), int(interval), float(s), float(dcrt))
            assert flag == bool(g[f"flags_{i}"][step])
            assert val == float(g[f"vals_{i}"][step])  # bit-exact float64
        i += 1
    assert i >= 5


def test_schedule_known_answers():
    # table held by the reference's tests (tests/test_flashinfer64_attention.py:122-144)
    expected = {11: (False, 0.30), 12: (True, 0.30), 23: (False, 0.30), 24: (True, 0.20),
                35: (False, 0.20), 36: (True, 0.10), 47: (False, 0.10), 48: (False, 0.10),
                49: (False, 0.10)}
    for step, (flag, val) in expected.items():
        f, v = oracle.compute_cache_schedule(step, 12, 12, 0.30, 0.10)
        assert f == flag and abs(v - val) < 1e-7
    with pytest.raises(ValueError):
        oracle.compute_cache_schedule(0, 0, 0, 0.3, 0.1)
    # the float64 drift matters for int(s*Kb)
    assert oracle.compute_cache_schedule(24, 12, 12, 0.3, 0.1)[1] == 0.19999999999999998
    assert oracle.compute_cache_schedule(36, 12, 12, 0.3, 0.1)[1] == 0.09999999999999998


@pytest.mark.parametrize("name", list(CASES))
def test_scores_masks_attention_match_reference(name):
    spec = CASES[name]
    g = load(name)
    q, k, v, vperm = inputs(name)
    assert checksum(q, k, v) == str(g["input_sha256"]), "synthetic generator changed: regenerate goldens"
    L = q.shape[2]
    video_len = L - spec["text"]
    perm, inv = oracle.build_permutation(vperm, L, video_len)

    sums = oracle.block_scores_hyvideo(q, k, perm, video_len)[0]
    np.testing.assert_array_equal(sums.numpy(), g["hy_block_sums"])
    mask = oracle.block_mask_hyvideo(q, k, perm, video_len, spec["sparsity"])
    np.testing.assert_array_equal(mask.numpy(), g["hy_mask"])
    assert oracle.block_interaction_count(mask, L) == int(g["hy_pairs"])

    o = oracle.block_sparse_attention(q, k, v, perm, inv, mask)
    np.testing.assert_allclose(o[:, :, ::ROW_STRIDE].numpy(), g["hy_attn"], atol=2e-6, rtol=1e-5)
    o2 = oracle.dense_masked_sdpa(q, k, v, perm, inv, mask)
    np.testing.assert_allclose(o2[:, :, ::ROW_STRIDE].numpy(), g["hy_attn"], atol=2e-6, rtol=1e-5)
    od = oracle.block_sparse_attention(q, k, v, perm, inv, torch.ones_like(mask))
    np.testing.assert_allclose(od[:, :, ::ROW_STRIDE].numpy(), g["dense_attn"], atol=2e-6, rtol=1e-5)

    if spec["text"] == 0:
        wsums = oracle.block_scores_wan(q, k, perm)[0]
        np.testing.assert_array_equal(wsums.numpy(), g["wan_block_sums"])
        wmask = oracle.block_mask_wan(q, k, perm, spec["sparsity"])
        np.testing.assert_array_equal(wmask.numpy(), g["wan_mask"])
        ow = oracle.block_sparse_attention(q, k, v, perm, inv, wmask)
        np.testing.assert_allclose(ow[:, :, ::ROW_STRIDE].numpy(), g["wan_attn"], atol=2e-6, rtol=1e-5)


def test_hy_and_wan_masks_agree_on_aligned_video_only_case():
    q, k, v, vperm = inputs("cfg0_4x16x16")
    perm, _ = oracle.build_permutation(vperm, 1024, 1024)
    assert torch.equal(oracle.block_mask_hyvideo(q, k, perm, 1024, 0.3),
                       oracle.block_mask_wan(q, k, perm, 0.3))


def test_index_lists_roundtrip():
    torch.manual_seed(1)
    mask = torch.rand(3, 7, 9) > 0.6
    mask[0, 0] = False
    idx, cnt = oracle.mask_to_index_lists(mask)
    back = torch.zeros_like(mask)
    for h in range(3):
        for r in range(7):
            c = int(cnt[h, r])
            assert (idx[h, r, c:] == -1).all()
            cols = idx[h, r, :c].long()
            assert (cols[1:] > cols[:-1]).all()
            back[h, r, cols] = True
    assert torch.equal(back, mask)


def test_varlen_second_segment_is_independent():
    # padding suffix = independent varlen segment (reference analogue:
    # tests/test_flashinfer64_attention.py:565-607)
    torch.manual_seed(2)
    L, valid = 300, 200
    q, k, v = (torch.randn(1, 2, L, 32) for _ in range(3))
    perm, inv = oracle.build_permutation(None, L)
    mask = torch.ones(2, 3, 3, dtype=torch.bool)
    o = odfs.block_sparse_attention(q, k, v, perm, inv, mask, valid_len=valid)
    first = torch.nn.functional.scaled_dot_product_attention(q[:, :, :valid], k[:, :, :valid], v[:, :, :valid])
    second = torch.nn.functional.scaled_dot_product_attention(q[:, :, valid:], k[:, :, valid:], v[:, :, valid:])
    torch.testing.assert_close(o[:, :, :valid], first, atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(o[:, :, valid:], second, atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("name", list(CASES))
@pytest.mark.parametrize("tag,p", [("p90", 0.9), ("p50", 0.5)])
def test_kp_fine_mask_matches_the_reference(name, tag, p):
    """oracle.fine_mask_hyvideo against the masks the reference's own kp selector produced."""
    g = np.load(os.path.join(GOLDEN, "kp_" + name + ".npz"))
    shape = tuple(int(x) for x in g[f"fine_shape_{tag}"])
    want = np.unpackbits(g[f"fine_bits_{tag}"])[: int(np.prod(shape))].reshape(shape).astype(bool)
    spec = CASES[name]
    q, k, v, vperm = inputs(name)
    L = q.shape[2]
    perm, _ = oracle.build_permutation(vperm, L, L - spec["text"])
    got = oracle.fine_mask_hyvideo(q, k, perm, L - spec["text"], spec["sparsity"], p).numpy()
    assert got.shape == shape and np.array_equal(got, want)
