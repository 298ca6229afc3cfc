import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN


def assert_masks_equal_up_to_near_ties(mine, q, k, perm, video_len, sparsity, flavor, tile=16, rtol=2e-4):
    """`mine` (bool [H, Qb, Kb], selection made on the GPU's own block scores) must equal the mask the
    oracle selects from ITS block scores on the same q, k -- except where the two scorings (fp32, different
    summation order, rtol 2e-4) can legitimately rank differently: a flipped entry's score must lie within
    `rtol` of the k-th largest score of its row, i.e. it is a near-tie at the cut."""
    import math
    import torch
    import oracle
    L = q.shape[2]
    kb = math.ceil(L / 128)
    if flavor == "wan":
        sums = oracle.block_scores_wan(q, k, perm, tile=tile)
        ref = oracle.dfs.select_wan(sums, L, sparsity)
        n_rank = kb
    else:
        sums = oracle.block_scores_hyvideo(q, k, perm, video_len, tile=tile)
        ref = oracle.dfs.select_hyvideo(sums, L, video_len, sparsity)
        n_rank = video_len // 128 if kb > video_len // 128 else kb
    diff = mine != ref
    for h, r, c in diff.nonzero().tolist():
        assert r < sums.shape[2] and c < n_rank, (h, r, c)           # forced rows and columns never flip
        ranked = sums[0, h, r, :n_rank]
        kth = torch.topk(ranked, k=int(ref[h, r, :n_rank].sum())).values[-1]
        assert abs(float(ranked[c] - kth)) <= rtol * float(kth), (h, r, c, float(ranked[c]), float(kth))
    return ref
