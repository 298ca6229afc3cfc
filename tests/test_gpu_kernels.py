"""GPU parity of the permute / score / select kernels against the CPU oracle,
through the C ABI (dfsattn_b200.ops wraps one entry point per function)."""
import math

import pytest
from conftest import assert_masks_equal_up_to_near_ties
import torch

import oracle
from golden_cases import CASES, inputs, load

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from dfsattn_b200 import ops as _ops
    return _ops


@pytest.mark.parametrize("dtype,D", [(torch.bfloat16, 128), (torch.float32, 64), (torch.bfloat16, 64),
                                     (torch.float32, 128)])
@pytest.mark.parametrize("L,text", [(1024, 0), (1191, 256), (37, 5)])
def test_permute_bit_exact(ops, dtype, D, L, text):
    # mirrors the reference's bit-equality check of fused permute vs gather
    # (tests/test_flashinfer64_attention.py:64-93), with a text tail
    g = torch.Generator().manual_seed(L * 7 + D)
    H = 3
    q, k, v = (torch.randn(H, L, D, generator=g).to(dtype) for _ in range(3))
    vperm = torch.randperm(L - text, generator=g)
    perm, inv = oracle.build_permutation(vperm, L, L - text)
    qd, kd, vd = (t.cuda() for t in (q, k, v))
    pi = perm.to(torch.int32).cuda()
    qo, ko, vo = ops.permute_qkv(qd, kd, vd, pi)
    assert torch.equal(qo.cpu(), q[:, perm]) and torch.equal(ko.cpu(), k[:, perm])
    assert torch.equal(vo.cpu(), v[:, perm])
    back = ops.unpermute(qo, inv.to(torch.int32).cuda())
    assert torch.equal(back.cpu(), q)
    only_k = ops.permute_qkv(None, kd, None, pi)
    assert only_k[0] is None and torch.equal(only_k[1].cpu(), k[:, perm])


def test_permute_rejects_bad_arguments(ops):
    x = torch.zeros(2, 8, 64, device="cuda", dtype=torch.bfloat16)
    p = torch.arange(8, device="cuda", dtype=torch.int32)
    with pytest.raises(ValueError):
        ops.lib.dfs_permute_qkv  # symbol exists
        ops.check(ops.lib.dfs_permute_qkv(x.data_ptr(), None, None, p.data_ptr(), x.data_ptr(), None, None,
                                          2, 8, 128, None), "in place")
    with pytest.raises(ValueError):
        ops.check(ops.lib.dfs_permute_qkv(x.data_ptr(), None, None, None, x.data_ptr() + 16, None, None,
                                          2, 8, 128, None), "null perm")


def _select_oracle(scores, n_rank, k_select, dense_row_start, q_rows):
    H, score_rows, n_cols = scores.shape
    mask = torch.zeros(H, q_rows, n_cols, dtype=torch.bool)
    top = torch.topk(scores[:, :min(dense_row_start, score_rows), :n_rank], k=k_select, dim=-1).indices
    mask[:, :top.shape[1]].scatter_(-1, top, True)
    mask[:, :, n_rank:] = True
    mask[:, dense_row_start:] = True
    return mask


@pytest.mark.parametrize("H,score_rows,q_rows,cols,n_rank,k,dense", [
    (2, 8, 8, 8, 8, 2, 8),              # config-0 like
    (3, 8, 10, 10, 7, 2, 7),            # text tail: forced columns + dense rows
    (2, 30, 30, 300, 300, 90, 30),      # more columns than one chunk of threads
    (1, 929, 931, 931, 928, 276, 928),  # 720p HunyuanVideo geometry
    (1, 40, 40, 600, 590, 100, 38),     # 16 keys per lane
    (1, 20, 20, 1100, 1090, 250, 20),   # rows past 1024 ranked columns: keys in shared memory
    (2, 6, 6, 6, 6, 6, 6),              # k == all
    (2, 6, 6, 6, 5, 1, 6),              # ragged video, no text: forced last column, no dense rows
])
def test_select_matches_topk_bit_exact(ops, H, score_rows, q_rows, cols, n_rank, k, dense):
    g = torch.Generator().manual_seed(score_rows * 131 + cols)
    scores = torch.rand(H, score_rows, cols, generator=g)  # continuous: no ties
    idx, cnt, mask = ops.select_topk(scores.cuda(), q_rows=q_rows, n_rank=n_rank, k_select=k,
                                     dense_row_start=dense, want_mask=True)
    want = _select_oracle(scores, n_rank, k, dense, q_rows)
    assert torch.equal(mask.cpu().bool(), want)
    widx, wcnt = oracle.mask_to_index_lists(want)
    kmax = idx.shape[-1]
    assert kmax == max(1, k + cols - n_rank)            # as long as a ranked row needs, not as a dense row
    idx, cnt = idx.cpu(), cnt.cpu()
    marked = kmax < cols                                # dense rows then carry the count -1 and no list
    last_listed = dense if marked else q_rows
    assert torch.equal(cnt[:, :last_listed], wcnt[:, :last_listed])
    assert torch.equal(idx[:, :last_listed], widx[:, :last_listed, :kmax])
    if marked:
        assert bool((cnt[:, dense:] == -1).all()) and bool((idx[:, dense:] == -1).all())
    from dfsattn_b200.engine import BlockLists
    lists = BlockLists(idx.cuda(), cnt.cuda(), cols)
    assert torch.equal(lists.to_bool_mask().cpu(), want)
    if q_rows == cols:                                  # the pair count is defined for square masks
        L = cols * 128 - 37
        assert ops.interaction_count(lists.idx, lists.cnt, H, L) == oracle.block_interaction_count(want, L)
    # with room for every column the dense rows are listed like the others
    from dfsattn_b200 import _lib
    big = torch.empty((H, q_rows, cols), dtype=torch.int32, device="cuda")
    bcnt = torch.empty((H, q_rows), dtype=torch.int32, device="cuda")
    sc = scores.cuda()
    assert _lib.lib.dfs_select_topk(sc.data_ptr(), H, score_rows, q_rows, cols, n_rank, k, dense, big.data_ptr(),
                                    bcnt.data_ptr(), cols, None, None) == 0
    torch.cuda.synchronize()
    assert torch.equal(bcnt.cpu(), wcnt)
    kk = widx.shape[-1]
    assert torch.equal(big.cpu()[..., :kk], widx) and bool((big.cpu()[..., kk:] == -1).all())


def test_select_ties_go_to_the_lowest_column(ops):
    scores = torch.tensor([[[1.0, 3.0, 3.0, 2.0, 3.0, 0.5]]])
    idx, cnt, _ = ops.select_topk(scores.cuda(), q_rows=1, n_rank=6, k_select=2, dense_row_start=1)
    assert idx.cpu()[0, 0].tolist() == [1, 2] and int(cnt) == 2


@pytest.mark.parametrize("cols", [200, 500, 1000, 1100])
def test_select_many_ties_every_row_length(ops, cols):
    """Scores with a handful of distinct values (the k-th place always falls inside a run of equal
    scores), for each way the kernel holds a row: 8, 16 or 32 keys per lane, or shared memory."""
    g = torch.Generator().manual_seed(cols)
    scores = torch.randint(0, 5, (2, 12, cols), generator=g).float() - 2.0      # negative, zero and positive
    n_rank, k = cols - 3, cols // 3
    idx, cnt, mask = ops.select_topk(scores.cuda(), q_rows=12, n_rank=n_rank, k_select=k, dense_row_start=12,
                                     want_mask=True)
    order = torch.sort(scores[..., :n_rank], dim=-1, descending=True, stable=True).indices[..., :k]
    want = torch.zeros(2, 12, cols, dtype=torch.bool)
    want.scatter_(-1, order, True)
    want[..., n_rank:] = True
    assert torch.equal(mask.cpu().bool(), want)
    widx, wcnt = oracle.mask_to_index_lists(want)
    assert torch.equal(cnt.cpu(), wcnt) and torch.equal(idx.cpu(), widx[..., :idx.shape[-1]])


def test_select_rejects_bad_arguments(ops):
    s = torch.zeros(1, 4, 4, device="cuda")
    with pytest.raises(ValueError):
        ops.select_topk(s, q_rows=4, n_rank=4, k_select=5, dense_row_start=4)   # k > candidates
    with pytest.raises(ValueError):
        ops.select_topk(s, q_rows=6, n_rank=4, k_select=2, dense_row_start=5)   # ranked row without scores


@pytest.mark.parametrize("name", list(CASES))
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_block_scores_and_lists_match_reference(ops, name, dtype):
    """fp32 scoring on the GPU vs the reference's block sums (golden, fp32) and,
    for bf16 inputs, vs the oracle run on the same bf16-rounded values."""
    from dfsattn_b200 import engine
    spec = CASES[name]
    g = load(name)
    q, k, v, vperm = inputs(name)
    L = q.shape[2]
    video_len = L - spec["text"]
    perm, _ = oracle.build_permutation(vperm, L, video_len)
    q, k = q.to(dtype), k.to(dtype)
    qp = q[0][:, perm].contiguous().cuda()
    kp = k[0][:, perm].contiguous().cuda()
    for flavor in ("hyvideo", "wan"):
        if flavor == "wan" and spec["text"]:
            continue
        got = ops.block_scores(qp, kp, video_len, flavor == "wan").cpu()
        if dtype == torch.float32:
            want = torch.from_numpy(g["hy_block_sums" if flavor == "hyvideo" else "wan_block_sums"])
        elif flavor == "hyvideo":
            want = oracle.block_scores_hyvideo(q.float(), k.float(), perm, video_len)[0]
        else:
            want = oracle.block_scores_wan(q.float(), k.float(), perm)[0]
        # fp32 with a different summation order: tolerance, then rows sum to 8
        torch.testing.assert_close(got, want, rtol=2e-4, atol=1e-6)
        torch.testing.assert_close(got.sum(-1), torch.full_like(got.sum(-1), 8.0), rtol=1e-4, atol=1e-4)
        # selection on the oracle's own fp32 scores must be bit-exact
        idx, cnt, mask = engine.select_lists(want.contiguous().cuda(), L, video_len, spec["sparsity"], flavor,
                                             want_mask=True)
        if dtype == torch.float32:
            ref_mask = torch.from_numpy(g["hy_mask" if flavor == "hyvideo" else "wan_mask"])
            assert torch.equal(mask.cpu().bool(), ref_mask)
            assert ops.interaction_count(idx, cnt, ref_mask.shape[0], L) == \
                oracle.block_interaction_count(ref_mask, L)
        # end to end (GPU scores -> GPU selection) agrees unless the k-th gap is within rounding
        lists = engine.compute_block_lists(qp, kp, video_len, spec["sparsity"], flavor)
        mine = lists.to_bool_mask().cpu()
        if flavor == "hyvideo":
            ref = oracle.dfs.select_hyvideo(want[None], L, video_len, spec["sparsity"])
        else:
            ref = oracle.dfs.select_wan(want[None], L, spec["sparsity"])
        diff = (mine != ref)
        if diff.any():  # only near-ties at the k-th place may flip
            kb = math.ceil(L / 128)
            n_rank = video_len // 128 if (flavor == "hyvideo" and kb > video_len // 128) else kb
            for h, r, c in diff.nonzero().tolist():
                ranked = want[h, r, :n_rank]
                kth = torch.topk(ranked, k=int(ref[h, r, :n_rank].sum())).values[-1]
                assert abs(float(want[h, r, c] - kth)) <= 2e-4 * float(kth)


@pytest.mark.parametrize("tile", [32, 64])
@pytest.mark.parametrize("name", ["hy_text_5x11x17_t256", "ragged_5x11x17"])
def test_block_scores_other_tile_sizes(ops, name, tile):
    """tile_size 32 and 64 (4 and 2 pooled tiles per block) against the oracle."""
    from dfsattn_b200 import engine
    spec = CASES[name]
    q, k, v, vperm = inputs(name)
    L = q.shape[2]
    video_len = L - spec["text"]
    perm, _ = oracle.build_permutation(vperm, L, video_len)
    q, k = q.bfloat16(), k.bfloat16()
    qp = q[0][:, perm].contiguous().cuda()
    kp = k[0][:, perm].contiguous().cuda()
    got = ops.block_scores(qp, kp, video_len, False, tile=tile).cpu()
    want = oracle.block_scores_hyvideo(q.float(), k.float(), perm, video_len, tile=tile)[0]
    torch.testing.assert_close(got, want, rtol=2e-4, atol=1e-6)
    tpb = 128 // tile
    torch.testing.assert_close(got.sum(-1), torch.full_like(got.sum(-1), float(tpb)), rtol=1e-4, atol=1e-4)
    lists = engine.compute_block_lists(qp, kp, video_len, spec["sparsity"], "hyvideo", tile=tile)
    assert_masks_equal_up_to_near_ties(lists.to_bool_mask().cpu(), q.float(), k.float(), perm, video_len,
                                       spec["sparsity"], "hyvideo", tile=tile)


@pytest.mark.parametrize("blocks", [1024, 1030])
def test_block_scores_rows_around_1024_key_blocks(ops, blocks):
    """The block-sum kernel holds a pooled row of up to 1024 key blocks in registers and falls back to a
    three-pass kernel past that: both sides of the switch against the oracle."""
    g = torch.Generator().manual_seed(blocks)
    L = blocks * 128 - 50
    q = torch.randn(1, 1, L, 64, generator=g)
    k = torch.randn(1, 1, L, 64, generator=g) * 2
    got = ops.block_scores(q[0].cuda(), k[0].cuda(), L, True).cpu()
    want = oracle.block_scores_wan(q, k, torch.arange(L))[0]
    torch.testing.assert_close(got, want, rtol=2e-4, atol=1e-6)
    torch.cuda.synchronize()
    ops.check_status("cuda")


# (heads, tokens, head width, tokens per pooled tile): 4, 3, 2 and 2 tiles of 128 pooled query rows (an odd count
# leaves the last pair with one CTA whose rows are all padding), key tiles cut into several ranges per CTA
_PAIR_SHAPES = [(2, 8192, 128, 16), (3, 128 * 40 + 57, 128, 16), (1, 128 * 33, 64, 32), (2, 128 * 70 + 5, 64, 64)]


def test_block_scores_pairs_equal_single_ctas(ops, tmp_path):
    """The logits kernel as CTA pairs (default: two CTAs share every pooled-K tile, 256 query rows per MMA)
    against its single-CTA form, which a child process runs with DFSATTN_SCORE_PAIRS=0 (the switch is read
    once per process): same bits, and both against the oracle.  Shapes with even and odd numbers of pooled
    query tiles, both head widths, every pooled-tile size."""
    import os
    import subprocess
    import sys
    assert os.environ.get("DFSATTN_SCORE_PAIRS", "1") != "0", "this test needs the default (pairs on)"
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = (
        "import sys, torch\n"
        f"sys.path.insert(0, {root!r})\n"
        "from dfsattn_b200 import ops\n"
        f"shapes = {_PAIR_SHAPES!r}\n"
        "outs = []\n"
        "for heads, L, D, tile in shapes:\n"
        "    g = torch.Generator(device='cuda').manual_seed(L)\n"
        "    q = torch.randn(heads, L, D, generator=g, device='cuda').bfloat16()\n"
        "    k = torch.randn(heads, L, D, generator=g, device='cuda').bfloat16()\n"
        "    outs.append(ops.block_scores(q, k, L, True, tile=tile).cpu())\n"
        "torch.cuda.synchronize(); ops.check_status('cuda')\n"
        "torch.save(outs, sys.argv[1])\n")
    path = str(tmp_path / "single.pt")
    res = subprocess.run([sys.executable, "-c", code, path], capture_output=True, text=True,
                         env=dict(os.environ, DFSATTN_SCORE_PAIRS="0"), timeout=600)
    assert res.returncode == 0, res.stderr[-3000:]
    single = torch.load(path)
    for (heads, L, D, tile), ref in zip(_PAIR_SHAPES, single):
        g = torch.Generator(device="cuda").manual_seed(L)
        q = torch.randn(heads, L, D, generator=g, device="cuda").bfloat16()
        k = torch.randn(heads, L, D, generator=g, device="cuda").bfloat16()
        got = ops.block_scores(q, k, L, True, tile=tile).cpu()
        assert torch.equal(got, ref), (heads, L, D, tile, float((got - ref).abs().max()))
        want = oracle.block_scores_wan(q.float().cpu()[None], k.float().cpu()[None], torch.arange(L), tile=tile)[0]
        torch.testing.assert_close(got, want, rtol=2e-4, atol=1e-6)
    torch.cuda.synchronize()
    ops.check_status("cuda")


def test_block_scores_rejects_bad_shapes(ops):
    x = torch.zeros(1, 256, 128, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        ops.block_scores(x, x, 256, True, tile=8)
    with pytest.raises(ValueError):
        ops.block_scores(x, x, 129, False)  # [video | gap | text] does not fit in Kb blocks
    with pytest.raises(ValueError):
        ops.block_scores(x.half(), x.half(), 256, True)


@pytest.mark.parametrize("heads,text", [(1, 0), (2, 200)])
def test_block_scores_few_heads_long_sequence(ops, heads, text):
    """Few heads and thousands of key tiles: the logits kernel then cuts the key tiles into several
    ranges per (query tile, head); every range must land in its own columns."""
    from dfsattn_b200.synthetic import structured_qkv
    grid = (5, 16, 64)                                          # 5 120 video tokens: 40 key blocks, 3 column tiles
    q, k, _ = structured_qkv(grid, heads, 128, text_len=text, dtype=torch.float32, device="cpu", seed=3)
    L = q.shape[2]
    video_len = L - text
    perm = torch.randperm(video_len, generator=torch.Generator().manual_seed(1))
    perm = torch.cat([perm, torch.arange(video_len, L)])
    qp, kp = q[0][:, perm].contiguous().cuda(), k[0][:, perm].contiguous().cuda()
    for wan in ((True,) if text == 0 else (False,)):
        got = ops.block_scores(qp, kp, L if wan else video_len, wan).cpu()
        want = (oracle.block_scores_wan(q, k, perm) if wan else oracle.block_scores_hyvideo(q, k, perm, video_len))[0]
        torch.testing.assert_close(got, want, rtol=2e-4, atol=1e-6)
    torch.cuda.synchronize()
    ops.check_status("cuda")
