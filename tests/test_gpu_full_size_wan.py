"""GPU: the whole path at the two full Wan2.1 shapes of the benchmark configurations (480p: 32 760
tokens, 720p: 75 600 tokens, in Hilbert and in raster order; 40 heads, D = 128, sparsity 0.3; both end in
a ragged block), checked
through properties that do not need a CPU pass over all heads, plus one head's mask against the CPU
oracle and the batched guidance pair against the two calls it stands for."""
import math

import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

HEADS, D, SPARSITY = 40, 128, 0.3
GRIDS = {"wan_480p": (21, 30, 52), "wan_720p": (21, 45, 80), "wan_720p_raster": (21, 45, 80)}


@pytest.fixture(scope="module", params=list(GRIDS))
def full(request):
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    if torch.cuda.get_device_properties(0).total_memory < 60e9:
        pytest.skip("needs the memory of a full-size run")
    from dfsattn_b200 import ops
    from dfsattn_b200 import attention_wan as wan
    from dfsattn_b200.order import hilbert3d_perm
    from dfsattn_b200.synthetic import structured_qkv
    grid = GRIDS[request.param]
    wan.DFS_Attention.clear_cache()
    wan._dfs_attention_instances.clear()
    q, k, v = structured_qkv(grid, HEADS, D, text_len=0, dtype=torch.bfloat16, device="cuda", seed=0)
    vperm = None if request.param.endswith("raster") else hilbert3d_perm(*grid)   # raster: no gather at all
    kw = dict(skip_steps=12, cache_interval=12, layer_idx=0, sparsity=SPARSITY, sparsity_dcrt=0.1,
              tile_size=16, block_size=128, video_perm=vperm)
    out = wan.dfs_attention(q, k, v, step_idx=24, **kw)
    torch.cuda.synchronize()
    ops.check_status("cuda")
    lists = next(iter(wan.DFS_Attention._cached_metadata.values()))["block_lists"]
    yield dict(ops=ops, wan=wan, q=q, k=k, v=v, out=out, lists=lists, vperm=vperm, kw=kw, L=q.shape[2])
    wan.DFS_Attention.clear_cache()
    wan._dfs_attention_instances.clear()


def test_every_row_selects_its_budget_and_pairs_follow_the_partial_edge_rule(full):
    lists, ops, L = full["lists"], full["ops"], full["L"]
    kb = math.ceil(L / 128)
    k_sel = max(1, int(SPARSITY * kb))                 # 76 of 256 / 177 of 591
    assert lists.idx.shape == (HEADS, kb, k_sel) and bool((lists.cnt == k_sel).all())
    assert bool((lists.idx[:, :, 1:] > lists.idx[:, :, :-1]).all()) and int(lists.idx.min()) >= 0
    assert int(lists.idx.max()) < kb
    # selected token pairs with the ragged last query and key block (dfsattn/attention_hyvideo.py:521-546),
    # counted here from the mask itself
    mask = lists.to_bool_mask()
    size = torch.full((kb,), 128.0, device="cuda", dtype=torch.float64)
    size[-1] = L - 128 * (kb - 1)
    pairs = int((mask.double() * size[None, :, None] * size[None, None, :]).sum().item())
    assert ops.interaction_count(lists.idx, lists.cnt, HEADS, L) == pairs


def test_one_head_selects_what_the_oracle_selects(full):
    """Head 0 against the CPU restatement of the reference's scoring and top-k on the same bf16 values:
    the same mask except where two block scores are tied to the last digits at the k-th place."""
    L, lists, ops = full["L"], full["lists"], full["ops"]
    perm, _ = oracle.build_permutation(full["vperm"], L, L)
    qh, kh = (full[n][:, :1].float().cpu() for n in ("q", "k"))
    sums = oracle.block_scores_wan(qh, kh, perm)[0, 0]                 # [Kb, Kb] fp32
    want = oracle.block_mask_wan(qh, kh, perm, SPARSITY)[0]
    got = lists.to_bool_mask()[0].cpu()
    differ = (got != want)
    assert int(differ.sum()) <= 0.1 * got.shape[0] and bool((differ.sum(1) % 2 == 0).all())   # few swaps
    k_sel = int(lists.cnt[0, 0])
    kth = sums.topk(k_sel, dim=-1).values[:, -1:]
    assert bool(((sums - kth).abs()[differ] <= 1e-3 * kth.expand_as(sums)[differ].abs()).all())


def test_softmax_rows_sum_to_one_everywhere(full):
    ones = torch.ones_like(full["v"])
    out = full["wan"].dfs_attention(full["q"], full["k"], ones, step_idx=25, **full["kw"])   # cached lists
    assert float((out.float() - 1).abs().max()) <= 1e-2


def test_sampled_rows_against_fp32_arithmetic(full):
    q, k, v, out, lists, L = (full[n] for n in ("q", "k", "v", "out", "lists", "L"))
    perm, _ = oracle.build_permutation(full["vperm"], L, L)
    perm = perm.cuda()
    mask = lists.to_bool_mask()
    for head in (0, HEADS - 1):
        rows_p = torch.cat([torch.arange(3, L, 2999, device="cuda"), torch.arange(L - 5, L, device="cuda")])
        tok = mask[head][rows_p // 128].repeat_interleave(128, 1)[:, :L]
        qs = q[0, head, perm[rows_p]].float()
        s = (qs @ k[0, head, perm].float().T) * D ** -0.5
        want = torch.softmax(s.masked_fill(~tok, float("-inf")), -1) @ v[0, head, perm].float()
        m = oracle.tensor_metrics(out[0, head, perm[rows_p]].float().cpu(), want.cpu())
        assert m["max_abs"] <= 2e-2 and m["cosine"] >= 0.9999, m


def test_guidance_pair_equals_two_calls(full):
    wan, kw = full["wan"], full["kw"]
    second = tuple(t.flip(1) for t in (full["q"], full["k"], full["v"]))        # other activations, same shape
    want = torch.cat([wan.dfs_attention(full["q"], full["k"], full["v"], step_idx=26, **kw),
                      wan.dfs_attention(*second, step_idx=27, **kw)])
    pair = tuple(torch.cat([a, b]) for a, b in zip((full["q"], full["k"], full["v"]), second))
    del second
    got = wan.dfs_attention_cfg_pair(*pair, step_idx=26, **kw)
    assert torch.equal(got, want)
    assert torch.equal(want[0:1], full["out"])                                   # cached lists, same inputs
