"""GPU: both classifier-free-guidance passes of a Wan step in one call.

The reference runs the two passes as two calls (its operator refuses a batch,
dfsattn/attention_wan.py:219); the batched call has to leave behind exactly
what those two calls leave: same outputs (bit-identical: every head runs the
same kernel on the same lists), same cached lists, same density records.
"""
import pytest
from conftest import assert_masks_equal_up_to_near_ties
import torch

import oracle
from golden_cases import CASES, inputs

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _fresh():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from dfsattn_b200 import attention_wan as wan
    wan.DFS_Attention.clear_cache()
    wan.DFS_Attention.set_record_density(False)
    wan._dfs_attention_instances.clear()
    yield
    wan.DFS_Attention.clear_cache()
    wan.DFS_Attention.set_record_density(False)
    wan._dfs_attention_instances.clear()


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("token_major", [False, True])
def test_batched_kernel_call_equals_one_call_per_element(D, token_major):
    """dfs_block_sparse_fwd_batched through the C ABI: shared lists, per-element output planes."""
    from dfsattn_b200 import ops
    from dfsattn_b200.engine import BlockLists
    torch.manual_seed(5)
    B, H, L = 2, 3, 700                      # ragged last block
    q, k, v = (torch.randn(B * H, L, D, device="cuda").bfloat16() for _ in range(3))
    kb = -(-L // 128)
    mask = torch.rand(H, kb, kb, device="cuda") > 0.4
    mask[:, :, 0] = True
    mask[1, 2] = False                       # an empty list: zero rows in both elements
    lists = BlockLists.from_bool_mask(mask)
    row_map = torch.randperm(L, device="cuda").to(torch.int32)
    got = ops.block_sparse_fwd(q, k, v, lists.idx, lists.cnt, out_row_map=row_map, token_major=token_major,
                               batch=B)
    assert got.shape == ((B, L, H, D) if token_major else (B, H, L, D))
    for b in range(B):
        sl = slice(b * H, (b + 1) * H)
        want = ops.block_sparse_fwd(q[sl].contiguous(), k[sl].contiguous(), v[sl].contiguous(), lists.idx,
                                    lists.cnt, out_row_map=row_map, token_major=token_major)
        assert torch.equal(got[b], want)
    dense = ops.block_sparse_fwd(q, k, v, None, None, batch=B)
    assert torch.equal(dense[1], ops.block_sparse_fwd(q[H:].contiguous(), k[H:].contiguous(),
                                                      v[H:].contiguous(), None, None))
    torch.cuda.synchronize()
    ops.check_status("cuda")
    with pytest.raises(ValueError):
        ops.block_sparse_fwd(q, k, v, lists.idx.repeat(2, 1, 1), lists.cnt.repeat(2, 1), batch=B)


def _pair_inputs():
    name = "ragged_5x11x17"
    q, k, v, vperm = inputs(name)
    qd, kd, vd = (t.bfloat16().cuda() for t in (q, k, v))
    # second pass: different activations of the same shape
    q2, k2 = kd.clone(), qd.clone()
    v2 = vd.flip(2).contiguous()
    return CASES[name], vperm, (qd, kd, vd), (q2, k2, v2)


@pytest.mark.parametrize("cache_flag", [True, False])
def test_pair_call_equals_two_successive_calls(cache_flag):
    from dfsattn_b200.attention_wan import DFS_Attention, dfs_attention, dfs_attention_cfg_pair
    from dfsattn_b200 import attention_wan as wan
    spec, vperm, a, b = _pair_inputs()
    kw = dict(skip_steps=12, cache_interval=12, layer_idx=2, sparsity=spec["sparsity"], sparsity_dcrt=0.1,
              tile_size=16, block_size=128, video_perm=vperm, cache_flag=cache_flag, record_density=True)
    want, lists_seq, dens_seq = {}, {}, None
    for step in (24, 26):                                   # a refresh step, then a reuse step
        want[step] = torch.cat([dfs_attention(*a, step_idx=step, **kw), dfs_attention(*b, step_idx=step + 1, **kw)])
        lists_seq[step] = {key: e["block_lists"].idx.clone() for key, e in DFS_Attention._cached_metadata.items()}
    dens_seq = {s: dict(d) for s, d in DFS_Attention.density_records.items()}
    DFS_Attention.clear_cache()
    DFS_Attention.set_record_density(False)
    wan._dfs_attention_instances.clear()
    pair = tuple(torch.cat([x, y]) for x, y in zip(a, b))
    for step in (24, 26):
        got = dfs_attention_cfg_pair(*pair, step_idx=step, **kw)
        assert got.shape == want[step].shape and torch.equal(got, want[step])
        now = {key: e["block_lists"].idx for key, e in DFS_Attention._cached_metadata.items()}
        assert now.keys() == lists_seq[step].keys()
        assert all(torch.equal(now[key], lists_seq[step][key]) for key in now)
        tm = dfs_attention_cfg_pair(*pair, step_idx=step, token_major_out=True, **kw)
        assert torch.equal(tm, want[step]) and tm.transpose(1, 2).flatten(2, 3).is_contiguous()
    assert (len(DFS_Attention._cached_metadata) == 1) == cache_flag
    assert {s: dict(d) for s, d in DFS_Attention.density_records.items()} == dens_seq
    assert sorted(dens_seq) == [24, 25, 26, 27]


def test_pair_call_against_the_oracle():
    from dfsattn_b200.attention_wan import DFS_Attention, dfs_attention_cfg_pair
    spec, vperm, a, b = _pair_inputs()
    pair = tuple(torch.cat([x, y]) for x, y in zip(a, b))
    out = dfs_attention_cfg_pair(*pair, step_idx=24, skip_steps=12, cache_interval=12, layer_idx=0,
                                 sparsity=spec["sparsity"], sparsity_dcrt=0.1, tile_size=16, video_perm=vperm)
    (_, entry), = DFS_Attention._cached_metadata.items()
    mask = entry["block_lists"].to_bool_mask().cpu()
    L = a[0].shape[2]
    perm, inv = oracle.build_permutation(vperm, L, L)
    qa, ka = (t.float().cpu() for t in a[:2])
    assert_masks_equal_up_to_near_ties(mask, qa, ka, perm, L, spec["sparsity"], "wan")   # from pass 0 only
    for i, trio in enumerate((a, b)):
        qr, kr, vr = (t.float().cpu() for t in trio)
        m = oracle.tensor_metrics(out[i:i + 1].float().cpu(),
                                  oracle.block_sparse_attention(qr, kr, vr, perm, inv, mask))
        assert m["max_abs"] <= 2e-2 and m["cosine"] >= 0.9999, m


class _FakeAttn(torch.nn.Module):
    def __init__(self, dim, heads):
        super().__init__()
        self.heads = heads
        self.to_q, self.to_k, self.to_v = (torch.nn.Linear(dim, dim) for _ in range(3))
        self.norm_q = torch.nn.RMSNorm(dim, eps=1e-6)
        self.norm_k = torch.nn.RMSNorm(dim, eps=1e-6)
        self.to_out = torch.nn.ModuleList([torch.nn.Linear(dim, dim), torch.nn.Identity()])
        self.add_k_proj = None


@pytest.mark.parametrize("fused", [True, False])
def test_wan_processor_takes_a_batch_of_two_as_the_guidance_pair(fused):
    from dfsattn_b200.replace_wan import Wan_DFSAttn_Processor2_0
    from dfsattn_b200.attention_wan import DFS_Attention
    from dfsattn_b200 import attention_wan as wan
    from dfsattn_b200.order import hilbert3d_perm
    torch.manual_seed(1)
    grid, heads, dim = (3, 8, 16), 2, 128
    V = grid[0] * grid[1] * grid[2]
    attn = _FakeAttn(heads * dim, heads).cuda().bfloat16()
    freqs = torch.polar(torch.ones(V, dim // 2, dtype=torch.float64),
                        torch.rand(V, dim // 2, dtype=torch.float64) * 6.28).cuda()[None, None]
    hs = torch.randn(2, V, heads * dim, device="cuda", dtype=torch.bfloat16)
    make = lambda: Wan_DFSAttn_Processor2_0("dfs", 0.5, 16, 128, hilbert3d_perm(*grid), 1, [0], 1, 1, 0.1, True,
                                            False)
    single, looped, paired = make(), make(), make()
    looped.cfg_pair_batch = False                # same batched projections, one operator call per pass
    for p in (single, looped, paired):
        p.fused_prepare = fused
    want = []
    for step in range(3):                        # denoising steps 0 (dense), 1 (refresh), 2 (refresh)
        want.append(looped(attn, hs, rotary_emb=freqs))
    assert looped.step_idx == 6 and looped.last_call_fused == fused
    DFS_Attention.clear_cache()
    wan._dfs_attention_instances.clear()
    for step in range(3):
        got = paired(attn, hs, rotary_emb=freqs)
        assert paired.step_idx == 2 * (step + 1) and paired.last_call_fused == fused
        assert got.shape == hs.shape and torch.equal(got, want[step])
    # and the batch is what two calls of batch one give (dense step: no near-tie of a selection can
    # tell the differently shaped projection GEMMs apart)
    two = torch.cat([single(attn, hs[0:1], rotary_emb=freqs), single(attn, hs[1:2], rotary_emb=freqs)])
    assert single.step_idx == 2
    m = oracle.tensor_metrics(want[0].detach().float().cpu(), two.detach().float().cpu())
    assert m["cosine"] >= 0.9995 and m["max_abs"] <= 6e-2, m
