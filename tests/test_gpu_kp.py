"""GPU: the "kp" selector -- fine top-p over the 16 x 16-token tiles inside the chosen blocks
(dfsattn/attention_hyvideo.py:211-302, :481-489) -- and the attention kernel restricted to the kept
tiles, against masks made by the reference's own code, the CPU oracle and plain fp32 arithmetic."""
import math
import os

import numpy as np
import pytest
import torch

import oracle
from golden_cases import CASES, GOLDEN, inputs

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _fresh():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from dfsattn_b200 import attention_hyvideo as hy
    hy.DFS_Attention.clear_cache()
    hy.DFS_Attention.set_record_density(False)
    hy._dfs_attention_instances.clear()
    yield
    hy.DFS_Attention.clear_cache()
    hy.DFS_Attention.set_record_density(False)
    hy._dfs_attention_instances.clear()


def _golden_fine(name, tag):
    g = np.load(os.path.join(GOLDEN, "kp_" + name + ".npz"))
    shape = tuple(int(x) for x in g[f"fine_shape_{tag}"])
    return torch.from_numpy(np.unpackbits(g[f"fine_bits_{tag}"])[: int(np.prod(shape))].reshape(shape).astype(bool))


@pytest.mark.parametrize("name", list(CASES))
@pytest.mark.parametrize("tag,p", [("p90", 0.9), ("p50", 0.5)])
def test_tile_maps_match_the_reference_fine_masks(name, tag, p):
    """Same fp32 inputs as the reference saw: the same 16 x 16 mask except where a cumulative score
    sits within rounding of the threshold (a tile or two per case)."""
    from dfsattn_b200 import engine, ops
    spec = CASES[name]
    q, k, v, vperm = inputs(name)
    L = q.shape[2]
    video_len = L - spec["text"]
    perm, _ = oracle.build_permutation(vperm, L, video_len)
    qp, kp = q[0][:, perm].contiguous().cuda(), k[0][:, perm].contiguous().cuda()      # fp32, permuted
    lists = engine.compute_block_lists(qp, kp, video_len, spec["sparsity"], "hyvideo", tile=16, fine_top_p=p)
    torch.cuda.synchronize()
    ops.check_status("cuda")
    assert lists.fine is not None and lists.fine.shape == lists.idx.shape
    got = lists.to_fine_mask(L).cpu()
    want = _golden_fine(name, tag)
    assert got.shape == want.shape
    differ = int((got != want).sum())
    assert differ <= max(2, int(2e-3 * int(want.sum()))), (differ, int(want.sum()))
    # the dense policy is exact: boundary / text columns and rows from the boundary block on
    dfs = min((video_len // 128) * 8, got.shape[1])
    assert bool(got[:, :dfs, dfs:].all()) and bool(got[:, dfs:, :].all())
    # whole blocks at p >= 1: no maps at all
    whole = engine.compute_block_lists(qp, kp, video_len, spec["sparsity"], "hyvideo", tile=16, fine_top_p=1.0)
    assert whole.fine is None and torch.equal(whole.idx, lists.idx)


@pytest.mark.parametrize("D", [64, 128])
def test_kernel_with_random_tile_maps_against_fp32_arithmetic(D):
    from dfsattn_b200 import ops
    from dfsattn_b200.engine import BlockLists
    torch.manual_seed(11)
    H, L = 2, 900                                   # ragged last block
    q, k, v = (torch.randn(H, L, D, device="cuda").bfloat16() for _ in range(3))
    kb = math.ceil(L / 128)
    mask = torch.rand(H, kb, kb, device="cuda") > 0.3
    mask[:, :, 0] = True
    lists = BlockLists.from_bool_mask(mask)
    fine = torch.randint(-2 ** 63, 2 ** 63 - 1, lists.idx.shape, device="cuda", dtype=torch.int64)
    fine &= torch.randint(-2 ** 63, 2 ** 63 - 1, lists.idx.shape, device="cuda", dtype=torch.int64)   # ~25 % kept
    fine[0, 1, :] = 0                               # a query block without any key: zero rows
    fine[1, 2, 0] = -1                              # a whole block
    fine[1, 3, :] &= ~0xFF00                        # query tile 1 of a block row without any key
    lists.fine = fine.contiguous()
    row_map = torch.randperm(L, device="cuda").to(torch.int32)
    for token_major in (False, True):
        got = ops.block_sparse_fwd(q, k, v, lists.idx, lists.cnt, out_row_map=row_map, fine=lists.fine,
                                   token_major=token_major)
        got = got.permute(1, 0, 2) if token_major else got
        torch.cuda.synchronize()
        ops.check_status("cuda")
        tok = lists.to_fine_mask(L).repeat_interleave(16, 1).repeat_interleave(16, 2)[:, :L, :L]
        s = torch.einsum("hqd,hkd->hqk", q.float(), k.float()) * D ** -0.5
        pr = torch.softmax(s.masked_fill(~tok, float("-inf")), -1).nan_to_num(0.0)   # rows without keys: zeros
        want = torch.einsum("hqk,hkd->hqd", pr, v.float())
        unperm = torch.empty_like(want)
        unperm[:, row_map.long()] = want
        m = oracle.tensor_metrics(got.float().cpu(), unperm.cpu())
        assert m["max_abs"] <= 2e-2 and m["cosine"] >= 0.9999, m
        assert float(got[0, row_map[128:256].long()].abs().max()) == 0.0
        assert float(got[1, row_map[3 * 128 + 16:3 * 128 + 32].long()].abs().max()) == 0.0
    with pytest.raises(ValueError):
        ops.block_sparse_fwd(q, k, v, None, None, fine=lists.fine)
    with pytest.raises(ValueError):
        ops.block_sparse_fwd(q, k, v, lists.idx, lists.cnt, fine=lists.fine[:, :, :1].contiguous())


@pytest.mark.parametrize("name", ["hy_text_5x11x17_t256", "ragged_5x11x17", "cfg0_4x16x16"])
def test_dfs_attention_kp_end_to_end(name):
    from dfsattn_b200.attention_hyvideo import DFS_Attention, dfs_attention
    from dfsattn_b200 import ops
    spec = CASES[name]
    q, k, v, vperm = inputs(name)
    L = q.shape[2]
    video_len = L - spec["text"]
    kw = dict(skip_steps=12, cache_interval=12, layer_idx=4, sparsity=spec["sparsity"], sparsity_dcrt=0.05,
              tile_size=16, block_size=128, video_len=video_len, video_perm=vperm, selector_mode="kp",
              fine_top_p=0.9, record_density=True)
    qd, kd, vd = (t.bfloat16().cuda() for t in (q, k, v))
    out = dfs_attention(qd, kd, vd, step_idx=12, **kw)
    ops.check_status("cuda")
    (key, entry), = DFS_Attention._cached_metadata.items()
    assert key[0] == 4 and key[8] == "kp" and key[9] == 0.9
    lists = entry["block_lists"]
    fine = lists.to_fine_mask(L).cpu()
    qr, kr, vr = (t.bfloat16().float() for t in (q, k, v))
    perm, inv = oracle.build_permutation(vperm, L, video_len)
    ref_fine = oracle.fine_mask_hyvideo(qr, kr, perm, video_len, spec["sparsity"], 0.9)
    assert int((fine != ref_fine).sum()) <= max(2, int(2e-3 * int(ref_fine.sum())))
    want = oracle.dense_masked_sdpa(qr, kr, vr, perm, inv, fine, block=16)
    m = oracle.tensor_metrics(out.float().cpu(), want)
    assert m["max_abs"] <= 2e-2 and m["cosine"] >= 0.9999, m
    # density of the 16 x 16 mask, partial last tile included
    size = torch.full((fine.shape[1],), 16.0, dtype=torch.float64)
    size[-1] = L - 16 * (fine.shape[1] - 1)
    pairs = float((fine.double() * size[None, :, None] * size[None, None, :]).sum())
    assert DFS_Attention.density_records[12][4] == pairs / (fine.shape[0] * L * L)
    # a reuse step keeps the maps; the next refresh (other sparsity, other key) replaces the entry
    out2 = dfs_attention(qd, kd, vd, step_idx=13, **kw)
    assert torch.equal(out2, out) and DFS_Attention._cached_metadata[key]["block_lists"] is lists
    dfs_attention(qd, kd, vd, step_idx=24, **kw)
    assert len(DFS_Attention._cached_metadata) == 1 and key not in DFS_Attention._cached_metadata
    # fine_top_p = 1 is the whole-block path
    full = dfs_attention(qd, kd, vd, step_idx=12, **dict(kw, fine_top_p=1.0, layer_idx=5))
    whole = next(e["block_lists"] for kk, e in DFS_Attention._cached_metadata.items() if kk[0] == 5)
    assert whole.fine is None
    m = oracle.tensor_metrics(full.float().cpu(), oracle.dense_masked_sdpa(qr, kr, vr, perm, inv,
                                                                           whole.to_bool_mask().cpu()))
    assert m["max_abs"] <= 2e-2 and m["cosine"] >= 0.9999, m


def test_kp_is_refused_where_it_does_not_apply():
    from dfsattn_b200 import attention_wan
    from dfsattn_b200.attention_hyvideo import dfs_attention
    x = torch.zeros(1, 1, 256, 128, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(TypeError):
        attention_wan.dfs_attention(x, x, x, tile_size=16, selector_mode="kp")      # no such knob on the Wan operator
    with pytest.raises(ValueError):
        dfs_attention(x, x, x, tile_size=32, video_len=256, selector_mode="kp")


class _Attn(torch.nn.Module):
    """Duck-typed stand-in for a diffusers Attention block with per-head RMSNorms."""

    def __init__(self, dim, heads, head_dim):
        super().__init__()
        self.heads = heads
        self.to_q, self.to_k, self.to_v = (torch.nn.Linear(dim, dim) for _ in range(3))
        self.norm_q, self.norm_k = (torch.nn.RMSNorm(head_dim, eps=1e-6) for _ in range(2))
        self.to_out = torch.nn.ModuleList([torch.nn.Linear(dim, dim), torch.nn.Identity()])
        self.add_q_proj = self.add_k_proj = self.add_v_proj = None
        self.norm_added_q = self.norm_added_k = None
        self.to_add_out = None


def test_hyvideo_processor_runs_the_kp_selector_on_both_paths():
    """The processor hands selector_mode / fine_top_p through; its fused path (token-major result, inputs
    already permuted) and its step-by-step path give the same result under the same tile maps."""
    from dfsattn_b200.replace_hyvideo import HunyuanVideo_DFSAttn_Processor2_0 as P
    from dfsattn_b200.attention_hyvideo import DFS_Attention
    from dfsattn_b200.order import hilbert3d_perm
    torch.manual_seed(3)
    grid, text, heads, D = (3, 8, 16), 64, 2, 128
    V = grid[0] * grid[1] * grid[2]
    attn = _Attn(heads * D, heads, D).cuda().bfloat16()
    hs = torch.randn(1, V, heads * D, device="cuda", dtype=torch.bfloat16)
    enc = torch.randn(1, text, heads * D, device="cuda", dtype=torch.bfloat16)
    am = torch.ones(1, V + text, dtype=torch.bool, device="cuda")
    ang = torch.rand(V, D // 2, device="cuda") * 6.28
    rope = (ang.cos().repeat_interleave(2, 1), ang.sin().repeat_interleave(2, 1))
    args = ("dfs", 0.75, 16, 128, V, hilbert3d_perm(*grid), 3, [], 1, 4, 0.0, True)
    slow, fast = (P(*args, selector_mode="kp", fine_top_p=0.8) for _ in range(2))
    slow.fused_prepare = False
    slow.step_idx = 1                           # refresh: lists and tile maps from the step-by-step inputs
    o1, e1 = slow(attn, hs, enc, attention_mask=am, image_rotary_emb=rope)
    (key, entry), = DFS_Attention._cached_metadata.items()
    assert key[8] == "kp" and key[9] == 0.8 and entry["block_lists"].fine is not None
    fine = entry["block_lists"].fine
    assert bool((fine != -1).any())             # something was dropped
    fast.step_idx = 2                           # reuse step: the same maps
    o2, e2 = fast(attn, hs, enc, attention_mask=am, image_rotary_emb=rope)
    assert fast.last_call_fused and not slow.last_call_fused
    for a, b in ((o1, o2), (e1, e2)):
        m = oracle.tensor_metrics(a.detach().float().cpu(), b.detach().float().cpu())
        assert m["cosine"] >= 0.9995 and m["max_abs"] <= 6e-2, m
