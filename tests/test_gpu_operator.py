"""GPU: the reference-shaped operator API (dfs_attention, DFS_Attention, the two
processors): schedule-driven mask caching and end-to-end parity."""
import math

import pytest
from conftest import assert_masks_equal_up_to_near_ties
import torch

import oracle
from golden_cases import CASES, inputs, load

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _fresh():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from dfsattn_b200 import attention_hyvideo as hy, attention_wan as wan
    for m in (hy, wan):
        m.DFS_Attention.clear_cache()
        m.DFS_Attention.set_record_density(False)
        m._dfs_attention_instances.clear()
    yield


def _close(got, want):
    m = oracle.tensor_metrics(got, want)
    assert m["max_abs"] <= 2e-2 and m["cosine"] >= 0.9999, m


@pytest.mark.parametrize("name", ["cfg0_4x16x16", "hy_text_4x12x20_t100", "hy_text_5x11x17_t256",
                                  "ragged_5x11x17", "raster_3x16x16"])
def test_dfs_attention_hyvideo_end_to_end(name):
    from dfsattn_b200.attention_hyvideo import DFS_Attention, dfs_attention
    from dfsattn_b200 import ops
    spec, g = CASES[name], load(name)
    q, k, v, vperm = inputs(name)
    L = q.shape[2]
    video_len = L - spec["text"]
    out = dfs_attention(q.cuda(), k.cuda(), v.cuda(), step_idx=12, skip_steps=12, cache_interval=12,
                        layer_idx=3, sparsity=spec["sparsity"], sparsity_dcrt=0.1, tile_size=16,
                        block_size=128, video_len=video_len, video_perm=vperm, record_density=True)
    assert out.dtype == torch.float32 and out.shape == q.shape
    ops.check_status("cuda")
    (key, entry), = DFS_Attention._cached_metadata.items()
    assert key[0] == 3 and key[4] == spec["sparsity"]
    mask = entry["block_lists"].to_bool_mask().cpu()
    # fp32 inputs are rounded to bf16 before scoring: compare with the oracle on the same values
    qr, kr, vr = (t.bfloat16().float() for t in (q, k, v))
    perm, inv = oracle.build_permutation(vperm, L, video_len)
    assert_masks_equal_up_to_near_ties(mask, qr, kr, perm, video_len, spec["sparsity"], "hyvideo")
    _close(out.cpu(), oracle.block_sparse_attention(qr, kr, vr, perm, inv, mask))
    pairs = oracle.block_interaction_count(mask, L)
    assert DFS_Attention.density_records[12][3] == pairs / (mask.shape[0] * L * L)


def test_dfs_attention_wan_end_to_end_and_cfg_mask_reuse():
    from dfsattn_b200.attention_wan import DFS_Attention, dfs_attention
    name = "ragged_5x11x17"
    spec = CASES[name]
    q, k, v, vperm = inputs(name)
    L = q.shape[2]
    qd, kd, vd = (t.bfloat16().cuda() for t in (q, k, v))
    kw = dict(skip_steps=12, cache_interval=12, layer_idx=1, sparsity=spec["sparsity"], sparsity_dcrt=0.1,
              tile_size=16, block_size=128, video_perm=vperm)
    out = dfs_attention(qd, kd, vd, step_idx=24, **kw)       # first CFG pass of denoising step 12: refresh
    (key, entry), = DFS_Attention._cached_metadata.items()
    assert key == (1, "native", 128, 16, 16)                 # no sparsity term in the Wan key
    lists = entry["block_lists"]
    mask = lists.to_bool_mask().cpu()
    qr, kr, vr = (t.bfloat16().float() for t in (q, k, v))
    perm, inv = oracle.build_permutation(vperm, L, L)
    assert_masks_equal_up_to_near_ties(mask, qr, kr, perm, L, spec["sparsity"], "wan")
    _close(out.float().cpu(), oracle.block_sparse_attention(qr, kr, vr, perm, inv, mask))
    # second CFG pass (odd counter): different inputs, SAME mask object reused
    out2 = dfs_attention(kd, qd, vd, step_idx=25, **kw)
    assert DFS_Attention._cached_metadata[key]["block_lists"] is lists
    _close(out2.float().cpu(), oracle.block_sparse_attention(kr, qr, vr, perm, inv, mask))


def test_mask_cache_follows_the_schedule():
    """Refresh at steps 12/24/36/48 with sparsity 0.9/0.8/0.7/0.6 (float64 drift kept),
    reuse in between; cache_flag=False recomputes every call and stores nothing."""
    from dfsattn_b200.attention_hyvideo import DFS_Attention, dfs_attention
    name = "hy_text_5x11x17_t256"
    spec = CASES[name]
    q, k, v, vperm = inputs(name)
    L = q.shape[2]
    video_len = L - spec["text"]
    qd, kd, vd = (t.bfloat16().cuda() for t in (q, k, v))
    kw = dict(skip_steps=12, cache_interval=12, layer_idx=0, sparsity=0.9, sparsity_dcrt=0.1, tile_size=16,
              block_size=128, video_len=video_len, video_perm=vperm)
    seen = {}
    for step in (12, 13, 23, 24, 30, 36, 47, 48, 49):
        dfs_attention(qd, kd, vd, step_idx=step, **kw)
        flag, cur = oracle.compute_cache_schedule(step, 12, 12, 0.9, 0.1)
        key = next(kk for kk in DFS_Attention._cached_metadata if kk[4] == cur)
        obj = DFS_Attention._cached_metadata[key]["block_lists"]
        if flag:
            assert seen.get(cur) is not obj            # recomputed and stored
        else:
            assert seen[cur] is obj                    # reused
        seen[cur] = obj
        kb = math.ceil(L / 128)
        per_row = int(obj.cnt[0, 0])
        assert per_row == max(1, int(cur * kb))        # int() truncation of the drifting float
    assert len(seen) == 4 and len(DFS_Attention._cached_metadata) == 4   # one entry per sparsity level
    # cache_flag False: nothing stored
    DFS_Attention.clear_cache()
    dfs_attention(qd, kd, vd, step_idx=12, cache_flag=False, **kw)
    assert not DFS_Attention._cached_metadata


def test_unsupported_knobs_raise():
    from dfsattn_b200.attention_hyvideo import dfs_attention
    x = torch.zeros(1, 1, 128, 128, device="cuda", dtype=torch.bfloat16)
    for bad in (dict(sparse_execution="hybrid"), dict(selector_mode="top_p"), dict(block_top_p=0.5),
                dict(selector_mode="kp", tile_size=32), dict(selector_mode="kp", fine_top_p=0.0),
                dict(token_top_k=4), dict(block_size=64), dict(tile_size=8)):
        kw = dict(tile_size=16, video_len=128)
        kw.update(bad)
        with pytest.raises(ValueError):
            dfs_attention(x, x, x, **kw)
    with pytest.raises(ValueError):
        dfs_attention(x, x, x, tile_size=16, video_len=128, cache_interval=0)
    with pytest.raises(ValueError):
        dfs_attention(x.cpu(), x.cpu(), x.cpu(), tile_size=16, video_len=128)


class _FakeAttn(torch.nn.Module):
    """Duck-typed stand-in for a diffusers Attention block."""

    def __init__(self, dim, heads, added=False):
        super().__init__()
        self.heads = heads
        self.to_q, self.to_k, self.to_v = (torch.nn.Linear(dim, dim) for _ in range(3))
        self.norm_q = self.norm_k = None
        self.to_out = torch.nn.ModuleList([torch.nn.Linear(dim, dim), torch.nn.Identity()])
        self.add_q_proj = self.add_k_proj = self.add_v_proj = None
        self.norm_added_q = self.norm_added_k = None
        self.to_add_out = None


def test_hyvideo_processor_gate_counter_and_parity():
    from dfsattn_b200.replace_hyvideo import HunyuanVideo_DFSAttn_Processor2_0
    from dfsattn_b200.attention_hyvideo import DFS_Attention
    from dfsattn_b200.order import hilbert3d_perm
    torch.manual_seed(0)
    grid, text, heads, dim = (3, 8, 16), 64, 2, 128
    V = grid[0] * grid[1] * grid[2]
    attn = _FakeAttn(heads * dim, heads).cuda().bfloat16()
    proc = HunyuanVideo_DFSAttn_Processor2_0("dfs", 0.5, 16, 128, V, hilbert3d_perm(*grid), 7, [], 2, 2, 0.0, True)
    hs = torch.randn(1, V, heads * dim, device="cuda", dtype=torch.bfloat16)
    enc = torch.randn(1, text, heads * dim, device="cuda", dtype=torch.bfloat16)
    am = torch.ones(1, V + text, dtype=torch.bool, device="cuda")
    outs = []
    for step in range(4):
        assert proc.step_idx == step
        assert proc._is_sparse_call() == (step >= 2)
        o, e = proc(attn, hs, enc, attention_mask=am)
        assert o.shape == hs.shape and e.shape == enc.shape
        outs.append(o)
    assert proc.step_idx == 4
    # dense steps equal plain SDPA through the same projections
    x = torch.cat([hs, enc], 1)
    q, k, v = (p(x).unflatten(2, (heads, -1)).transpose(1, 2) for p in (attn.to_q, attn.to_k, attn.to_v))
    ref = torch.nn.functional.scaled_dot_product_attention(q.float(), k.float(), v.float())
    ref = attn.to_out[0](ref.transpose(1, 2).flatten(2, 3).bfloat16()[:, :V])
    m = oracle.tensor_metrics(outs[0].detach().float().cpu(), ref.detach().float().cpu())
    assert m["cosine"] > 0.999, m
    assert len(DFS_Attention._cached_metadata) >= 1
    proc.step_idx = 49
    proc(attn, hs, enc, attention_mask=am)
    assert proc.step_idx == 0          # wraps at 50 like the reference


def test_wan_processor_gate_and_counter():
    from dfsattn_b200.replace_wan import Wan_DFSAttn_Processor2_0
    from dfsattn_b200.order import hilbert3d_perm
    torch.manual_seed(0)
    grid, heads, dim = (2, 8, 16), 2, 128
    V = grid[0] * grid[1] * grid[2]
    attn = _FakeAttn(heads * dim, heads).cuda().bfloat16()
    proc = Wan_DFSAttn_Processor2_0("dfs", 0.5, 16, 128, hilbert3d_perm(*grid), 1, [0], 1, 1, 0.1, True, False)
    hs = torch.randn(1, V, heads * dim, device="cuda", dtype=torch.bfloat16)
    gates = []
    for step in range(4):
        gates.append(proc._gate())
        out = proc(attn, hs)
        assert out.shape == hs.shape
    assert gates == ["dense", "dense", "sparse", "sparse"]   # two calls per denoising step
    cross = Wan_DFSAttn_Processor2_0("dfs", 0.5, 16, 128, None, 1, [0], 1, 1, 0.1, True, True)
    assert cross._gate() == "dense"
    with pytest.raises(ValueError):
        Wan_DFSAttn_Processor2_0("dfs", 0.5, 16, 128, None, 1, [0], 1, 1, 0.1, True, False,
                                 sparse_execution="flex64")


def test_host_buffer_entry_point_matches_device_call():
    from dfsattn_b200.attention_hyvideo import dfs_attention
    from dfsattn_b200.host_io import dfs_attention_host
    name = "hy_text_5x11x17_t256"
    spec = CASES[name]
    q, k, v, vperm = inputs(name)
    L = q.shape[2]
    kw = dict(step_idx=12, skip_steps=12, cache_interval=12, sparsity=spec["sparsity"], sparsity_dcrt=0.1,
              tile_size=16, block_size=128, video_len=L - spec["text"], video_perm=vperm)
    qh, kh, vh = (t.bfloat16().pin_memory() for t in (q, k, v))
    want = dfs_attention(qh.cuda(), kh.cuda(), vh.cuda(), layer_idx=5, **kw).cpu()
    got = dfs_attention_host(qh, kh, vh, head_groups=2, layer_idx=6, **kw)
    torch.cuda.synchronize()
    assert got.is_pinned() and got.shape == want.shape
    assert torch.equal(got, want)       # heads are independent: grouping them changes nothing
    with pytest.raises(ValueError):
        dfs_attention_host(qh.cuda(), kh.cuda(), vh.cuda(), **kw)
    # enough heads for the ramp (single heads at both ends, uneven groups in between)
    q12, k12, v12 = (torch.cat([t, t.flip(2), t * 0.5, -t], 1).contiguous().pin_memory()
                     for t in (qh, kh, vh))
    assert q12.shape[1] == 12
    want = dfs_attention(q12.cuda(), k12.cuda(), v12.cuda(), layer_idx=7, **kw).cpu()
    got = dfs_attention_host(q12, k12, v12, head_groups=7, layer_idx=8, **kw)
    torch.cuda.synchronize()
    assert torch.equal(got, want)
