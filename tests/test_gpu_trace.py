"""GPU: a scaled-down mask-caching trace (denoising steps x layers with drifting
Q/K) through the HunyuanVideo and Wan operators: which steps are dense, which
refresh the lists, which reuse them, with the sparsity decrement -- checked step
by step against the oracle's schedule and masks."""
import math

import pytest
from conftest import assert_masks_equal_up_to_near_ties
import torch

import oracle
from dfsattn_b200.synthetic import drift, structured_qkv

pytestmark = pytest.mark.gpu


def _close(got, want):
    m = oracle.tensor_metrics(got, want)
    assert m["max_abs"] <= 2e-2 and m["cosine"] >= 0.9999, m


def test_hunyuan_trace_small():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from dfsattn_b200.attention_hyvideo import DFS_Attention, _dfs_attention_instances, dfs_attention
    from dfsattn_b200.fullattention import full_attention
    from dfsattn_b200.order import hilbert3d_perm
    DFS_Attention.clear_cache()
    _dfs_attention_instances.clear()
    grid, text, heads, dim = (4, 12, 20), 224, 2, 128       # L = 1184: 7 video blocks + boundary + text
    layers, steps, skip, interval, s0, dcrt = 2, 16, 4, 4, 0.9, 0.1
    vperm = hilbert3d_perm(*grid)
    V = grid[0] * grid[1] * grid[2]
    L = V + text
    perm, inv = oracle.build_permutation(vperm, L, V)
    state = []
    for layer in range(layers):       # step-0 inputs: seed = layer index
        q, k, v = structured_qkv(grid, heads, dim, text_len=text, dtype=torch.bfloat16, device="cuda", seed=layer)
        state.append([q, k, v])
    refreshes = 0
    for step in range(steps):
        flag, cur = oracle.compute_cache_schedule(step, skip, interval, s0, dcrt)
        for layer in range(layers):
            q, k, v = state[layer]
            if step < skip:       # dense warm-up steps of the schedule
                out = full_attention(q, k, v, mode="flash")
                if layer == 0 and step == 0:
                    want = torch.nn.functional.scaled_dot_product_attention(q.float(), k.float(), v.float())
                    _close(out.float().cpu(), want.cpu())
            else:
                before = dict(DFS_Attention._cached_metadata)
                out = dfs_attention(q, k, v, step_idx=step, skip_steps=skip, cache_interval=interval,
                                    layer_idx=layer, sparsity=s0, sparsity_dcrt=dcrt, tile_size=16,
                                    block_size=128, video_len=V, video_perm=vperm)
                key = next(kk for kk in DFS_Attention._cached_metadata if kk[0] == layer and kk[4] == cur)
                lists = DFS_Attention._cached_metadata[key]["block_lists"]
                if flag:
                    refreshes += 1
                    assert before.get(key, {}).get("block_lists") is not lists       # recomputed
                    qc, kc = q.float().cpu(), k.float().cpu()
                    assert_masks_equal_up_to_near_ties(lists.to_bool_mask().cpu(), qc, kc, perm, V, cur, "hyvideo")
                    assert int(lists.cnt[0, 0]) == max(1, int(cur * math.ceil(L / 128)))
                else:
                    assert before[key]["block_lists"] is lists                      # reused
                if layer == 1 and step in (skip, steps - 1):
                    want = oracle.block_sparse_attention(q.float().cpu(), k.float().cpu(), v.float().cpu(), perm,
                                                         inv, lists.to_bool_mask().cpu())
                    _close(out.float().cpu(), want)
            # drift of Q and K for the next step
            state[layer][0] = drift(q, step * 100 + layer * 2)
            state[layer][1] = drift(k, step * 100 + layer * 2 + 1)
    expected = sum(1 for st in range(skip, steps) if oracle.compute_cache_schedule(st, skip, interval, s0, dcrt)[0])
    assert refreshes == expected * layers
    from dfsattn_b200 import ops
    ops.check_status("cuda")
    DFS_Attention.clear_cache()


def test_timing_recorder_phases(tmp_path):
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from dfsattn_b200.attention_hyvideo import DFS_Attention, _dfs_attention_instances, dfs_attention
    DFS_Attention.clear_cache()
    _dfs_attention_instances.clear()
    DFS_Attention.set_record_timing(True)
    q, k, v = structured_qkv((2, 8, 16), 2, 128, dtype=torch.bfloat16, device="cuda", seed=3)
    kw = dict(skip_steps=12, cache_interval=12, layer_idx=0, sparsity=0.5, sparsity_dcrt=0.1, tile_size=16,
              block_size=128, video_len=256, video_perm=None)
    dfs_attention(q, k, v, step_idx=12, **kw)     # refresh: all three phases
    dfs_attention(q, k, v, step_idx=13, **kw)     # cached: attention only
    raw = DFS_Attention.timing_recorder.summary()
    assert raw["topk_mask"]["calls"] == 1 and raw["topk_routing"]["calls"] == 1
    summary = DFS_Attention.dump_timing_records(str(tmp_path / "timing.csv"), extra_totals={"wall": 1.0})
    DFS_Attention.set_record_timing(False)
    # the written table: the reference's columns and categories (dfsattn/utils/timing.py:140-200)
    assert summary["attention_execution"]["calls"] == 2 and summary["top_k_selection"]["calls"] == 1
    assert summary["wall"] == {"calls": 1.0, "total_ms": 1.0, "mean_ms": 1.0}
    lines = (tmp_path / "timing.csv").read_text().splitlines()
    assert lines[0] == "phase,total_ms,calls,mean_ms"
    assert [ln.split(",")[0] for ln in lines[1:]] == ["top_k_selection", "attention_execution", "wall"]
    DFS_Attention.clear_cache()
