"""CPU: the C-ABI library loads, exports every symbol the header declares, and
its host-only entry points (no GPU needed) agree with the oracle."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

import oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    from dfsattn_b200 import _lib
    header = open(os.path.join(ROOT, "include", "dfs_b200.h")).read()
    declared = set(re.findall(r"\b(dfs_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    assert declared == set(_lib.SIGNATURES), (declared ^ set(_lib.SIGNATURES))
    raw = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared:
        assert hasattr(raw, name), name
    assert _lib.lib.dfs_version() == 1
    assert b"aligned" in _lib.lib.dfs_status_string(-2)


def test_missing_library_fails_loudly(tmp_path, monkeypatch):
    from dfsattn_b200 import _lib
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(_lib.DfsLibraryError):
        _lib._load()


def test_schedule_entry_point_matches_reference_tables(golden_dir):
    from dfsattn_b200.attention_hyvideo import _compute_cache_schedule
    g = np.load(golden_dir + "/schedule.npz")
    i = 0
    while f"params_{i}" in g:
        skip, interval, s, dcrt, steps = g[f"params_{i}"]
        for step in range(int(steps)):
            flag, val = _compute_cache_schedule(step, int(skip), int(interval), float(s), float(dcrt))
            assert flag == bool(g[f"flags_{i}"][step]) and val == float(g[f"vals_{i}"][step])
        i += 1
    with pytest.raises(ValueError):
        _compute_cache_schedule(0, 0, 0, 0.3, 0.1)


def test_interaction_count_entry_point_handles_partial_edges():
    # reference analogue: tests/test_flashinfer64_attention.py:95-120
    from dfsattn_b200 import ops
    torch.manual_seed(38)
    for L in (193, 256, 1191):
        kb = -(-L // 128)
        mask = torch.rand(2, kb, kb) > 0.5
        idx, cnt = oracle.mask_to_index_lists(mask)
        if idx.shape[-1] == 0:
            continue
        assert ops.interaction_count(idx, cnt, 2, L) == oracle.block_interaction_count(mask, L)
        assert ops.interaction_count(None, None, 2, L) == 2 * L * L


def test_cpu_tensors_are_rejected_not_computed():
    from dfsattn_b200 import ops
    x = torch.zeros(1, 128, 128, dtype=torch.bfloat16)
    p = torch.arange(128, dtype=torch.int32)
    with pytest.raises(ValueError):
        ops.permute_qkv(x, x, x, p)
    with pytest.raises(ValueError):
        ops.block_scores(x, x, 128, True)
    with pytest.raises(ValueError):
        ops.block_sparse_fwd(x, x, x, None, None)


def test_processor_constructors_keep_the_reference_argument_order():
    from dfsattn_b200.replace_hyvideo import HunyuanVideo_DFSAttn_Processor2_0 as HP
    from dfsattn_b200.replace_wan import Wan_DFSAttn_Processor2_0 as WP
    hp = HP("dfs", 0.3, 16, 128, 1024, None, 5, [0], 12, 12, 0.1, True)
    assert (hp.layer_idx, hp.video_len, hp.skip_steps, hp.cache_flag, hp.step_idx) == (5, 1024, 12, True, 0)
    wp = WP("dfs", 0.3, 16, 128, None, 4, [0], 12, 12, 0.1, True, False)
    assert (wp.layer_idx, wp.cross_flag, wp.dense_step_idx) == (4, False, -1)
    # the gate follows step and layer
    hp.step_idx = 11
    assert not hp._is_sparse_call()
    hp.step_idx = 12
    assert hp._is_sparse_call()
    hp.skip_layers = [5]
    assert not hp._is_sparse_call()
    for bad in (dict(sparse_execution="flashinfer64"), dict(selector_mode="top_p"), dict(token_top_k=8)):
        with pytest.raises(ValueError):
            HP("dfs", 0.3, 16, 128, 1024, None, 5, [0], 12, 12, 0.1, True, **bad)
    kp = HP("dfs", 0.3, 16, 128, 1024, None, 5, [0], 12, 12, 0.1, True, selector_mode="kp", fine_top_p=0.8)
    assert (kp.selector_mode, kp.fine_top_p) == ("kp", 0.8)
    with pytest.raises(ValueError):      # the tile maps are 8 x 8: 16-token tiles only
        HP("dfs", 0.3, 32, 128, 1024, None, 5, [0], 12, 12, 0.1, True, selector_mode="kp")
    with pytest.raises(ValueError):
        HP("dfs", 0.3, 8, 128, 1024, None, 5, [0], 12, 12, 0.1, True)   # tile sizes: 16, 32, 64


def test_sharded_entry_points_reject_bad_tables_before_any_launch():
    # nothing is launched for rejected arguments, so this runs without a GPU
    from dfsattn_b200 import _lib, ops
    lib = _lib.lib
    tab = ops.ShardTable([0x1000, 0x2000], shard_rows=64, stride_rows=64)
    assert tab.world == 2
    # null output
    assert lib.dfs_permute_qkv_sharded(tab.array, tab.array, tab.array, 2, 64, 64, 0, None, None, None, None,
                                       1, 100, 256, None) == -1
    # shards do not cover the sequence
    assert lib.dfs_permute_qkv_sharded(tab.array, tab.array, tab.array, 2, 64, 64, 0, None, 0x3000, 0x4000, 0x5000,
                                       1, 200, 256, None) == -5
    # more shards than the table type holds
    assert lib.dfs_permute_qkv_sharded(tab.array, tab.array, tab.array, 9, 64, 64, 0, None, 0x3000, 0x4000, 0x5000,
                                       1, 100, 256, None) == -5
    # a misaligned shard pointer
    bad = ops.ShardTable([0x1000, 0x2008], shard_rows=64, stride_rows=64)
    assert lib.dfs_permute_qkv_sharded(bad.array, tab.array, tab.array, 2, 64, 64, 0, None, 0x3000, 0x4000, 0x5000,
                                       1, 100, 256, None) == -2
    assert lib.dfs_block_sparse_fwd_sharded(0x1000, 0x1000, 0x1000, None, None, 0, None, None, 2, 64, 64, 0, 1,
                                            100, 100, 128, 0.1, None, None) == -1
    assert lib.dfs_block_sparse_fwd_sharded(0x1000, 0x1000, 0x1000, None, None, 0, None, tab.array, 2, 32, 32, 0,
                                            1, 100, 100, 128, 0.1, None, None) == -5


def test_batched_attention_entry_point_rejects_bad_arguments_before_any_launch():
    from dfsattn_b200 import _lib, ops
    lib = _lib.lib
    args = lambda batch, heads, q=0x1000: (q, 0x2000, 0x3000, None, None, 0, None, 0x4000, 0, batch, heads,
                                           256, 256, 128, 0.1, None, None)
    assert lib.dfs_block_sparse_fwd_batched(*args(0, 2)) == -3          # no batch element
    assert lib.dfs_block_sparse_fwd_batched(*args(2, 0)) == -3          # no heads
    assert lib.dfs_block_sparse_fwd_batched(*args(2, 40000)) == -3      # more grid rows than a launch has
    assert lib.dfs_block_sparse_fwd_batched(*args(2, 2, q=None)) == -1  # null input
    assert lib.dfs_block_sparse_fwd_batched(*args(2, 2, q=0x1008)) == -2
    x = torch.zeros(3, 128, 128, dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        ops.block_sparse_fwd(x, x, x, None, None, batch=2)              # CPU tensors; 3 is not 2 * heads


def test_wan_processor_counts_a_batch_of_two_as_both_guidance_passes():
    from dfsattn_b200.replace_wan import Wan_DFSAttn_Processor2_0 as WP
    wp = WP("dfs", 0.3, 16, 128, None, 4, [0], 12, 12, 0.1, True, False)
    wp.step_idx = 98
    wp._advance(2)
    assert wp.step_idx == 0                      # wraps at 100 like two single calls
    wp.step_idx = 25
    q = torch.zeros(2, 1, 128, 64)
    with pytest.raises(ValueError):
        wp._attend_self(q, q, q)                 # a pair cannot straddle two denoising steps
    with pytest.raises(AssertionError):
        wp._attend_self(torch.zeros(3, 1, 128, 64), q, q)


def test_host_entry_point_head_groups_cover_every_head_once():
    from dfsattn_b200.host_io import group_bounds
    for heads, groups in ((24, 12), (40, 12), (3, 12), (10, 6), (24, 4), (7, 7), (5, 1), (1, 1)):
        for ramp in (True, False):
            b = group_bounds(heads, groups, ramp)
            assert b[0][0] == 0 and b[-1][1] == heads and len(b) == min(groups, heads)
            assert all(x[1] == y[0] for x, y in zip(b, b[1:])) and all(h1 > h0 for h0, h1 in b)
    sizes = [h1 - h0 for h0, h1 in group_bounds(24, 12)]
    assert sizes[:3] == [1, 1, 1] and sizes[-2:] == [1, 1]      # short first upload, short last download
    assert [h1 - h0 for h0, h1 in group_bounds(24, 12, ramp=False)] == [2] * 12


def test_fine_selector_entry_points_reject_bad_arguments_before_any_launch():
    from dfsattn_b200 import _lib
    lib = _lib.lib
    ws, idx, cnt, bits = 0x10000, 0x20000, 0x30000, 0x40000
    ok = dict(workspace=ws, nbytes=1 << 30, heads=2, L=1024, V=1024, D=128, tile=16, block=128, wan=0, idx=idx,
              cnt=cnt, kmax=4, q_rows=8, n_rank=8, dense=8, p=0.9, bits=bits)

    def call(**kw):
        a = dict(ok, **kw)
        return lib.dfs_fine_top_p(a["workspace"], a["nbytes"], a["heads"], a["L"], a["V"], a["D"], a["tile"],
                                  a["block"], a["wan"], a["idx"], a["cnt"], a["kmax"], a["q_rows"], a["n_rank"],
                                  a["dense"], a["p"], a["bits"], None)
    assert call(idx=None) == -1 and call(bits=None) == -1 and call(workspace=None) == -1
    assert call(workspace=ws + 16) == -2 and call(bits=bits + 4) == -2
    assert call(tile=32) == -3                      # the maps are 8 x 8: 16-token tiles only
    assert call(nbytes=1024) == -6                  # not the scratch of this shape
    assert call(kmax=0) == -5 and call(q_rows=7) == -5 and call(n_rank=9) == -5 and call(p=0.0) == -5
    # attention with maps: maps need lists, and 8-byte alignment
    f = lambda idx_, cnt_, fine_: lib.dfs_block_sparse_fwd_fine(0x1000, 0x2000, 0x3000, idx_, cnt_, fine_, 4, None,
                                                                0x4000, 0, 2, 256, 256, 128, 0.1, None, None)
    assert f(idx, cnt, None) == -1 and f(None, None, bits) == -1 and f(idx, cnt, bits + 4) == -2


def test_pair_count_under_tile_maps_equals_the_count_on_the_expanded_mask():
    """Host logic of the kp density record: counting from the 64-bit maps (whole blocks with their
    true sizes, refined pairs 256 per bit) against the 16 x 16 mask built out of the same maps."""
    import math
    from dfsattn_b200.engine import BlockLists
    torch.manual_seed(0)
    for L in (1000, 1024, 935):
        kb = math.ceil(L / 128)
        mask = torch.rand(2, kb, kb) > 0.4
        mask[:, :, 0] = True
        lists = BlockLists.from_bool_mask(mask)
        dense_start = L // 128
        fine = torch.randint(-2 ** 63, 2 ** 63 - 1, lists.idx.shape, dtype=torch.int64)
        refined = (torch.arange(kb)[None, :, None] < dense_start) & (lists.idx < dense_start) & (lists.idx >= 0)
        lists.fine = torch.where(refined, fine, torch.full_like(fine, -1))
        lists.fine[0, 0, 0] = -1                      # a refined pair that kept every tile
        fm = lists.to_fine_mask(L)
        size = torch.full((fm.shape[1],), 16.0, dtype=torch.float64)
        size[-1] = L - 16 * (fm.shape[1] - 1)
        want = int((fm.double() * size[None, :, None] * size[None, None, :]).sum().item())
        assert lists.fine_pair_count(L) == want
