"""GPU: the whole path at the full HunyuanVideo-720p shape of the headline benchmark (119 056 tokens,
24 heads, D = 128, sparsity 0.3), checked through properties that do not need a CPU pass over it."""
import math

import pytest
import torch

import oracle
from oracle.prepare import qkv_prepare_ref

pytestmark = pytest.mark.gpu

GRID, TEXT, HEADS, D, SPARSITY = (33, 45, 80), 256, 24, 128, 0.3
VIDEO = GRID[0] * GRID[1] * GRID[2]
L = VIDEO + TEXT
KB = math.ceil(L / 128)                      # 931 key blocks
DENSE_START = VIDEO // 128                   # 928: first block with a text token
K_SEL = max(1, int(SPARSITY * KB))           # 279 blocks per video row, three of them forced
# selected token pairs per head, from the reference's own counting rule on this shape
PAIRS_PER_HEAD = 928 * 128 * (276 * 128 + 272) + 272 * L


@pytest.fixture(scope="module")
def full():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    if torch.cuda.get_device_properties(0).total_memory < 60e9:
        pytest.skip("needs the memory of a full-size run")
    from dfsattn_b200 import ops
    from dfsattn_b200.attention_hyvideo import DFS_Attention, _dfs_attention_instances, dfs_attention
    from dfsattn_b200.order import hilbert3d_perm
    from dfsattn_b200.synthetic import structured_qkv
    DFS_Attention.clear_cache()
    _dfs_attention_instances.clear()
    q, k, v = structured_qkv(GRID, HEADS, D, text_len=TEXT, dtype=torch.bfloat16, device="cuda", seed=0)
    vperm = hilbert3d_perm(*GRID)
    kw = dict(step_idx=12, skip_steps=12, cache_interval=12, layer_idx=0, sparsity=SPARSITY, sparsity_dcrt=0.1,
              tile_size=16, block_size=128, video_len=VIDEO, video_perm=vperm)
    out = dfs_attention(q, k, v, **kw)
    torch.cuda.synchronize()
    ops.check_status("cuda")
    lists = next(iter(DFS_Attention._cached_metadata.values()))["block_lists"]
    yield dict(ops=ops, q=q, k=k, v=v, out=out, lists=lists, vperm=vperm, kw=kw, attention=dfs_attention)
    DFS_Attention.clear_cache()
    _dfs_attention_instances.clear()


def test_every_row_selects_its_budget_and_the_pair_count_is_the_references(full):
    lists, ops = full["lists"], full["ops"]
    cnt = lists.cnt.cpu()
    assert cnt.shape == (HEADS, KB)
    assert bool((cnt[:, :DENSE_START] == K_SEL).all())          # 276 ranked + 3 forced key blocks
    assert bool((cnt[:, DENSE_START:] == KB).all())             # rows with text tokens are dense
    idx = lists.idx[:, :DENSE_START, :K_SEL]
    assert bool((idx[:, :, 1:] > idx[:, :, :-1]).all())         # ascending, no duplicates
    assert bool((idx[:, :, -3:] == torch.arange(DENSE_START, KB, device=idx.device, dtype=idx.dtype)).all())
    assert ops.interaction_count(lists.idx, lists.cnt, HEADS, L) == HEADS * PAIRS_PER_HEAD


def test_softmax_rows_sum_to_one_everywhere(full):
    # V = 1 turns every output element into its row's softmax mass
    ones = torch.ones_like(full["v"])
    out = full["attention"](full["q"], full["k"], ones, **dict(full["kw"], step_idx=13))   # cached lists
    assert float((out.float() - 1).abs().max()) <= 1e-2


def test_sampled_rows_against_fp32_arithmetic(full):
    q, k, v, out, lists = (full[n] for n in ("q", "k", "v", "out", "lists"))
    perm, inv = oracle.build_permutation(full["vperm"], L, VIDEO)
    perm, inv = perm.cuda(), inv.cuda()
    mask = lists.to_bool_mask()
    for head in (0, 23):
        rows_p = torch.arange(5, L, 4999, device="cuda")            # rows in the permuted order
        tok = mask[head][rows_p // 128].repeat_interleave(128, 1)[:, :L]   # selected keys, permuted order
        qs = q[0, head, perm[rows_p]].float()
        s = (qs @ k[0, head, perm].float().T) * D ** -0.5
        want = torch.softmax(s.masked_fill(~tok, float("-inf")), -1) @ v[0, head, perm].float()
        m = oracle.tensor_metrics(out[0, head, perm[rows_p]].float().cpu(), want.cpu())
        assert m["max_abs"] <= 2e-2 and m["cosine"] >= 0.9999, m


def test_permute_round_trip_is_the_identity(full):
    ops = full["ops"]
    perm, inv = oracle.build_permutation(full["vperm"], L, VIDEO)
    p32, i32 = perm.to(torch.int32).cuda(), inv.to(torch.int32).cuda()
    qp, kp, vp = ops.permute_qkv(full["q"][0], full["k"][0], full["v"][0], p32)
    assert torch.equal(ops.unpermute(qp, i32), full["q"][0])
    assert torch.equal(qp[3, 1000], full["q"][0, 3, int(perm[1000])])


def test_fused_prepare_rows_against_the_oracle_arithmetic(full):
    ops = full["ops"]
    g = torch.Generator(device="cuda").manual_seed(3)
    src = [torch.randn(L, HEADS * D, generator=g, device="cuda").bfloat16() for _ in range(3)]
    gq, gk = ((torch.rand(D, generator=g, device="cuda") + 0.5).bfloat16() for _ in range(2))
    ang = torch.rand(VIDEO, D // 2, generator=g, device="cuda") * 6.2831853
    cos, sin = ang.cos().repeat_interleave(2, 1).contiguous(), ang.sin().repeat_interleave(2, 1).contiguous()
    perm, _ = oracle.build_permutation(full["vperm"], L, VIDEO)
    p32 = perm.to(torch.int32).cuda()
    got = ops.qkv_prepare(*src, HEADS, gamma_q=gq, gamma_k=gk, cos=cos, sin=sin, rope_rows=VIDEO, perm=p32)
    rows = torch.cat([torch.arange(0, L, 3001, device="cuda"), torch.arange(L - 300, L, 37, device="cuda")])
    take = p32[rows].long()                       # their source tokens (the last ones are text: not rotated)
    # the oracle arithmetic on the sampled source rows: a table row per sampled token
    tab = take.clamp(max=VIDEO - 1)
    is_video = (take < VIDEO)
    want = qkv_prepare_ref(*(t[take] for t in src), HEADS, gamma_q=gq, gamma_k=gk, cos=cos[tab], sin=sin[tab])
    plain = qkv_prepare_ref(*(t[take] for t in src), HEADS, gamma_q=gq, gamma_k=gk)
    for t in range(3):
        ref = torch.where(is_video[None, :, None], want[t], plain[t]) if t < 2 else want[t]
        diff = (got[t][:, rows].float() - ref.float()).abs()
        assert float(diff.max()) <= 0.07, float(diff.max())
        assert float((diff > 0).float().mean()) <= 5e-3
    assert torch.equal(got[2][:, rows], want[2])
