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
    assert bool((cnt[:, DENSE_START:] == -1).all())             # rows with text tokens attend every block
    assert lists.idx.shape[-1] == K_SEL                         # lists as long as a video row needs
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


def test_dense_call_at_full_size(full):
    """The dense call of the warm-up steps on the full shape (466 CTA pairs per head; the last pair has
    one CTA without rows): softmax mass one on every row, sampled rows against fp32 arithmetic."""
    from dfsattn_b200.fullattention import full_attention
    q, k, v = full["q"], full["k"], full["v"]
    ones = full_attention(q, k, torch.ones_like(v), mode="flash")
    assert float((ones.float() - 1).abs().max()) <= 1e-2
    del ones
    out = full_attention(q, k, v, mode="flash")
    torch.cuda.synchronize()
    full["ops"].check_status("cuda")
    rows = torch.cat([torch.arange(3, L, 7001, device="cuda"), torch.arange(L - 260, L, 41, device="cuda")])
    for head in (0, 11, 23):
        s = (q[0, head, rows].float() @ k[0, head].float().T) * D ** -0.5
        want = torch.softmax(s, -1) @ v[0, head].float()
        m = oracle.tensor_metrics(out[0, head, rows].float().cpu(), want.cpu())
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


def test_kp_tile_maps_at_full_size(full):
    """The kp selector on the full shape: dense policy exact, every refined pair keeps a top set of its
    64 tile scores whose mass just reaches fine_top_p (checked for whole query-block rows against fp32
    arithmetic on the pooled means), and the attention under the maps still has softmax mass one."""
    from dfsattn_b200 import engine
    ops, q, k = full["ops"], full["q"], full["k"]
    P = 0.9
    perm, _ = oracle.build_permutation(full["vperm"], L, VIDEO)
    p32 = perm.to(torch.int32).cuda()
    qp, kp, vp = ops.permute_qkv(q[0], k[0], torch.ones_like(q[0]), p32)
    lists = engine.compute_block_lists(qp, kp, VIDEO, SPARSITY, "hyvideo", tile=16, fine_top_p=P)
    assert torch.equal(lists.idx, full["lists"].idx) and lists.fine.shape == lists.idx.shape
    fine = lists.fine
    assert lists.fine.shape[-1] == K_SEL                                   # no slots beyond a video row's budget
    assert bool((fine[:, :DENSE_START, K_SEL - 3:K_SEL] == -1).all())      # forced text / boundary columns
    refined = fine[:, :DENSE_START, :K_SEL - 3]
    assert bool((refined != 0).all())                                      # the largest tile always stays
    shifts = torch.arange(64, device="cuda", dtype=torch.int64)
    scale = D ** -0.5
    for head, qb in ((0, 0), (7, 411), (23, DENSE_START - 1)):
        # pooled fp32 means of this query block and of all keys (scoring layout: video | gap | text)
        qm = qp[head, qb * 128:(qb + 1) * 128].float().view(8, 16, D).mean(1)
        kv = torch.zeros((KB * 128, D), device="cuda")
        kv[:VIDEO] = kp[head, :VIDEO].float()
        kv[(DENSE_START + 1) * 128:(DENSE_START + 1) * 128 + TEXT] = kp[head, VIDEO:].float()
        km = kv.view(KB * 8, 16, D).mean(1)
        score = torch.softmax((qm @ km.T) * scale, -1).view(8, KB, 8)       # [q tile, key block, key tile]
        blocks = lists.idx[head, qb, :K_SEL - 3].long()
        vals = score[:, blocks].permute(1, 0, 2).reshape(-1, 64)            # [pair, 8 * i + j]
        keep = ((refined[head, qb, :, None] >> shifts) & 1).bool()
        total = vals.sum(-1)
        kept_mass = (vals * keep).sum(-1)
        smallest_kept = vals.masked_fill(~keep, float("inf")).min(-1).values
        largest_dropped = vals.masked_fill(keep, 0.0).max(-1).values
        tol = 1e-4 * total
        assert bool((smallest_kept + tol >= largest_dropped).all())         # a top set
        assert bool((kept_mass + tol >= P * total).all())                   # reaches the mass ...
        assert bool((kept_mass - smallest_kept - tol < P * total).all())    # ... and not with one tile less
    out = ops.block_sparse_fwd(qp, kp, vp, lists.idx, lists.cnt, out_row_map=p32, fine=lists.fine)
    assert float((out.float() - 1).abs().max()) <= 1e-2
    ops.check_status("cuda")
