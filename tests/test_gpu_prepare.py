"""GPU parity of the fused pre-attention kernel (dfs_qkv_prepare) and of the token-major attention
output (dfs_block_sparse_fwd_ex) against the CPU oracle and the reference-made fixtures."""
import pytest
import torch

from oracle.prepare import qkv_prepare_ref
from test_oracle_prepare import PREPARE_CASES, assert_within_one_ulp, load_prepare

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from dfsattn_b200 import ops as _ops
    return _ops


def cuda(t):
    return None if t is None else t.cuda()


@pytest.mark.parametrize("name", PREPARE_CASES)
def test_matches_the_reference_processor_fixtures(ops, golden_dir, name):
    d = load_prepare(golden_dir, name)
    q, k, v = ops.qkv_prepare(cuda(d["q_src"]), cuda(d["k_src"]), cuda(d["v_src"]), d["heads"],
                              gamma_q=cuda(d["gamma_q"]), gamma_k=cuda(d["gamma_k"]), eps_q=d["eps"],
                              eps_k=d["eps"], norm_across_heads=True, cos=cuda(d["cos"]), sin=cuda(d["sin"]))
    assert_within_one_ulp(q.cpu(), d["q"])
    assert_within_one_ulp(k.cpu(), d["k"])
    assert torch.equal(v.cpu(), d["v"])


@pytest.mark.parametrize("rows,text,H,D,across,pairs", [
    (1191, 256, 3, 128, False, False),   # HunyuanVideo single stream: per-head norm, text last, [S, D] tables
    (1000, 0, 5, 128, True, True),       # Wan: norm over H*D, complex frequencies
    (333, 77, 4, 64, False, True),
    (129, 0, 24, 128, False, False),
    (5, 2, 2, 64, True, False),
])
def test_against_oracle(ops, rows, text, H, D, across, pairs):
    g = torch.Generator().manual_seed(rows + H)
    video = rows - text
    src = [torch.randn(rows, H * D, generator=g).mul(2.0).to(torch.bfloat16) for _ in range(3)]
    gq = (torch.rand(H * D if across else D, generator=g) + 0.5).to(torch.bfloat16)
    gk = (torch.rand(H * D if across else D, generator=g) + 0.5).to(torch.bfloat16)
    ang = torch.rand(video, D // 2, generator=g) * 6.2831853
    cos, sin = ang.cos(), ang.sin()
    if not pairs:
        cos, sin = cos.repeat_interleave(2, 1).contiguous(), sin.repeat_interleave(2, 1).contiguous()
    perm = torch.cat([torch.randperm(video, generator=g), torch.arange(video, rows)]).to(torch.int32)
    want = qkv_prepare_ref(*src, H, gamma_q=gq, gamma_k=gk, eps_q=1e-6, eps_k=1e-5, norm_across_heads=across,
                           cos=cos, sin=sin, rope_rows=video, perm=perm)
    got = ops.qkv_prepare(*(cuda(t) for t in src), H, gamma_q=cuda(gq), gamma_k=cuda(gk), eps_q=1e-6, eps_k=1e-5,
                          norm_across_heads=across, cos=cuda(cos), sin=cuda(sin), rope_rows=video, perm=cuda(perm))
    assert_within_one_ulp(got[0].cpu(), want[0])
    assert_within_one_ulp(got[1].cpu(), want[1])
    assert torch.equal(got[2].cpu(), want[2])


def test_plain_transpose_gather_is_bit_exact_and_partial_inputs_work(ops):
    g = torch.Generator().manual_seed(9)
    rows, H, D = 203, 3, 128
    src = torch.randn(rows, H * D, generator=g).to(torch.bfloat16)
    perm = torch.randperm(rows, generator=g).to(torch.int32)
    q, k, v = ops.qkv_prepare(None, None, src.cuda(), H, perm=perm.cuda())
    assert q is None and k is None
    assert torch.equal(v.cpu(), src.view(rows, H, D).permute(1, 0, 2)[:, perm.long()])


def test_two_calls_assemble_video_and_text_rows(ops):
    # double-stream blocks: text Q/K/V come from their own projections and norm weights
    # (dfsattn/replace_hyvideo.py:292-312)
    g = torch.Generator().manual_seed(10)
    video, text, H, D = 300, 40, 2, 128
    vs = [torch.randn(video, H * D, generator=g).to(torch.bfloat16) for _ in range(3)]
    ts = [torch.randn(text, H * D, generator=g).to(torch.bfloat16) for _ in range(3)]
    gv = [(torch.rand(D, generator=g) + 0.5).to(torch.bfloat16) for _ in range(2)]
    gt = [(torch.rand(D, generator=g) + 0.5).to(torch.bfloat16) for _ in range(2)]
    ang = torch.rand(video, D // 2, generator=g) * 6.28
    cos, sin = ang.cos().repeat_interleave(2, 1).contiguous(), ang.sin().repeat_interleave(2, 1).contiguous()
    perm = torch.randperm(video, generator=g).to(torch.int32)
    out = tuple(torch.zeros(H, video + text, D, dtype=torch.bfloat16, device="cuda") for _ in range(3))
    ops.qkv_prepare(*(cuda(t) for t in vs), H, gamma_q=cuda(gv[0]), gamma_k=cuda(gv[1]), cos=cuda(cos), sin=cuda(sin),
                    perm=cuda(perm), out=out, out_row0=0, out_len=video + text)
    ops.qkv_prepare(*(cuda(t) for t in ts), H, gamma_q=cuda(gt[0]), gamma_k=cuda(gt[1]), out=out, out_row0=video,
                    out_len=video + text)
    wv = qkv_prepare_ref(*vs, H, gamma_q=gv[0], gamma_k=gv[1], cos=cos, sin=sin, perm=perm)
    wt = qkv_prepare_ref(*ts, H, gamma_q=gt[0], gamma_k=gt[1])
    for o, a, b in zip(out, wv, wt):
        assert_within_one_ulp(o.cpu(), torch.cat([a, b], dim=1))


def test_bad_arguments_are_rejected(ops):
    x = torch.zeros(16, 256, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError):
        ops.qkv_prepare(x, x, x, 3)                      # 256 is not a multiple of 3 heads
    with pytest.raises(ValueError):
        ops.qkv_prepare(x, x, x, 8)                      # D = 32 is not supported
    with pytest.raises(ValueError):
        ops.qkv_prepare(x, x, x, 2, gamma_q=torch.ones(64, dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(ValueError):
        ops.qkv_prepare(x.float(), x, x, 2)


@pytest.mark.parametrize("L,H,D", [(1191, 3, 128), (640, 2, 64)])
def test_token_major_output_equals_the_transposed_head_major_output(ops, L, H, D):
    g = torch.Generator().manual_seed(L)
    q, k, v = (torch.randn(H, L, D, generator=g).to(torch.bfloat16).cuda() for _ in range(3))
    kb = -(-L // 128)
    mask = torch.rand(H, kb, kb, generator=g) > 0.4
    mask[:, :, 0] = True
    import oracle
    idx, cnt = oracle.mask_to_index_lists(mask)
    rowmap = torch.randperm(L, generator=g).to(torch.int32).cuda()
    a = ops.block_sparse_fwd(q, k, v, idx.cuda(), cnt.cuda(), out_row_map=rowmap)
    b = ops.block_sparse_fwd(q, k, v, idx.cuda(), cnt.cuda(), out_row_map=rowmap, token_major=True)
    assert b.shape == (L, H, D)
    assert torch.equal(a.permute(1, 0, 2).contiguous(), b)


# ---- the processors' fused path against their unfused (reference-shaped) path -------------------
class _Attn(torch.nn.Module):
    """Duck-typed stand-in for a diffusers Attention block with RMSNorms."""

    def __init__(self, dim, heads, norm_width, added=False):
        super().__init__()
        self.heads = heads
        self.to_q, self.to_k, self.to_v = (torch.nn.Linear(dim, dim) for _ in range(3))
        self.norm_q, self.norm_k = (torch.nn.RMSNorm(norm_width, eps=1e-6) for _ in range(2))
        self.to_out = torch.nn.ModuleList([torch.nn.Linear(dim, dim), torch.nn.Identity()])
        self.add_q_proj = self.add_k_proj = self.add_v_proj = None
        self.norm_added_q = self.norm_added_k = None
        self.to_add_out = None
        if added:
            self.add_q_proj, self.add_k_proj, self.add_v_proj = (torch.nn.Linear(dim, dim) for _ in range(3))
            self.norm_added_q, self.norm_added_k = (torch.nn.RMSNorm(norm_width, eps=1e-6) for _ in range(2))
            self.to_add_out = torch.nn.Linear(dim, dim)
        with torch.no_grad():
            for m in self.modules():
                if isinstance(m, torch.nn.RMSNorm):
                    m.weight.uniform_(0.5, 1.5)


def _reset_operator_state():
    from dfsattn_b200 import attention_hyvideo as hy, attention_wan as wan
    for m in (hy, wan):
        m.DFS_Attention.clear_cache()
        m._dfs_attention_instances.clear()


def _close(a, b, cos_min=0.9995, max_abs=6e-2):
    import oracle
    m = oracle.tensor_metrics(a.detach().float().cpu(), b.detach().float().cpu())
    assert m["cosine"] >= cos_min and m["max_abs"] <= max_abs, m


@pytest.mark.parametrize("added", [False, True])
def test_hyvideo_processor_fused_path_matches_unfused(ops, added):
    from dfsattn_b200.replace_hyvideo import HunyuanVideo_DFSAttn_Processor2_0 as P
    from dfsattn_b200.order import hilbert3d_perm
    torch.manual_seed(1)
    _reset_operator_state()
    grid, text, heads, D = (3, 8, 16), 64, 2, 128
    V = grid[0] * grid[1] * grid[2]
    attn = _Attn(heads * D, heads, D, added=added).cuda().bfloat16()
    hs = torch.randn(1, V, heads * D, device="cuda", dtype=torch.bfloat16)
    enc = torch.randn(1, text, heads * D, device="cuda", dtype=torch.bfloat16)
    am = torch.ones(1, V + text, dtype=torch.bool, device="cuda")
    ang = torch.rand(V, D // 2, device="cuda") * 6.28
    rope = (ang.cos().repeat_interleave(2, 1), ang.sin().repeat_interleave(2, 1))
    args = ("dfs", 0.5, 16, 128, V, hilbert3d_perm(*grid), 3, [], 1, 4, 0.0, True)
    slow, fast = P(*args), P(*args)
    slow.fused_prepare = False
    for step in range(3):   # step 0 dense, step 1 refresh (slow fills the cache, fast reuses it), step 2 cached
        slow.step_idx = fast.step_idx = step
        o1, e1 = slow(attn, hs, enc, attention_mask=am, image_rotary_emb=rope)
        if step == 1:
            fast.step_idx = 2   # same layer, no refresh: the lists the unfused call just stored
        o2, e2 = fast(attn, hs, enc, attention_mask=am, image_rotary_emb=rope)
        assert fast.last_call_fused and not slow.last_call_fused
        assert o2.shape == o1.shape and e2.shape == e1.shape
        _close(o2, o1)
        _close(e2, e1)


def test_wan_processor_fused_path_matches_unfused(ops):
    from dfsattn_b200.replace_wan import Wan_DFSAttn_Processor2_0 as P
    from dfsattn_b200.order import hilbert3d_perm
    torch.manual_seed(2)
    _reset_operator_state()
    grid, heads, D = (2, 8, 16), 2, 128
    V = grid[0] * grid[1] * grid[2]
    attn = _Attn(heads * D, heads, heads * D).cuda().bfloat16()
    hs = torch.randn(1, V, heads * D, device="cuda", dtype=torch.bfloat16)
    ang = torch.rand(V, D // 2, device="cuda", dtype=torch.float64) * 6.28
    freqs = torch.polar(torch.ones_like(ang), ang)[None, None]
    args = ("dfs", 0.5, 16, 128, hilbert3d_perm(*grid), 1, [], 1, 4, 0.0, True, False)
    slow, fast = P(*args), P(*args)
    slow.fused_prepare = False
    for step in (0, 2, 3):   # dense; refresh by the unfused call; the fused call reuses its lists
        slow.step_idx = fast.step_idx = step
        o1 = slow(attn, hs, rotary_emb=freqs)
        if step == 2:
            fast.step_idx = 3
        o2 = fast(attn, hs, rotary_emb=freqs)
        assert fast.last_call_fused and not slow.last_call_fused
        _close(o2, o1)
