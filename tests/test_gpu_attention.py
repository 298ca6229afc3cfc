"""GPU parity of the tcgen05 block-sparse attention kernel and of the
reference-shaped operator API against the CPU oracle and the golden fixtures.

Tolerance (bf16 tensor-core attention vs fp32 oracle): max-abs <= 2e-2 and
cosine >= 0.9999.
"""
import math

import pytest
import torch

import oracle
from golden_cases import CASES, ROW_STRIDE, inputs, load

pytestmark = pytest.mark.gpu

MAX_ABS, MIN_COS = 2e-2, 0.9999


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from dfsattn_b200 import ops as _ops
    return _ops


def _close(got, want, max_abs=MAX_ABS):
    m = oracle.tensor_metrics(got, want)
    assert m["max_abs"] <= max_abs and m["cosine"] >= MIN_COS, m
    return m


# The golden outputs were produced by the reference from the un-rounded fp32
# inputs; the kernel sees those inputs rounded to bf16, which alone moves the
# result by up to ~3e-2 on these structured inputs.  Against them the max-abs
# band is 5e-2 (cosine unchanged); against the oracle on identical bf16-rounded
# inputs the band is the 2e-2 stated above.
GOLDEN_MAX_ABS = 5e-2


def _run(ops, q, k, v, perm, mask, kv_len=None):
    """q,k,v fp32 [1,H,L,D] on CPU -> kernel output [1,H,L,D] fp32 on CPU (un-permuted)."""
    from dfsattn_b200.engine import BlockLists
    qb, kb, vb = (t[0].bfloat16().cuda() for t in (q, k, v))
    pi = perm.to(torch.int32).cuda()
    qp, kp, vp = ops.permute_qkv(qb, kb, vb, pi)
    if mask is None:
        out = ops.block_sparse_fwd(qp, kp, vp, None, None, out_row_map=pi, kv_len=kv_len)
    else:
        lists = BlockLists.from_bool_mask(mask.cuda())
        out = ops.block_sparse_fwd(qp, kp, vp, lists.idx, lists.cnt, out_row_map=pi, kv_len=kv_len)
    torch.cuda.synchronize()
    ops.check_status("cuda")
    return out.float().cpu()[None]


@pytest.mark.parametrize("name", list(CASES))
def test_attention_matches_reference_outputs(ops, name):
    """Kernel vs outputs of the reference's own packed CPU loop (golden)."""
    spec = CASES[name]
    g = load(name)
    q, k, v, vperm = inputs(name)
    L = q.shape[2]
    perm, inv = oracle.build_permutation(vperm, L, L - spec["text"])
    # the oracle sees the same bf16-rounded inputs
    qr, kr, vr = (t.bfloat16().float() for t in (q, k, v))
    mask = torch.from_numpy(g["hy_mask"])
    out = _run(ops, q, k, v, perm, mask)
    _close(out, oracle.block_sparse_attention(qr, kr, vr, perm, inv, mask))
    _close(out, oracle.dense_masked_sdpa(qr, kr, vr, perm, inv, mask))
    # golden = reference on the un-rounded fp32 inputs: same tolerance band
    _close(out[:, :, ::ROW_STRIDE], torch.from_numpy(g["hy_attn"]), GOLDEN_MAX_ABS)
    dense = _run(ops, q, k, v, perm, None)
    _close(dense[:, :, ::ROW_STRIDE], torch.from_numpy(g["dense_attn"]), GOLDEN_MAX_ABS)
    if "wan_mask" in g:
        wmask = torch.from_numpy(g["wan_mask"])
        _close(_run(ops, q, k, v, perm, wmask)[:, :, ::ROW_STRIDE], torch.from_numpy(g["wan_attn"]), GOLDEN_MAX_ABS)


@pytest.mark.parametrize("L,text,D,H", [(640, 0, 128, 2), (700, 100, 128, 3), (333, 77, 64, 2), (128, 0, 64, 1),
                                        (1, 0, 128, 1), (129, 0, 128, 1)])
def test_all_blocks_equals_dense_sdpa_under_permutation(ops, L, text, D, H):
    # reference analogue: top_p=1 equals dense SDPA under a random permutation
    # with a text tail (tests/test_flashinfer64_attention.py:536-563)
    g = torch.Generator().manual_seed(L + D)
    q, k, v = (torch.randn(1, H, L, D, generator=g) for _ in range(3))
    vperm = torch.randperm(L - text, generator=g)
    perm, inv = oracle.build_permutation(vperm, L, L - text)
    kb = math.ceil(L / 128)
    full = torch.ones(H, kb, kb, dtype=torch.bool)
    qr, kr, vr = (t.bfloat16().float() for t in (q, k, v))
    want = torch.nn.functional.scaled_dot_product_attention(qr, kr, vr)
    _close(_run(ops, q, k, v, perm, full), want)
    _close(_run(ops, q, k, v, perm, None), want)


def test_random_ragged_masks_many_tiles(ops):
    """Rows with different list lengths, single-block rows, last partial block."""
    g = torch.Generator().manual_seed(5)
    H, L, D = 2, 128 * 11 + 57, 128
    kb = math.ceil(L / 128)
    q, k, v = (torch.randn(1, H, L, D, generator=g) for _ in range(3))
    mask = torch.rand(H, kb, kb, generator=g) > 0.6
    mask[:, :, 0] |= ~mask.any(-1)      # every row attends something
    mask[0, 3] = False
    mask[0, 3, kb - 1] = True           # a row that only sees the partial block
    mask[1, 5] = True                   # a dense row
    perm, inv = oracle.build_permutation(torch.randperm(L, generator=g), L, L)
    qr, kr, vr = (t.bfloat16().float() for t in (q, k, v))
    _close(_run(ops, q, k, v, perm, mask), oracle.block_sparse_attention(qr, kr, vr, perm, inv, mask))


def test_large_magnitude_scores_exercise_the_rescale_path(ops):
    """Row maxima that keep growing tile after tile force the O rescale."""
    g = torch.Generator().manual_seed(9)
    H, L, D = 1, 128 * 6, 128
    q = torch.randn(1, H, L, D, generator=g)
    k = torch.randn(1, H, L, D, generator=g)
    v = torch.randn(1, H, L, D, generator=g)
    ramp = torch.linspace(0.5, 6.0, L)[None, None, :, None]   # later keys score much higher
    k = k + ramp * q.mean(dim=2, keepdim=True) * 4
    q = q * 3
    perm, inv = oracle.build_permutation(None, L)
    qr, kr, vr = (t.bfloat16().float() for t in (q, k, v))
    want = torch.nn.functional.scaled_dot_product_attention(qr, kr, vr)
    _close(_run(ops, q, k, v, perm, None), want)


@pytest.mark.parametrize("jump", [40.0, 400.0, 4000.0])
def test_scores_far_above_the_reference_move_it(ops, jump):
    """The D = 128 softmax takes its exponentials against the reference maximum of the first tile and moves
    it only when a partial row sum leaves the safe range.  Keys whose scores lie `jump` (raw units, i.e.
    jump * 0.128 in log2 units after scaling) above everything before them: below the bound (exponentials
    up to 2^5 times the reference), above it (2^51 ... and, accumulated over a tile, past the bound), and
    far beyond the range of fp32 (inf in the first pass).  Dense and listed rows, every row against SDPA."""
    g = torch.Generator().manual_seed(int(jump))
    H, L, D = 2, 128 * 5, 128
    q = torch.randn(1, H, L, D, generator=g)
    k = torch.randn(1, H, L, D, generator=g) * 0.1
    v = torch.randn(1, H, L, D, generator=g)
    u = torch.nn.functional.normalize(q.mean(dim=2, keepdim=True), dim=-1)       # a direction most queries like
    q = q + 4 * u
    late = slice(128 * 3 + 17, 128 * 3 + 40)                                      # a few keys in the fourth tile
    k[:, :, late] = k[:, :, late] + u * (jump / 4)                                # q.k grows by about `jump`
    perm, inv = oracle.build_permutation(None, L)
    qr, kr, vr = (t.bfloat16().float() for t in (q, k, v))
    want = torch.nn.functional.scaled_dot_product_attention(qr, kr, vr)
    _close(_run(ops, q, k, v, perm, None), want)                                  # dense call (CTA pairs)
    full = torch.ones(H, 5, 5, dtype=torch.bool)
    _close(_run(ops, q, k, v, perm, full), want)                                  # the same through lists
    torch.cuda.synchronize()
    ops.check_status("cuda")


def test_padded_tail_is_an_independent_segment(ops):
    # reference analogue: tests/test_flashinfer64_attention.py:565-607
    from dfsattn_b200 import engine
    g = torch.Generator().manual_seed(3)
    H, L, valid, D = 2, 500, 420, 128
    q, k, v = (torch.randn(1, H, L, D, generator=g) for _ in range(3))
    qb, kb_, vb = (t[0].bfloat16().cuda() for t in (q, k, v))
    out = engine.run_attention(qb, kb_, vb, None, None, valid).float().cpu()[None]
    qr, kr, vr = (t.bfloat16().float() for t in (q, k, v))
    perm, inv = oracle.build_permutation(None, L)
    full = torch.ones(H, 4, 4, dtype=torch.bool)
    want = oracle.block_sparse_attention(qr, kr, vr, perm, inv, full, valid_len=valid)
    _close(out, want)


def test_linearity_and_scale_invariance_at_size(ops):
    """Size-independent properties on a Wan-480p-sized single head (32 760
    tokens): output is linear in V, and listing all blocks equals dense."""
    g = torch.Generator(device="cuda").manual_seed(11)
    H, L, D = 1, 32760, 128
    q, k, v = (torch.randn(H, L, D, generator=g, device="cuda").bfloat16() for _ in range(3))
    kb = math.ceil(L / 128)
    mask = torch.rand(H, kb, kb, generator=g, device="cuda") > 0.7
    mask[:, :, 0] = True
    from dfsattn_b200.engine import BlockLists
    lists = BlockLists.from_bool_mask(mask)
    o1 = ops.block_sparse_fwd(q, k, v, lists.idx, lists.cnt).float()
    o2 = ops.block_sparse_fwd(q, k, (v.float() * 2).bfloat16(), lists.idx, lists.cnt).float()
    torch.testing.assert_close(o2, 2 * o1, rtol=2e-2, atol=2e-3)
    # pair count of the lists == pair count of the mask (partial last block)
    assert ops.interaction_count(lists.idx, lists.cnt, H, L) == oracle.block_interaction_count(mask.cpu(), L)
    # a strided sample of rows against the fp32 oracle arithmetic on the GPU
    rows = torch.arange(0, L, 997, device="cuda")
    tok = mask[0].repeat_interleave(128, 0).repeat_interleave(128, 1)[:L, :L][rows]
    s = (q[0, rows].float() @ k[0].float().T) * D ** -0.5
    want = torch.softmax(s.masked_fill(~tok, float("-inf")), -1) @ v[0].float()
    m = oracle.tensor_metrics(o1[0, rows].cpu(), want.cpu())
    assert m["max_abs"] <= MAX_ABS and m["cosine"] >= MIN_COS, m
    ops.check_status("cuda")


def test_attention_rejects_bad_arguments(ops):
    x = torch.zeros(1, 128, 128, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        ops.block_sparse_fwd(x.float(), x.float(), x.float(), None, None)
    y = torch.zeros(1, 128, 96, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        ops.block_sparse_fwd(y, y, y, None, None)                 # head_dim 96
    with pytest.raises(ValueError):
        ops.block_sparse_fwd(x, x, x, None, None, kv_len=129)     # kv_len > L
    with pytest.raises(ValueError):
        ops.block_sparse_fwd(x.cpu(), x.cpu(), x.cpu(), None, None)
