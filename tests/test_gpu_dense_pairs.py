"""GPU: the dense call as CTA pairs (two CTAs share every K and V tile, one tcgen05.mma.cta_group::2 over
256 query rows) against dense SDPA and against the single-CTA form of the same kernel, which a child
process runs with DFSATTN_DENSE_PAIRS=0 (the switch is read once per process)."""
import os
import subprocess
import sys

import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# (heads, L, kv_len): even and odd numbers of query blocks (an odd count leaves the last pair with one
# CTA that has no rows), a single block, a partial last block, keys cut off before the end
SHAPES = [(2, 1024, 1024), (3, 1280 + 57, 1280 + 57), (1, 100, 100), (2, 128 * 7, 128 * 5 + 3), (1, 128 * 40 + 1, 128 * 40 + 1)]


def _inputs(heads, L, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return [torch.randn(heads, L, 128, generator=g, device="cuda").bfloat16() for _ in range(3)]


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    assert os.environ.get("DFSATTN_DENSE_PAIRS", "1") != "0", "this module tests the default (pairs on)"
    from dfsattn_b200 import ops as _ops
    return _ops


@pytest.mark.parametrize("heads,L,kv_len", SHAPES)
def test_pairs_equal_dense_sdpa(ops, heads, L, kv_len):
    q, k, v = _inputs(heads, L, L)
    perm = torch.randperm(L, generator=torch.Generator().manual_seed(L)).to(torch.int32).cuda()
    out = ops.block_sparse_fwd(q, k, v, None, None, kv_len=kv_len, out_row_map=perm)
    torch.cuda.synchronize()
    ops.check_status("cuda")
    want = torch.nn.functional.scaled_dot_product_attention(q.float(), k[:, :kv_len].float(), v[:, :kv_len].float())
    got = torch.empty_like(out)
    got[:, torch.arange(L, device="cuda")] = out[:, perm.long()]        # undo the row map
    m = oracle.tensor_metrics(got.float().cpu(), want.cpu())
    assert m["max_abs"] <= 2e-2 and m["cosine"] >= 0.9999, m


def test_pairs_batched_and_token_major(ops):
    heads, L = 2, 128 * 5 + 40
    q, k, v = _inputs(2 * heads, L, 7)                                    # two batch elements
    out = ops.block_sparse_fwd(q, k, v, None, None, batch=2, token_major=True)   # [2, L, H, D]
    torch.cuda.synchronize()
    ops.check_status("cuda")
    want = torch.nn.functional.scaled_dot_product_attention(q.float(), k.float(), v.float()).view(2, heads, L, 128)
    m = oracle.tensor_metrics(out.permute(0, 2, 1, 3).float().cpu(), want.cpu())
    assert m["max_abs"] <= 2e-2 and m["cosine"] >= 0.9999, m


def test_pairs_give_the_bits_of_single_ctas(ops, tmp_path):
    """Same softmax code, same accumulation order per row: the two forms agree bit for bit."""
    code = (
        "import sys, torch\n"
        f"sys.path.insert(0, {ROOT!r})\n"
        "from dfsattn_b200 import ops\n"
        f"shapes = {SHAPES!r}\n"
        "outs = []\n"
        "for heads, L, kv_len in shapes:\n"
        "    g = torch.Generator(device='cuda').manual_seed(L)\n"
        "    q, k, v = [torch.randn(heads, L, 128, generator=g, device='cuda').bfloat16() for _ in range(3)]\n"
        "    outs.append(ops.block_sparse_fwd(q, k, v, None, None, kv_len=kv_len).cpu())\n"
        "torch.cuda.synchronize(); ops.check_status('cuda')\n"
        "torch.save(outs, sys.argv[1])\n")
    path = str(tmp_path / "single.pt")
    env = dict(os.environ, DFSATTN_DENSE_PAIRS="0")
    res = subprocess.run([sys.executable, "-c", code, path], capture_output=True, text=True, env=env, timeout=600)
    assert res.returncode == 0, res.stderr[-3000:]
    single = torch.load(path)
    for (heads, L, kv_len), ref in zip(SHAPES, single):
        q, k, v = _inputs(heads, L, L)
        got = ops.block_sparse_fwd(q, k, v, None, None, kv_len=kv_len).cpu()
        assert torch.equal(got, ref), (heads, L, kv_len, float((got.float() - ref.float()).abs().max()))
    ops.check_status("cuda")
