"""The restated pre-attention step (oracle/prepare.py) against fixtures produced by the
reference's own Wan processor (tests/golden/make_golden_prepare.py), plus its simple identities."""
import numpy as np
import pytest
import torch

from oracle.prepare import qkv_prepare_ref

PREPARE_CASES = ["wan_prepare_96x3x128", "wan_prepare_70x4x64"]


def bf16(a):
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


def load_prepare(golden_dir, name):
    z = np.load(f"{golden_dir}/{name}.npz")
    d = {k: bf16(z[k]) for k in ("q_src", "k_src", "v_src", "gamma_q", "gamma_k", "q", "k", "v")}
    d.update(cos=torch.from_numpy(z["cos"]), sin=torch.from_numpy(z["sin"]), eps=float(z["eps"]),
             heads=int(z["heads"]))
    return d


def assert_within_one_ulp(got, want, max_mismatch=5e-3):
    """bf16 results [.., D]: equal except for a few elements.  The fp32 arithmetic differs in
    detail (fused multiply-add, approximate reciprocal square root), which can move the
    bf16-rounded output of the norm by one unit in the last place; the rotation then mixes an
    element with its pair partner, so the bound is one such unit of the larger of the two."""
    g, w = got.float(), want.float()
    diff = (g - w).abs()
    partner = w.view(*w.shape[:-1], -1, 2).flip(-1).reshape(w.shape)
    bound = torch.maximum(w.abs(), partner.abs()) * 2.0 ** -7 + 1e-30
    assert (diff <= bound).all(), float((diff / bound).max())
    assert float((g != w).float().mean()) <= max_mismatch


@pytest.mark.parametrize("name", PREPARE_CASES)
def test_restatement_matches_the_reference_processor(golden_dir, name):
    d = load_prepare(golden_dir, name)
    q, k, v = qkv_prepare_ref(d["q_src"], d["k_src"], d["v_src"], d["heads"], gamma_q=d["gamma_q"],
                              gamma_k=d["gamma_k"], eps_q=d["eps"], eps_k=d["eps"], norm_across_heads=True,
                              cos=d["cos"], sin=d["sin"])
    assert_within_one_ulp(q, d["q"])
    assert_within_one_ulp(k, d["k"])
    assert torch.equal(v, d["v"])


def test_without_norm_and_rotation_it_is_a_transpose_and_gather():
    g = torch.Generator().manual_seed(5)
    rows, H, D = 37, 3, 64
    src = torch.randn(rows, H * D, generator=g).to(torch.bfloat16)
    perm = torch.randperm(rows, generator=g).to(torch.int32)
    q, k, v = qkv_prepare_ref(src, None, src, H, perm=perm)
    assert k is None
    want = src.view(rows, H, D).permute(1, 0, 2)[:, perm.long()]
    assert torch.equal(q, want) and torch.equal(v, want)


def test_text_rows_are_not_rotated_and_pair_tables_equal_element_tables():
    g = torch.Generator().manual_seed(6)
    rows, H, D, video = 50, 2, 128, 41
    src = torch.randn(rows, H * D, generator=g).to(torch.bfloat16)
    ang = torch.rand(video, D // 2, generator=g) * 6.28
    cos_p, sin_p = ang.cos(), ang.sin()
    cos_e, sin_e = cos_p.repeat_interleave(2, 1), sin_p.repeat_interleave(2, 1)
    a = qkv_prepare_ref(src, src, None, H, cos=cos_p, sin=sin_p)[0]
    b = qkv_prepare_ref(src, src, None, H, cos=cos_e, sin=sin_e)[0]
    assert torch.equal(a, b)
    plain = src.view(rows, H, D).permute(1, 0, 2)
    assert torch.equal(a[:, video:], plain[:, video:]) and not torch.equal(a[:, :video], plain[:, :video])
    # a rotation keeps the length of every pair
    n_in = plain[:, :video].float().view(H, video, D // 2, 2).norm(dim=-1)
    n_out = a[:, :video].float().view(H, video, D // 2, 2).norm(dim=-1)
    assert torch.allclose(n_in, n_out, rtol=2e-2, atol=2e-2)
