"""Golden fixtures for the fused pre-attention step, from the REFERENCE's own Wan processor.

    python tests/golden/make_golden_prepare.py /path/to/reference

The reference's ``Wan_DFSAttn_Processor2_0.__call__`` (``dfsattn/replace_wan.py:135-324``) is run
on CPU in bf16 with mode="flash", which takes its PyTorch fallback for the RMSNorm and for the
rotary embedding; the dense attention call it would make next is replaced by a recorder, so the
fixture holds exactly the Q/K/V tensors [1, H, L, D] the reference hands to its attention.  The
``attn`` object is a stand-in with fixed projections, a ``torch.nn.RMSNorm`` over H*D (what the Wan
transformer uses) and identity output layers.  ``diffusers`` is not installed here; the reference
imports one class name from it for a type annotation only, which this script satisfies with an
empty placeholder module.  Only inputs and outputs are stored, no reference source.
"""
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

CASES = {
    # name: tokens, heads, head_dim
    "wan_prepare_96x3x128": (96, 3, 128),
    "wan_prepare_70x4x64": (70, 4, 64),
}


def u16(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def main():
    if len(sys.argv) < 2:
        raise SystemExit(f"usage: python {sys.argv[0]} <checkout of codesiena/DFSattn>")
    ref_root = sys.argv[1]
    sys.path.insert(0, ref_root)
    for name in ("diffusers", "diffusers.models", "diffusers.models.attention_processor"):
        sys.modules.setdefault(name, types.ModuleType(name))
    sys.modules["diffusers.models.attention_processor"].Attention = type("Attention", (), {})
    from dfsattn import replace_wan

    captured = {}

    def recorder(q, k, v, **kwargs):
        captured["qkv"] = (q.clone(), k.clone(), v.clone())
        return q

    replace_wan.full_attention = recorder

    for name, (L, H, D) in CASES.items():
        g = torch.Generator().manual_seed(len(name))
        proj = [torch.randn(1, L, H * D, generator=g).mul(1.5).to(torch.bfloat16) for _ in range(3)]
        attn = types.SimpleNamespace()
        attn.heads = H
        attn.add_k_proj = None
        attn.to_q, attn.to_k, attn.to_v = (lambda x, t=t: t for t in proj)
        attn.norm_q = torch.nn.RMSNorm(H * D, eps=1e-6).to(torch.bfloat16)
        attn.norm_k = torch.nn.RMSNorm(H * D, eps=1e-6).to(torch.bfloat16)
        with torch.no_grad():
            attn.norm_q.weight.copy_(torch.rand(H * D, generator=g) + 0.5)
            attn.norm_k.weight.copy_(torch.rand(H * D, generator=g) + 0.5)
        attn.to_out = [torch.nn.Identity(), torch.nn.Identity()]
        angle = torch.rand(L, D // 2, generator=g, dtype=torch.float64) * 6.283185307179586
        freqs = torch.polar(torch.ones_like(angle), angle)[None, None]  # complex128 [1, 1, L, D/2]
        proc = replace_wan.Wan_DFSAttn_Processor2_0(
            "flash", 0.3, 16, 128, None, 0, [], 0, 1, 0.0, True, False)
        hidden = torch.zeros(1, L, H * D, dtype=torch.bfloat16)
        proc(attn, hidden, rotary_emb=freqs)
        q, k, v = captured["qkv"]
        assert q.shape == (1, H, L, D) and q.dtype == torch.bfloat16
        np.savez_compressed(
            os.path.join(HERE, name + ".npz"),
            q_src=u16(proj[0][0]), k_src=u16(proj[1][0]), v_src=u16(proj[2][0]),
            gamma_q=u16(attn.norm_q.weight.detach()), gamma_k=u16(attn.norm_k.weight.detach()),
            eps=np.float32(1e-6), heads=np.int32(H),
            cos=freqs.real[0, 0].to(torch.float32).numpy(), sin=freqs.imag[0, 0].to(torch.float32).numpy(),
            q=u16(q[0]), k=u16(k[0]), v=u16(v[0]))
        print("wrote", name)


if __name__ == "__main__":
    main()
