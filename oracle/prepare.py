"""CPU restatement of the reference's pre-attention step (test infrastructure only).

Only tests, the smoke check and the bench's CPU baseline may import this module;
the product path never does.

What it restates, for token-major projections [rows, H*D]:

* unflatten / transpose to head-major: ``dfsattn/replace_hyvideo.py:247-249``,
  ``dfsattn/replace_wan.py:174-176``;
* RMSNorm ``y = (x * rsqrt(mean(x^2) + eps)) * gamma`` in fp32, rounded to the tensor
  type -- per head (``dfsattn/kernels/include/norm/narrow_rms_norm.cuh:22-71`` through
  ``dfsattn/kernels/__init__.py:34-52``) or over the whole H*D row
  (``dfsattn/kernels/triton/rmsnorm.py:8-49`` as called at ``replace_wan.py:162-166``);
* rotary embedding of the leading ``rope_rows`` tokens on the rounded result,
  ``out[i] = x[i]*cos[i] + (i even ? -x[i+1] : x[i-1])*sin[i]`` in fp32
  (``dfsattn/kernels/include/rope/rope_enc.cuh:17-36``; rows past the video part are
  left alone, ``rope_enc_txtlast.cuh:46-50``); with a table of one value per pair this
  is the complex product of ``replace_wan.py:207-215``;
* the token gather of ``dfsattn/attention_hyvideo.py:1034-1036``.

Parity status: the whole-row norm + complex rotation + transpose is pinned by
``tests/golden/wan_prepare_*.npz`` (outputs of the reference's own Wan processor run
on CPU); the per-head norm and the text-last rotation restate the reference's CUDA
kernels, whose Python fallback needs a package that is absent here: parity unpinned
for those two variants.
"""
import torch


def _rmsnorm(x, gamma, eps, heads, across_heads):
    rows, hd = x.shape
    if across_heads:
        rstd = torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + eps)
        y = (x * rstd) * gamma.float()[None, :]
    else:
        d = hd // heads
        xh = x.view(rows, heads, d)
        rstd = torch.rsqrt((xh * xh).mean(dim=-1, keepdim=True) + eps)
        y = ((xh * rstd) * gamma.float()[None, None, :]).reshape(rows, hd)
    return y.to(torch.bfloat16).float()


def _rope(xh, cos, sin, rope_rows):
    """xh: [rows, H, D] fp32; cos/sin: [>=rope_rows, D] or [.., D/2] fp32."""
    d = xh.shape[-1]
    if cos.shape[1] == d // 2:
        cos = cos.repeat_interleave(2, dim=1)
        sin = sin.repeat_interleave(2, dim=1)
    n = min(rope_rows, xh.shape[0])
    x = xh[:n]
    even, odd = x[..., 0::2], x[..., 1::2]
    partner = torch.stack([-odd, even], dim=-1).flatten(-2)  # (-x1, x0, -x3, x2, ...)
    out = xh.clone()
    out[:n] = x * cos[:n, None, :] + partner * sin[:n, None, :]
    return out


def qkv_prepare_ref(q_src, k_src, v_src, heads, gamma_q=None, gamma_k=None, eps_q=1e-6, eps_k=1e-6,
                    norm_across_heads=False, cos=None, sin=None, rope_rows=None, perm=None):
    """bf16 CPU tensors [rows, H*D] -> (q, k, v) bf16 [H, n, D] (None stays None)."""
    outs = []
    for t, (src, gamma, eps) in enumerate(((q_src, gamma_q, eps_q), (k_src, gamma_k, eps_k), (v_src, None, 0.0))):
        if src is None:
            outs.append(None)
            continue
        x = src.float()
        rows, hd = x.shape
        if gamma is not None:
            x = _rmsnorm(x, gamma, eps, heads, norm_across_heads)
        xh = x.view(rows, heads, hd // heads)
        if t < 2 and cos is not None:
            xh = _rope(xh, cos.float(), sin.float(), cos.shape[0] if rope_rows is None else rope_rows)
        out = xh.to(torch.bfloat16).permute(1, 0, 2)
        if perm is not None:
            out = out[:, perm.long()]
        outs.append(out.contiguous())
    return tuple(outs)
