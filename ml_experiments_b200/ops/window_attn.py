"""Local window attention with a per-tap additive bias, with autograd.

``out[b,l,h] = sum_w softmax_w(scale * q[b,l,h] . k[b, l + w - (K-1)//2, h] + bias[b,l,h,w]) v[b, l + w - (K-1)//2, h]``.
Keys and values beyond the ends of the sequence are zero vectors that stay inside the softmax, which is what unfolding a
zero-padded sequence gives (src/heuristic_secrets/models/scatter_attention.py:996-1023). CUDA kernels for
``D in {16, 32, 64}`` and ``K <= 64``; the unfold restatement otherwise and as the oracle.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .runtime import ops


def window_attention_ref(q, k, v, bias, scale: float):
    """``q, k, v [B, L, H, D]``, ``bias [B, L, H, K]``."""
    K = bias.shape[-1]
    pl, pr = (K - 1) // 2, K // 2
    kw = F.pad(k, (0, 0, 0, 0, pl, pr)).unfold(1, K, 1)  # [B, L, H, D, K]
    vw = F.pad(v, (0, 0, 0, 0, pl, pr)).unfold(1, K, 1)
    s = torch.einsum("blhd,blhdw->blhw", q, kw) * scale + bias.to(q.dtype)
    return torch.einsum("blhw,blhdw->blhd", F.softmax(s, dim=-1), vw)


class _WindowAttn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, bias, scale):
        q16, k16, v16 = (t.to(torch.bfloat16).contiguous() for t in (q, k, v))
        b32 = bias.float().contiguous()
        out = torch.empty_like(q16)
        P = torch.empty_like(b32)
        ops().window_attn_fwd(q16, k16, v16, b32, out, P, float(scale))
        ctx.save_for_backward(q16, k16, v16, P)
        ctx.scale, ctx.dtypes = float(scale), (q.dtype, k.dtype, v.dtype, bias.dtype)
        return out.to(q.dtype)

    @staticmethod
    def backward(ctx, dout):
        q16, k16, v16, P = ctx.saved_tensors
        dq, dk, dv = torch.empty_like(q16), torch.empty_like(k16), torch.empty_like(v16)
        dbias = torch.empty_like(P)
        ops().window_attn_bwd(q16, k16, v16, P, dout.to(torch.bfloat16).contiguous(), dq, dk, dv, dbias, ctx.scale)
        t = ctx.dtypes
        return dq.to(t[0]), dk.to(t[1]), dv.to(t[2]), dbias.to(t[3]), None


def window_attention(q, k, v, bias, scale: float):
    if q.is_cuda and q.shape[-1] in (16, 32, 64) and bias.shape[-1] <= 64:
        return _WindowAttn.apply(q, k, v, bias, scale)
    return window_attention_ref(q, k, v, bias, scale)
