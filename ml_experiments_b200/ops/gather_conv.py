"""Weighted bilinear gather ("gather convolution") with autograd: the data-movement core of the telephone,
adaptive-local-conv and scatter attention operators.

``x`` is ``[B, L, C]`` (source rows), ``pos`` / ``wgt`` are ``[B, Lq, H, S]`` (``Lq`` query rows, ``Lq == L`` for a whole sequence):
``out[b, l, h] = sum_s wgt[b, l, h, s] * lerp(x[b, floor(p)], x[b, floor(p) + 1], frac(p))`` with ``p = pos[b, l, h, s]``
clamped to ``[0, pos_max]``. The default ``pos_max = L - 1.001`` is the rule of the reference's PyTorch modules
(src/heuristic_secrets/models/telephone_attention.py:150-156); ``pos_max = L - 1`` reads integer positions, the last row
included, exactly (the scatter operator uses it). Gradients flow to ``x``, ``pos`` and ``wgt``.
"""
from __future__ import annotations

import torch

from .runtime import ops


def gather_conv_ref(x: torch.Tensor, pos: torch.Tensor, wgt: torch.Tensor, num_heads: int, pos_max: float | None = None) -> torch.Tensor:
    """Plain-torch restatement (differentiable)."""
    B, L, C = x.shape
    H, S, Lq = num_heads, pos.shape[-1], pos.shape[1]
    D = C // H
    xh = x.view(B, L, H, D)
    pc = pos.clamp(0, L - 1.001 if pos_max is None else pos_max)
    fl = pc.detach().floor().long().clamp(0, max(L - 2, 0))
    ce = (fl + 1).clamp(0, L - 1)
    fr = (pc - fl.to(pc.dtype)).unsqueeze(-1)
    bidx = torch.arange(B, device=x.device).view(B, 1, 1, 1).expand(B, Lq, H, S)
    hidx = torch.arange(H, device=x.device).view(1, 1, H, 1).expand(B, Lq, H, S)
    vf, vc = xh[bidx, fl, hidx], xh[bidx, ce, hidx]  # [B, L, H, S, D]
    val = vf * (1 - fr) + vc * fr
    return (val * wgt.unsqueeze(-1).to(val.dtype)).sum(3).reshape(B, Lq, C)


class _GatherConv(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, pos, wgt, num_heads, pos_max):
        x16 = x.to(torch.bfloat16).contiguous()
        p32, w32 = pos.float().contiguous(), wgt.float().contiguous()
        out = torch.empty(x16.shape[0], pos.shape[1], x16.shape[2], dtype=torch.bfloat16, device=x16.device)
        ops().gather_conv_fwd(x16, p32, w32, out, num_heads, pos_max)
        ctx.save_for_backward(x16, p32, w32)
        ctx.h, ctx.pos_max, ctx.dt = num_heads, pos_max, (x.dtype, pos.dtype, wgt.dtype)
        return out.to(x.dtype)

    @staticmethod
    def backward(ctx, dout):
        x16, p32, w32 = ctx.saved_tensors
        dx = torch.zeros(x16.shape, dtype=torch.float32, device=x16.device)
        dpos, dwgt = torch.empty_like(p32), torch.empty_like(w32)
        ops().gather_conv_bwd(x16, p32, w32, dout.to(torch.bfloat16).contiguous(), dx, dpos, dwgt, ctx.h, ctx.pos_max)
        return dx.to(ctx.dt[0]), dpos.to(ctx.dt[1]), dwgt.to(ctx.dt[2]), None, None


def gather_conv(x: torch.Tensor, pos: torch.Tensor, wgt: torch.Tensor, num_heads: int, pos_max: float | None = None) -> torch.Tensor:
    d = x.shape[-1] // num_heads
    pos_max = float(x.shape[1] - 1.001 if pos_max is None else pos_max)
    if x.is_cuda and d in (8, 16, 32, 64, 128):
        return _GatherConv.apply(x, pos, wgt, num_heads, pos_max)
    return gather_conv_ref(x, pos, wgt, num_heads, pos_max)


def linear_resample(x: torch.Tensor, size: int) -> torch.Tensor:
    """``[B, L, C] -> [B, size, C]`` with the sample positions of ``F.interpolate(mode="linear", align_corners=False)``:
    one fractional tap per output row on the gather kernel (channel-last, no transposes, fp32 atomics backward)."""
    B, L, C = x.shape
    d = next((d for d in (128, 64, 32, 16, 8) if C % d == 0), None)
    if not x.is_cuda or d is None:
        return torch.nn.functional.interpolate(x.transpose(1, 2), size=size, mode="linear", align_corners=False).transpose(1, 2)
    H = C // d
    src = ((torch.arange(size, device=x.device, dtype=torch.float32) + 0.5) * (L / size) - 0.5).clamp(min=0)
    pos = src.view(1, size, 1, 1).expand(B, size, H, 1).contiguous()
    return gather_conv(x, pos, torch.ones_like(pos), H, pos_max=float(L - 1))
