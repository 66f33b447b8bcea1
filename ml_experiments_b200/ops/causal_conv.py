"""Causal depthwise conv1d (width 4) + bias + SiLU on channel-last activations, with autograd.

CUDA kernels for bf16 inputs; the same math through ``F.conv1d`` otherwise. ``x`` may be a channel slice of a wider
tensor (for example the first half of an ``in_proj`` output), which avoids a split copy.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .runtime import ops


def causal_conv1d_silu_ref(x, weight, bias):
    """x: [B, L, C]; weight: [C, 1, K]; bias: [C]."""
    k = weight.shape[-1]
    y = F.conv1d(x.transpose(1, 2), weight.to(x.dtype), None if bias is None else bias.to(x.dtype), padding=k - 1,
                 groups=x.shape[-1])[..., : x.shape[1]]
    return F.silu(y.transpose(1, 2))


class _CausalConv(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias):
        w32 = weight.detach().float().reshape(weight.shape[0], 4).contiguous()
        b32 = None if bias is None else bias.detach().float().contiguous()
        y = torch.empty(x.shape, dtype=torch.bfloat16, device=x.device)
        ops().causal_conv1d_silu_fwd(x, w32, b32, y)
        ctx.save_for_backward(x, w32, b32)
        ctx.wshape, ctx.wdtype, ctx.bdtype = weight.shape, weight.dtype, None if bias is None else bias.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w32, b32 = ctx.saved_tensors
        dy = dy.to(torch.bfloat16).contiguous()
        dx = torch.empty(x.shape, dtype=torch.bfloat16, device=x.device)
        dw = torch.zeros_like(w32)
        db = None if b32 is None else torch.zeros_like(b32)
        ops().causal_conv1d_silu_bwd(x, w32, b32, dy, dx, dw, db)
        return dx, dw.view(ctx.wshape).to(ctx.wdtype), None if db is None else db.to(ctx.bdtype)


def causal_conv1d_silu(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None) -> torch.Tensor:
    ok = (x.is_cuda and x.dtype == torch.bfloat16 and weight.shape[-1] == 4 and x.shape[-1] % 8 == 0 and x.stride(2) == 1
          and x.stride(1) % 8 == 0 and x.stride(0) == x.shape[1] * x.stride(1))
    if not ok:
        return causal_conv1d_silu_ref(x, weight, bias)
    return _CausalConv.apply(x, weight, bias)
