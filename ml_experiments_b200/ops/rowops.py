"""Fused row-scaled add and three-term linear combination (``csrc/fused/rowops.cu``) with autograd; eager fallbacks off
CUDA / bf16. Used by the current speedrun GPT for the attention-output gate, the value-embedding mix and the per-layer
residual / x0 / bigram mix (modded-nanogpt/train_gpt.py: ``CausalSelfAttention.forward``, ``GPT.forward``)."""
from __future__ import annotations

import torch


def _bf16_cuda(*ts) -> bool:
    return all(t is None or (t.is_cuda and t.dtype == torch.bfloat16) for t in ts)


class _RowscaleAdd(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, g, b):
        from .runtime import add_launches, ops

        bc, gc = b.contiguous(), g.contiguous().view(-1)
        out = torch.empty_like(bc)
        ops().rowscale_add_fwd(a, gc, bc, out)
        add_launches(1)
        ctx.save_for_backward(gc, bc)
        ctx.has_a, ctx.gshape = a is not None, g.shape
        return out

    @staticmethod
    def backward(ctx, dout):
        from .runtime import add_launches, ops

        gc, bc = ctx.saved_tensors
        dout = dout.contiguous()
        db, dg = torch.empty_like(bc), torch.empty_like(gc)
        ops().rowscale_add_bwd(gc, bc, dout, db, dg)
        add_launches(1)
        return (dout if ctx.has_a else None), dg.view(ctx.gshape), db


def rowscale_add(a, g, b):
    """``a + g[..., None] * b`` (``a`` may be ``None``): ``a, b [B, T, H, D]`` with ``D`` in {64, 128}, ``g [B, T, H]``.
    ``a`` may be a strided view with a dense last dim (the v slice of a fused projection); the result is contiguous."""
    ok = (_bf16_cuda(a, g, b) and b.dim() == 4 and b.shape[-1] in (64, 128) and g.numel() == b.numel() // b.shape[-1]
          and (a is None or (a.shape == b.shape and a.stride(-1) == 1 and (a.shape[0] == 1 or a.stride(0) == a.shape[1] * a.stride(1)))))
    if not ok:
        out = g.reshape(*b.shape[:-1], 1) * b
        return out if a is None else a + out
    return _RowscaleAdd.apply(a, g, b)


class _Lincomb3(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, y, z, c):
        from .runtime import add_launches, ops

        xc, yc, zc = x.contiguous(), y.contiguous(), None if z is None else z.contiguous()
        cc = c.detach().float().contiguous()
        out = torch.empty_like(xc)
        ops().lincomb3_fwd(xc, yc, zc, cc, out)
        add_launches(1)
        ctx.save_for_backward(xc, yc, zc, cc)
        ctx.cdtype = c.dtype
        return out

    @staticmethod
    def backward(ctx, dout):
        from .runtime import add_launches, ops

        xc, yc, zc, cc = ctx.saved_tensors
        dout = dout.contiguous()
        dx, dy = torch.empty_like(xc), torch.empty_like(yc)
        dz = None if zc is None else torch.empty_like(zc)
        dc = torch.zeros(3, dtype=torch.float32, device=xc.device)
        ops().lincomb3_bwd(xc, yc, zc, cc, dout, dx, dy, dz, dc)
        add_launches(1)
        return dx, dy, dz, dc[: cc.numel()].to(ctx.cdtype)


def lincomb3(x, y, z, c):
    """``c[0] x + c[1] y (+ c[2] z)`` for same-shaped tensors and a coefficient vector ``c`` on the device (``z`` and
    ``c[2]`` optional). The coefficients' gradients are the three dot products with the incoming gradient."""
    n = 2 if z is None else 3
    ok = _bf16_cuda(x, y, z) and x.shape == y.shape and (z is None or z.shape == x.shape) and x.numel() % 4 == 0 and c.is_cuda and c.numel() == n
    if not ok:
        out = c[0].to(x.dtype) * x + c[1].to(x.dtype) * y
        return out if z is None else out + c[2].to(x.dtype) * z
    return _Lincomb3.apply(x, y, z, c)
