"""Weighted RMSNorm with a fused activation (one kernel forward, one backward): ``act(w * x * rsqrt(mean(x^2) + eps))``.

The Ripple-family operators normalise every small projection this way (telephone / adaptive-conv wave, kernel, window
and exponent heads: src/heuristic_secrets/models/telephone_attention.py:17-30,124-140 of the reference) and the
unfused PyTorch form costs about eight elementwise kernels forward and twice that backward per call.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .runtime import ops

_ACTS = {"none": 0, "silu": 1, "sigmoid": 2, "tanh": 3}
_ACT_FN = {"none": lambda t: t, "silu": F.silu, "sigmoid": torch.sigmoid, "tanh": torch.tanh}


def rms_norm_act_ref(x, weight, eps: float = 1e-6, act: str = "none", out_dtype=None):
    xf = x.float()
    y = _ACT_FN[act](weight.float() * (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)))
    return y.to(out_dtype or x.dtype)


class _RmsAct(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps, act, out_dtype):
        xc = x.contiguous()
        w32 = weight.detach().float().contiguous()
        y = torch.empty(xc.shape, dtype=out_dtype, device=x.device)
        rstd = torch.empty(xc.numel() // xc.shape[-1], dtype=torch.float32, device=x.device)
        ops().rms_act_fwd(xc, w32, y, rstd, eps, act)
        ctx.save_for_backward(xc, w32, rstd)
        ctx.act, ctx.wdtype = act, weight.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        xc, w32, rstd = ctx.saved_tensors
        if dy.dtype not in (torch.bfloat16, torch.float32):
            dy = dy.float()
        dx = torch.empty_like(xc)
        dw = torch.zeros_like(w32)
        ops().rms_act_bwd(xc, w32, rstd, dy.contiguous(), None, None, dx, dw, ctx.act)
        return dx, dw.to(ctx.wdtype), None, None, None


class _RmsActSkip(torch.autograd.Function):
    """``(norm(x), x[, norm(x)[..., :lead]])``: the second output is the skip connection around the norm, so that the
    backward kernel adds the skip's gradient to the norm's in the pass that writes ``dx`` (autograd would run an
    elementwise add after it). With ``lead > 0`` the first ``lead`` columns of the normed rows are a third output (the
    input of small gate projections): the kernel adds their gradient to those columns of ``dy`` as it reads them,
    instead of a zero-filled full-size tensor and another add."""

    @staticmethod
    def forward(ctx, x, weight, eps, act, lead):
        xc = x.contiguous()
        w32 = weight.detach().float().contiguous()
        y = torch.empty_like(xc)
        rstd = torch.empty(xc.numel() // xc.shape[-1], dtype=torch.float32, device=x.device)
        ops().rms_act_fwd(xc, w32, y, rstd, eps, act)
        ctx.save_for_backward(xc, w32, rstd)
        ctx.act, ctx.wdtype, ctx.lead = act, weight.dtype, lead
        if lead:
            return y, x.view_as(x), y[..., :lead].contiguous()
        return y, x.view_as(x)

    @staticmethod
    def backward(ctx, dy, dskip, dlead=None):
        xc, w32, rstd = ctx.saved_tensors
        if dy.dtype not in (torch.bfloat16, torch.float32):
            dy = dy.float()
        dx = torch.empty_like(xc)
        dw = torch.zeros_like(w32)
        lead = dlead.to(dy.dtype).contiguous() if (ctx.lead and dlead is not None) else None
        ops().rms_act_bwd(xc, w32, rstd, dy.contiguous(), dskip.to(xc.dtype).contiguous(), lead, dx, dw, ctx.act)
        return dx, dw.to(ctx.wdtype), None, None, None


def rms_norm_act(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6, act: str = "none", out_dtype=None) -> torch.Tensor:
    out_dtype = out_dtype or x.dtype
    ok = (x.is_cuda and x.dtype in (torch.bfloat16, torch.float32) and out_dtype in (torch.bfloat16, torch.float32)
          and 1 <= x.shape[-1] <= 4096 and weight.numel() == x.shape[-1])
    if not ok:
        return rms_norm_act_ref(x, weight, eps, act, out_dtype)
    return _RmsAct.apply(x, weight, float(eps), _ACTS[act], out_dtype)


def rms_norm_act_skip(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6, act: str = "none", lead_cols: int = 0):
    """``(rms_norm_act(x), x)`` for a pre-norm residual block ``skip + f(norm(x))``: use the returned ``x`` as the skip
    and both gradients meet inside the norm's backward kernel. ``lead_cols = k > 0`` adds a third output, the first ``k``
    columns of the normed rows as a dense tensor, whose gradient joins the same kernel launch."""
    ok = x.is_cuda and x.dtype in (torch.bfloat16, torch.float32) and 1 <= x.shape[-1] <= 4096 and weight.numel() == x.shape[-1]
    if not ok:
        y = rms_norm_act_ref(x, weight, eps, act)
        return (y, x, y[..., :lead_cols]) if lead_cols else (y, x)
    return _RmsActSkip.apply(x, weight, float(eps), _ACTS[act], int(lead_cols))
