"""fp8 linear layer with the weight stored transposed, ``(in_features, out_features)``.

``mm_t(x, w, x_s, w_s, grad_s)`` computes ``x @ w`` with ``x / x_s`` and ``w / w_s`` quantised to e4m3; its backward
quantises the incoming gradient (``/ grad_s``) to e5m2 and produces ``grad_x`` in bf16 and ``grad_w`` in fp32, already in
the ``(in, out)`` layout of the weight. Semantics of the reference's ``nanogpt::mm_t`` custom op
(modded-nanogpt/train_gpt.py:44-138), whose three products go through ``torch._scaled_mm`` and two explicit transposes;
here they are three calls of the tcgen05 GEMM (kind::f8f6f4) that read the operands in the majorness they are stored
in, so no transposed copy is made. ``CastedLinearT`` is the module (:784-813).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import fused as Fz
from . import gemm as G


class _MMT(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, x_s, w_s, grad_s):
        x8 = Fz.cast_fp8(x.contiguous(), 1.0 / x_s, torch.float8_e4m3fn)
        w8 = Fz.cast_fp8(w.contiguous(), 1.0 / w_s, torch.float8_e4m3fn)
        ctx.save_for_backward(x8, w8)
        ctx.scales = (x_s, w_s, grad_s)
        return G.gemm(x8, w8, b_mn=True, alpha=x_s * w_s)

    @staticmethod
    def backward(ctx, g):
        x8, w8 = ctx.saved_tensors
        x_s, w_s, grad_s = ctx.scales
        g8 = Fz.cast_fp8(g.contiguous(), 1.0 / grad_s, torch.float8_e5m2)
        grad_x = G.gemm(g8, w8, alpha=grad_s * w_s) if ctx.needs_input_grad[0] else None          # [M, N] x [K, N]^T
        grad_w = (G.gemm(x8, g8, a_mn=True, b_mn=True, out_dtype=torch.float32, alpha=x_s * grad_s)  # [M, K]^T x [M, N]
                  if ctx.needs_input_grad[1] else None)
        return grad_x, grad_w, None, None, None


class _HeadCE(torch.autograd.Function):
    """fp8 output projection and the soft-capped multi-token cross entropy as ONE autograd node returning the summed
    loss. The loss kernel writes ``dL/dlogits / grad_s`` straight in e5m2 while it computes the loss, so between the
    three GEMMs there is no bf16 gradient of the logits, no cast pass over it and no ``[T, V] x [T, 1]`` multiply by the
    incoming gradient: the node's incoming gradient is a scalar and scales the two small results instead."""

    @staticmethod
    def forward(ctx, x, w, targets, mtp_weights, x_s, w_s, grad_s, A, B, C):
        x8 = Fz.cast_fp8(x.contiguous(), 1.0 / x_s, torch.float8_e4m3fn)
        w8 = Fz.cast_fp8(w.contiguous(), 1.0 / w_s, torch.float8_e4m3fn)
        logits = G.gemm(x8, w8, b_mn=True, alpha=x_s * w_s)
        g8 = torch.empty(logits.shape, dtype=torch.float8_e5m2, device=x.device)
        mw = None if mtp_weights is None else mtp_weights.float().contiguous()
        rows = Fz.softcap_ce(logits, targets.contiguous(), grad_out=g8, cap=A, div=C, shift=B, grad_scale=1.0 / grad_s, mtp_weights=mw)
        ctx.save_for_backward(x8, w8, g8)
        ctx.scales = (x_s, w_s, grad_s)
        return rows.sum()

    @staticmethod
    def backward(ctx, gout):
        x8, w8, g8 = ctx.saved_tensors
        x_s, w_s, grad_s = ctx.scales
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = G.gemm(g8, w8, alpha=grad_s * w_s)
            dx = dx * gout.to(dx.dtype)
        if ctx.needs_input_grad[1]:
            dw = G.gemm(x8, g8, a_mn=True, b_mn=True, out_dtype=torch.float32, alpha=x_s * grad_s)
            dw = dw * gout.float()
        return dx, dw, None, None, None, None, None, None, None, None


def head_ce_loss(x, w, targets, mtp_weights=None, x_s: float = 1.0, w_s: float = 1.0, grad_s: float = 1.0,
                 A: float = 23.0, B: float = 5.0, C: float = 7.5) -> torch.Tensor:
    """``sum_t loss_t`` of ``softcapped_cross_entropy(x @ w, targets, mtp_weights)`` with ``w [K, V]``: the fused node on a
    GPU (bf16 ``x``, K and V multiples of 16), the two separate operators elsewhere."""
    if x.is_cuda and x.dtype == torch.bfloat16 and w.shape[0] % 16 == 0 and w.shape[1] % 16 == 0:
        return _HeadCE.apply(x, w.to(torch.bfloat16), targets, mtp_weights, float(x_s), float(w_s), float(grad_s), A, B, C)
    return Fz.softcapped_cross_entropy(x @ w.to(x.dtype), targets, mtp_weights, A, B, C).sum()


def mm_t(x: torch.Tensor, w: torch.Tensor, x_s: float = 1.0, w_s: float = 1.0, grad_s: float = 1.0) -> torch.Tensor:
    """``x [M, K] @ w [K, N]`` in fp8 on a GPU (K and N multiples of 16); plain matmul elsewhere."""
    if x.is_cuda and x.dtype == torch.bfloat16 and w.shape[0] % 16 == 0 and w.shape[1] % 16 == 0:
        return _MMT.apply(x, w.to(torch.bfloat16), float(x_s), float(w_s), float(grad_s))
    return x @ w.to(x.dtype)


def mm_t_ref(x, w, x_s, w_s, grad_s=1.0):
    """What the fp8 product computes, in fp32: quantise, multiply, rescale."""
    xq = (x.float() / x_s).to(torch.float8_e4m3fn).float()
    wq = (w.float() / w_s).to(torch.float8_e4m3fn).float()
    return (xq @ wq) * (x_s * w_s)


class CastedLinearT(nn.Module):
    def __init__(self, in_features: int, out_features: int, use_fp8: bool = False, x_s: float = 1.0, w_s: float = 1.0, grad_s: float = 1.0):
        super().__init__()
        self.in_features, self.out_features, self.use_fp8 = in_features, out_features, use_fp8
        self.x_s, self.w_s, self.grad_s = x_s, w_s, grad_s
        self.weight = nn.Parameter(torch.zeros(in_features, out_features, dtype=torch.bfloat16))

    def forward(self, x):
        if self.use_fp8 and self.training and x.is_cuda:
            return mm_t(x.flatten(0, -2), self.weight, self.x_s, self.w_s, self.grad_s).reshape(*x.shape[:-1], -1)
        return x @ self.weight.type_as(x)
