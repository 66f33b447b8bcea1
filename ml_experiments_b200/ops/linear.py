"""``y = x @ W.T`` as an autograd function on the tcgen05 GEMM (forward, data gradient and weight gradient).

Used by every model of the package whose projections should not go through a library GEMM; falls back to
``torch.nn.functional.linear`` for CPU tensors or shapes the TMA descriptors cannot express (row pitch not a multiple
of 16 bytes).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import gemm as G


def _ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    return x.is_cuda and x.shape[-1] % 8 == 0 and w.shape[0] % 8 == 0 and x.numel() > 0


def _residual_operand(residual, rows: int, cols: int):
    """The residual as a bf16 ``[rows, cols]`` operand of the GEMM epilogue, or ``None`` when it cannot be one."""
    if residual is None or residual.dtype != torch.bfloat16 or residual.numel() != rows * cols or not residual.is_contiguous():
        return None
    return residual.view(rows, cols)


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, epilogue, residual=None):
        x2 = x.reshape(-1, x.shape[-1])
        x16 = x2 if x2.dtype == torch.bfloat16 else x2.to(torch.bfloat16)
        w16 = w if w.dtype == torch.bfloat16 else w.to(torch.bfloat16)
        x16, w16 = x16.contiguous(), w16.contiguous()
        if residual is not None:      # out = x W^T + residual in the GEMM epilogue (the caller checked the operand)
            y = G.gemm(x16, w16, epilogue=G.EPI_AXPBY, aux=residual.view(x16.shape[0], w16.shape[0]), alpha=1.0, beta=1.0)
        else:
            y = G.gemm(x16, w16, epilogue=epilogue)
        ctx.save_for_backward(x16, w16, y if epilogue == G.EPI_RELU2 else None)
        ctx.epilogue, ctx.x_shape, ctx.x_dtype, ctx.w_dtype = epilogue, x.shape, x.dtype, w.dtype
        ctx.has_res = residual is not None
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x16, w16, h = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).to(torch.bfloat16).contiguous()
        if ctx.epilogue == G.EPI_RELU2:  # d relu(z)^2 / dz = 2 relu(z) = 2 sqrt(h)
            dy2 = dy2 * h.sqrt().mul_(2)
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = G.gemm(dy2, w16, b_mn=True).view(ctx.x_shape).to(ctx.x_dtype)
        if ctx.needs_input_grad[1]:
            sk = G.auto_split_k(w16.shape[0], w16.shape[1], x16.shape[0])
            dw = G.gemm(dy2, x16, a_mn=True, b_mn=True, split_k=sk, out_dtype=torch.float32).to(ctx.w_dtype)
        return dx, dw, None, (dy if ctx.has_res else None)


def linear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None, relu2: bool = False,
           residual: torch.Tensor | None = None) -> torch.Tensor:
    """bf16 tensor-core linear layer; ``relu2=True`` fuses ``relu(.)**2`` into the GEMM epilogue (no bias then);
    ``residual`` (the output's shape) is added in the epilogue as well when it is a dense bf16 tensor."""
    if not _ok(x, w):
        y = F.linear(x, w.to(x.dtype), None if bias is None else bias.to(x.dtype))
        y = F.relu(y).square() if relu2 else y
        return y if residual is None else residual + y
    if residual is not None:
        rows = x.numel() // x.shape[-1]
        if relu2 or bias is not None or _residual_operand(residual, rows, w.shape[0]) is None or residual.shape[:-1] != x.shape[:-1]:
            return residual + linear(x, w, bias, relu2)
        return _Linear.apply(x, w, G.EPI_NONE, residual)
    y = _Linear.apply(x, w, G.EPI_RELU2 if (relu2 and bias is None) else G.EPI_NONE, None)
    if bias is not None:
        y = y + bias.to(y.dtype)
        if relu2:
            y = F.relu(y).square()
    return y


class _LinearTee(torch.autograd.Function):
    """``(x @ W.T, x)``: the second output stands for ``x`` in its other uses, so that their gradient arrives here and is
    added in the epilogue of the data-gradient GEMM (autograd would add the two gradients of ``x`` in a pass of its own)."""

    @staticmethod
    def forward(ctx, x, w):
        x16 = x.reshape(-1, x.shape[-1])
        w16 = w.to(torch.bfloat16).contiguous()
        ctx.save_for_backward(x16, w16)
        ctx.x_shape, ctx.w_dtype = x.shape, w.dtype
        return G.gemm(x16, w16).view(*x.shape[:-1], w.shape[0]), x.view_as(x)

    @staticmethod
    def backward(ctx, dy, dtee):
        x16, w16 = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).to(torch.bfloat16).contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            other = dtee.reshape(-1, dtee.shape[-1]).to(torch.bfloat16).contiguous()
            dx = G.gemm(dy2, w16, b_mn=True, epilogue=G.EPI_AXPBY, aux=other, alpha=1.0, beta=1.0).view(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            sk = G.auto_split_k(w16.shape[0], w16.shape[1], x16.shape[0])
            dw = G.gemm(dy2, x16, a_mn=True, b_mn=True, split_k=sk, out_dtype=torch.float32).to(ctx.w_dtype)
        return dx, dw


def linear_tee(x: torch.Tensor, w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """``(x @ w.T, x)`` for an ``x`` with further consumers: feed them the returned ``x`` and the sum of the two
    gradients costs no pass of its own. Both outputs must be used in the differentiated result."""
    if not (_ok(x, w) and x.dtype == torch.bfloat16 and x.is_contiguous()):
        return linear(x, w), x
    return _LinearTee.apply(x, w)


class _LinearPair(torch.autograd.Function):
    """``(x @ W[:split].T, x @ W[split:].T)`` as one node: two forward GEMMs on row ranges of ``W`` (each output dense,
    no strided halves of one wide output), and in the backward the second data-gradient GEMM adds the first one's
    result in its epilogue and the two weight-gradient GEMMs write the row ranges of one ``W``-shaped buffer. Two
    separate nodes would leave autograd an elementwise add of the two ``dx`` and a zero-fill + copy + add per half of
    ``dW``."""

    @staticmethod
    def forward(ctx, x, w, split):
        x16 = x.reshape(-1, x.shape[-1]).to(torch.bfloat16).contiguous()
        w16 = w.to(torch.bfloat16).contiguous()
        ctx.save_for_backward(x16, w16)
        ctx.split, ctx.x_shape, ctx.x_dtype, ctx.w_dtype = split, x.shape, x.dtype, w.dtype
        ya, yb = G.gemm(x16, w16[:split]), G.gemm(x16, w16[split:])
        return ya.view(*x.shape[:-1], split), yb.view(*x.shape[:-1], w.shape[0] - split)

    @staticmethod
    def backward(ctx, dya, dyb):
        x16, w16 = ctx.saved_tensors
        s = ctx.split
        da = dya.reshape(-1, dya.shape[-1]).to(torch.bfloat16).contiguous()
        db = dyb.reshape(-1, dyb.shape[-1]).to(torch.bfloat16).contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = G.gemm(da, w16[:s], b_mn=True)
            dx = G.gemm(db, w16[s:], b_mn=True, epilogue=G.EPI_AXPBY, aux=dx, alpha=1.0, beta=1.0).view(ctx.x_shape).to(ctx.x_dtype)
        if ctx.needs_input_grad[1]:
            dw = torch.empty(w16.shape, dtype=torch.float32, device=w16.device)
            for rows, dy2 in ((slice(0, s), da), (slice(s, None), db)):
                sk = G.auto_split_k(dy2.shape[1], w16.shape[1], x16.shape[0])
                G.gemm(dy2, x16, a_mn=True, b_mn=True, split_k=sk, out=dw[rows])
            dw = dw.to(ctx.w_dtype)
        return dx, dw, None


def linear_pair(x: torch.Tensor, w: torch.Tensor, split: int) -> tuple[torch.Tensor, torch.Tensor]:
    """The two halves ``x @ w[:split].T`` and ``x @ w[split:].T`` of one projection as separate dense tensors."""
    if not (_ok(x, w) and split % 8 == 0 and (w.shape[0] - split) % 8 == 0 and w.shape[1] % 8 == 0):
        y = F.linear(x, w.to(x.dtype))
        return y[..., :split], y[..., split:]
    return _LinearPair.apply(x, w, split)


class _LinearT(torch.autograd.Function):
    """``y = x @ W`` for a weight stored ``(in_features, out_features)``: all three GEMMs read it as stored."""

    @staticmethod
    def forward(ctx, x, w):
        x16 = x.reshape(-1, x.shape[-1]).to(torch.bfloat16).contiguous()
        w16 = w.to(torch.bfloat16).contiguous()
        ctx.save_for_backward(x16, w16)
        ctx.x_shape, ctx.x_dtype, ctx.w_dtype = x.shape, x.dtype, w.dtype
        return G.gemm(x16, w16, b_mn=True).view(*x.shape[:-1], w.shape[1])

    @staticmethod
    def backward(ctx, dy):
        x16, w16 = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).to(torch.bfloat16).contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = G.gemm(dy2, w16).view(ctx.x_shape).to(ctx.x_dtype)
        if ctx.needs_input_grad[1]:
            sk = G.auto_split_k(w16.shape[0], w16.shape[1], x16.shape[0])
            dw = G.gemm(x16, dy2, a_mn=True, b_mn=True, split_k=sk, out_dtype=torch.float32).to(ctx.w_dtype)
        return dx, dw


def linear_t(x: torch.Tensor, w_t: torch.Tensor) -> torch.Tensor:
    """``x @ w_t`` with ``w_t`` of shape ``(in_features, out_features)``."""
    if not (x.is_cuda and w_t.shape[0] % 8 == 0 and w_t.shape[1] % 8 == 0 and x.numel() > 0):
        return x @ w_t.to(x.dtype)
    return _LinearT.apply(x, w_t)


class _MlpRelu2(torch.autograd.Function):
    """``relu(x @ Wfc.T)^2 @ Wproj`` (both weights stored ``[hidden, d]``) as one autograd node: four GEMMs in the
    backward, the ``2 relu(z)`` factor of the activation applied in the epilogue of the first of them, so no
    elementwise pass over the ``[T, hidden]`` tensors is left (a chain of two separate nodes has to form
    ``dh * 2 sqrt(h)`` with PyTorch operators between its GEMMs)."""

    @staticmethod
    def forward(ctx, x, w_fc, w_proj, residual=None):
        to16 = lambda t: (t if t.dtype == torch.bfloat16 else t.to(torch.bfloat16)).contiguous()
        x16, fc16, pj16 = to16(x.reshape(-1, x.shape[-1])), to16(w_fc), to16(w_proj)
        h = G.gemm(x16, fc16, epilogue=G.EPI_RELU2)
        if residual is not None:
            y = G.gemm(h, pj16, b_mn=True, epilogue=G.EPI_AXPBY, aux=residual.view(h.shape[0], pj16.shape[1]), alpha=1.0, beta=1.0)
        else:
            y = G.gemm(h, pj16, b_mn=True)
        ctx.save_for_backward(x16, fc16, pj16, h)
        ctx.x_shape, ctx.dtypes, ctx.has_res = x.shape, (x.dtype, w_fc.dtype, w_proj.dtype), residual is not None
        return y.view(*x.shape[:-1], w_proj.shape[1])

    @staticmethod
    def backward(ctx, dy):
        x16, fc16, pj16, h = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).to(torch.bfloat16).contiguous()
        dpre = G.gemm(dy2, pj16, epilogue=G.EPI_RELU2_BWD, aux=h)            # (dy @ Wproj.T) * 2 relu(z)
        dx = dfc = dpj = None
        if ctx.needs_input_grad[2]:
            dpj = G.gemm(h, dy2, a_mn=True, b_mn=True, split_k=G.auto_split_k(pj16.shape[0], pj16.shape[1], h.shape[0]),
                         out_dtype=torch.float32).to(ctx.dtypes[2])
        if ctx.needs_input_grad[0]:
            dx = G.gemm(dpre, fc16, b_mn=True).view(ctx.x_shape).to(ctx.dtypes[0])
        if ctx.needs_input_grad[1]:
            dfc = G.gemm(dpre, x16, a_mn=True, b_mn=True, split_k=G.auto_split_k(fc16.shape[0], fc16.shape[1], x16.shape[0]),
                         out_dtype=torch.float32).to(ctx.dtypes[1])
        return dx, dfc, dpj, (dy if ctx.has_res else None)


def mlp_relu2(x: torch.Tensor, w_fc: torch.Tensor, w_proj: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
    """``relu(x @ w_fc.T)**2 @ w_proj (+ residual)`` with ``w_fc, w_proj`` of shape ``(hidden, d)``; a dense bf16
    ``residual`` of the output's shape is added in the epilogue of the second GEMM."""
    if not (_ok(x, w_fc) and w_proj.shape[1] % 8 == 0 and w_fc.shape == w_proj.shape):
        y = F.relu(F.linear(x, w_fc.to(x.dtype))).square() @ w_proj.to(x.dtype)
        return y if residual is None else residual + y
    if residual is not None and (_residual_operand(residual, x.numel() // x.shape[-1], w_proj.shape[1]) is None or residual.shape[:-1] != x.shape[:-1]):
        return residual + _MlpRelu2.apply(x, w_fc, w_proj, None)
    return _MlpRelu2.apply(x, w_fc, w_proj, residual)
