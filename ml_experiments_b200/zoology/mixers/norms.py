"""RMS norms used by the Mamba blocks: plain, fused with the residual add, and gated (``norm(x * silu(z))`` or
``norm(x) * silu(z)``, optionally per group). The reference takes these from vendored Triton kernels
(zoology/mixers/mamba_ssm/ops/triton/layer_norm.py, layernorm_gated.py); they are memory-bound elementwise passes
that PyTorch expresses directly."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F


class RMSNorm(nn.Module):
    def __init__(self, hidden_size: int, eps: float = 1e-5, device=None, dtype=None):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(hidden_size, device=device, dtype=dtype))
        self.register_parameter("bias", None)

    def forward(self, x, residual=None, prenorm: bool = False, residual_in_fp32: bool = False):
        return rms_norm_fn(x, self.weight, self.bias, residual=residual, eps=self.eps, prenorm=prenorm, residual_in_fp32=residual_in_fp32)


def rms_norm_fn(x, weight, bias=None, residual=None, eps: float = 1e-6, prenorm: bool = False, residual_in_fp32: bool = False):
    """``y = rmsnorm(x + residual)``; with ``prenorm`` also returns the summed residual stream."""
    dtype = x.dtype
    if residual is not None:
        x = (x + residual).to(x.dtype)
    res = x.float() if residual_in_fp32 else x
    xf = x.float()
    y = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * weight.float())
    if bias is not None:
        y = y + bias.float()
    y = y.to(dtype)
    return (y, res) if prenorm else y


def layer_norm_fn(x, weight, bias=None, residual=None, eps: float = 1e-6, prenorm: bool = False, residual_in_fp32: bool = False):
    dtype = x.dtype
    if residual is not None:
        x = (x + residual).to(x.dtype)
    res = x.float() if residual_in_fp32 else x
    y = F.layer_norm(x.float(), (x.shape[-1],), weight.float(), None if bias is None else bias.float(), eps).to(dtype)
    return (y, res) if prenorm else y


def rms_norm_ref(x, weight, bias=None, residual=None, eps: float = 1e-6, prenorm: bool = False, upcast: bool = False):
    """Plain-PyTorch statement of :func:`rms_norm_fn` (the two are the same code here; the reference keeps a Triton kernel
    and this oracle)."""
    return rms_norm_fn(x, weight, bias, residual=residual, eps=eps, prenorm=prenorm, residual_in_fp32=upcast)


def layer_norm_ref(x, weight, bias=None, residual=None, eps: float = 1e-6, prenorm: bool = False, upcast: bool = False):
    return layer_norm_fn(x, weight, bias, residual=residual, eps=eps, prenorm=prenorm, residual_in_fp32=upcast)


class RMSNormGated(nn.Module):
    def __init__(self, hidden_size: int, eps: float = 1e-5, group_size: int | None = None, norm_before_gate: bool = True,
                 device=None, dtype=None):
        super().__init__()
        self.eps, self.group_size, self.norm_before_gate = eps, group_size, norm_before_gate
        self.weight = nn.Parameter(torch.ones(hidden_size, device=device, dtype=dtype))
        self.register_parameter("bias", None)

    def forward(self, x, z=None):
        dtype = x.dtype
        xf = x.float()
        if z is not None and not self.norm_before_gate:
            xf = xf * F.silu(z.float())
        g = self.group_size or xf.shape[-1]
        xg = xf.unflatten(-1, (-1, g))
        y = (xg * torch.rsqrt(xg.pow(2).mean(-1, keepdim=True) + self.eps)).flatten(-2) * self.weight.float()
        if z is not None and self.norm_before_gate:
            y = y * F.silu(z.float())
        return y.to(dtype)
