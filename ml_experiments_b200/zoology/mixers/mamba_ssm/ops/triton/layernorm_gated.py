"""Gated RMSNorm / LayerNorm of the Mamba-2 block (zoology/mixers/mamba_ssm/ops/triton/layernorm_gated.py:18-437):
``norm(x) * silu(z)`` (``norm_before_gate``) or ``norm(x * silu(z))``, optionally normalising groups of ``group_size``
channels separately. Memory-bound elementwise passes, written in PyTorch."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F


def _norm_ref(x, weight, bias, z, eps, group_size, norm_before_gate, rms: bool, upcast: bool = True):
    dtype = x.dtype
    xf = x.float() if upcast else x
    zf = None if z is None else (z.float() if upcast else z)
    if zf is not None and not norm_before_gate:
        xf = xf * F.silu(zf)
    g = group_size or xf.shape[-1]
    xg = xf.unflatten(-1, (-1, g))
    if not rms:
        xg = xg - xg.mean(-1, keepdim=True)
    y = (xg * torch.rsqrt(xg.pow(2).mean(-1, keepdim=True) + eps)).flatten(-2) * weight.to(xf.dtype)
    if bias is not None:
        y = y + bias.to(xf.dtype)
    if zf is not None and norm_before_gate:
        y = y * F.silu(zf)
    return y.to(dtype)


def rms_norm_ref(x, weight, bias, z=None, eps=1e-6, group_size=None, norm_before_gate=True, upcast=True):
    return _norm_ref(x, weight, bias, z, eps, group_size, norm_before_gate, True, upcast)


def layernorm_fn(x, weight, bias, z=None, eps=1e-6, group_size=None, norm_before_gate=True, is_rms_norm=False):
    return _norm_ref(x, weight, bias, z, eps, group_size, norm_before_gate, is_rms_norm)


def rmsnorm_fn(x, weight, bias, z=None, eps=1e-6, group_size=None, norm_before_gate=True):
    return _norm_ref(x, weight, bias, z, eps, group_size, norm_before_gate, True)


class LayerNorm(nn.Module):
    def __init__(self, hidden_size, eps=1e-5, group_size=None, norm_before_gate=True, device=None, dtype=None):
        super().__init__()
        self.eps, self.group_size, self.norm_before_gate = eps, group_size, norm_before_gate
        self.weight = nn.Parameter(torch.ones(hidden_size, device=device, dtype=dtype))
        self.bias = nn.Parameter(torch.zeros(hidden_size, device=device, dtype=dtype))

    def forward(self, x, z=None):
        return layernorm_fn(x, self.weight, self.bias, z, self.eps, self.group_size, self.norm_before_gate)


class RMSNorm(nn.Module):
    def __init__(self, hidden_size, eps=1e-5, group_size=None, norm_before_gate=True, device=None, dtype=None):
        super().__init__()
        self.eps, self.group_size, self.norm_before_gate = eps, group_size, norm_before_gate
        self.weight = nn.Parameter(torch.ones(hidden_size, device=device, dtype=dtype))
        self.register_parameter("bias", None)

    def forward(self, x, z=None):
        return rmsnorm_fn(x, self.weight, self.bias, z, self.eps, self.group_size, self.norm_before_gate)
