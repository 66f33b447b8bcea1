"""Mamba (S6) mixer and its residual block (zoology/mixers/mamba.py:22-297).

in_proj -> (x, z); causal depthwise conv (width ``d_conv``) + SiLU on x; x_proj -> (dt, B, C); dt_proj; selective scan
with the softplus, the dt bias, the ``D`` skip and the ``silu(z)`` gate all inside the scan kernels; out_proj. On a GPU
the conv is the fused causal-conv1d+SiLU kernel (width 4) and the scan is the S6 kernel (state 16); other shapes and the
CPU take the PyTorch path. The reference needs the external ``causal_conv1d`` and ``selective_scan_cuda`` packages.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...ops.causal_conv import causal_conv1d_silu
from ...ops.selective_scan import causal_conv1d_update, selective_scan, selective_state_update
from .norms import RMSNorm, layer_norm_fn, rms_norm_fn


class Mamba(nn.Module):
    def __init__(self, d_model, d_state: int = 16, d_conv: int = 4, expand: int = 2, dt_rank="auto", dt_min: float = 0.001,
                 dt_max: float = 0.1, dt_init: str = "random", dt_scale: float = 1.0, dt_init_floor: float = 1e-4,
                 conv_bias: bool = True, bias: bool = False, use_fast_path: bool = True, layer_idx=None, device=None, dtype=None,
                 **kwargs):
        fk = {"device": device, "dtype": dtype}
        super().__init__()
        self.d_model, self.d_state, self.d_conv, self.expand = d_model, d_state, d_conv, expand
        self.d_inner = int(expand * d_model)
        self.dt_rank = math.ceil(d_model / 16) if dt_rank == "auto" else dt_rank
        self.use_fast_path, self.layer_idx = use_fast_path, layer_idx
        self.in_proj = nn.Linear(d_model, self.d_inner * 2, bias=bias, **fk)
        self.conv1d = nn.Conv1d(self.d_inner, self.d_inner, bias=conv_bias, kernel_size=d_conv, groups=self.d_inner,
                                padding=d_conv - 1, **fk)
        self.activation, self.act = "silu", nn.SiLU()
        self.x_proj = nn.Linear(self.d_inner, self.dt_rank + d_state * 2, bias=False, **fk)
        self.dt_proj = nn.Linear(self.dt_rank, self.d_inner, bias=True, **fk)
        std = self.dt_rank ** -0.5 * dt_scale
        if dt_init == "constant":
            nn.init.constant_(self.dt_proj.weight, std)
        elif dt_init == "random":
            nn.init.uniform_(self.dt_proj.weight, -std, std)
        else:
            raise NotImplementedError
        dt = torch.exp(torch.rand(self.d_inner, **fk) * (math.log(dt_max) - math.log(dt_min)) + math.log(dt_min)).clamp(min=dt_init_floor)
        with torch.no_grad():
            self.dt_proj.bias.copy_(dt + torch.log(-torch.expm1(-dt)))
        self.dt_proj.bias._no_reinit = True
        self.A_log = nn.Parameter(torch.log(torch.arange(1, d_state + 1, dtype=torch.float32, device=device)).repeat(self.d_inner, 1))
        self.A_log._no_weight_decay = True
        self.D = nn.Parameter(torch.ones(self.d_inner, device=device))
        self.D._no_weight_decay = True
        self.out_proj = nn.Linear(self.d_inner, d_model, bias=bias, **fk)

    def forward(self, hidden_states, inference_params=None):
        L = hidden_states.shape[1]
        x, z = self.in_proj(hidden_states).chunk(2, dim=-1)
        if x.is_cuda and self.d_conv == 4 and x.dtype == torch.bfloat16:
            x = causal_conv1d_silu(x, self.conv1d.weight, self.conv1d.bias)
        else:
            x = self.act(self.conv1d(x.transpose(1, 2))[..., :L].transpose(1, 2))
        dt, B, C = self.x_proj(x).split([self.dt_rank, self.d_state, self.d_state], dim=-1)
        y = selective_scan(x.contiguous(), F.linear(dt, self.dt_proj.weight), -torch.exp(self.A_log.float()), B, C, self.D.float(),
                           z=z.contiguous(), delta_bias=self.dt_proj.bias.float(), delta_softplus=True)
        return self.out_proj(y)

    def allocate_inference_cache(self, batch_size: int, max_seqlen: int = 0, dtype=None):
        """``(conv_state [B, Din, K], ssm_state [B, Din, N])`` for token-by-token decoding with :meth:`step`."""
        w = self.conv1d.weight
        return (torch.zeros(batch_size, self.d_inner, self.d_conv, device=w.device, dtype=dtype or w.dtype),
                torch.zeros(batch_size, self.d_inner, self.d_state, device=w.device, dtype=torch.float32))

    def step(self, hidden_states, conv_state, ssm_state):
        """One token ``[B, 1, d_model]`` through the layer, updating both states in place (mamba.py:199-249 of the reference)."""
        x, z = self.in_proj(hidden_states.squeeze(1)).chunk(2, dim=-1)
        x = causal_conv1d_update(x, conv_state, self.conv1d.weight.squeeze(1), self.conv1d.bias, "silu")
        dt, B, C = self.x_proj(x).split([self.dt_rank, self.d_state, self.d_state], dim=-1)
        y = selective_state_update(ssm_state, x, F.linear(dt, self.dt_proj.weight), -torch.exp(self.A_log.float()), B, C, self.D.float(),
                                   z=z, dt_bias=self.dt_proj.bias.float(), dt_softplus=True)
        return self.out_proj(y).unsqueeze(1), conv_state, ssm_state

    def state_size(self, sequence_length: int = 2048):
        return 2 * self.d_model * self.d_state


class _AddNormMixerBlock(nn.Module):
    """``residual += hidden; hidden = mixer(norm(residual))`` -- the residual-stream form (add -> norm -> mixer)."""

    def _setup(self, norm, mixer, residual_in_fp32: bool):
        self.norm, self.mixer, self.residual_in_fp32 = norm, mixer, residual_in_fp32

    def forward(self, hidden_states, residual: Optional[torch.Tensor] = None, inference_params=None, **mixer_kwargs):
        fn = rms_norm_fn if isinstance(self.norm, RMSNorm) else layer_norm_fn
        hidden_states, residual = fn(hidden_states, self.norm.weight, self.norm.bias, residual=residual, prenorm=True,
                                     residual_in_fp32=self.residual_in_fp32, eps=self.norm.eps)
        return self.mixer(hidden_states, **mixer_kwargs), residual


class MambaBlock(_AddNormMixerBlock):
    def __init__(self, config, fused_add_norm: bool = True, residual_in_fp32: bool = True, norm_epsilon: float = 1e-5,
                 layer_idx: int = None, **factory_kwargs):
        super().__init__()
        self.fused_add_norm = fused_add_norm
        self._setup(RMSNorm(config.d_model, eps=norm_epsilon), Mamba(config.d_model, **factory_kwargs, **config.sequence_mixer.kwargs),
                    residual_in_fp32)


def MambaInit(module, n_layer, initializer_range: float = 0.02, rescale_prenorm_residual: bool = True, n_residuals_per_layer: int = 1):
    if isinstance(module, nn.Linear):
        if module.bias is not None and not getattr(module.bias, "_no_reinit", False):
            nn.init.zeros_(module.bias)
    elif isinstance(module, nn.Embedding):
        nn.init.normal_(module.weight, std=initializer_range)
    if rescale_prenorm_residual:
        for name, p in module.named_parameters():
            if "out_proj.weight" in name or "fc2.weight" in name:
                nn.init.kaiming_uniform_(p, a=math.sqrt(5))
                with torch.no_grad():
                    p /= math.sqrt(n_residuals_per_layer * n_layer)
