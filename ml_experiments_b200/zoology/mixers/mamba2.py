"""Mamba-2 (SSD) mixer and block (zoology/mixers/mamba2.py:25-310).

in_proj -> (z0, x0, z, xBC, dt); causal conv + SiLU over xBC; per-head scalar decay ``exp(dt * A)`` with
``dt = softplus(dt + dt_bias)``; grouped B / C; ``y = SSD(x * dt, B, C) + D x``; gated RMS norm; out_proj. The scan is
``ops.ssd_scan.ssd_chunk_scan`` (all chunks at once on batched GEMMs) where the reference chains five Triton kernels
(zoology/mixers/mamba_ssm/ops/triton/ssd_combined.py:281-332). ``sequence_parallel`` / ``process_group`` are accepted
for signature compatibility; as in the reference no collective is issued.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...ops.ssd_scan import ssd_chunk_scan
from .mamba import _AddNormMixerBlock
from .norms import RMSNorm, RMSNormGated


def mamba_chunk_scan_combined(x, dt, A, B, C, chunk_size: int = 64, D=None, z=None, dt_bias=None, dt_softplus: bool = False,
                              dt_limit=(0.0, float("inf")), return_final_states: bool = False, initial_states=None, **kwargs):
    """``x [b,l,h,p]``, ``dt [b,l,h]``, ``A [h]``, ``B, C [b,l,g,n]`` -> ``y [b,l,h,p]`` (+ final state ``[b,h,p,n]``)."""
    b, l, h, p = x.shape
    g = B.shape[2]
    dt = dt.float()
    if dt_bias is not None:
        dt = dt + dt_bias.float()
    if dt_softplus:
        dt = F.softplus(dt)
    if dt_limit != (0.0, float("inf")):
        dt = dt.clamp(*dt_limit)
    rep = h // g
    Bh = B if g == h or g == 1 else B.repeat_interleave(rep, dim=2)
    Ch = C if g == h or g == 1 else C.repeat_interleave(rep, dim=2)
    init = None if initial_states is None else initial_states.transpose(-1, -2)
    out = ssd_chunk_scan(x, Bh, Ch, dt * A.float(), gamma=dt, chunk=min(chunk_size, 128), init_state=init, return_state=return_final_states)
    y, state = out if return_final_states else (out, None)
    if D is not None:
        y = y + x * (D.view(h, -1) if D.dim() > 0 else D).to(y.dtype).view(1, 1, h, -1)
    if z is not None:
        y = y * F.silu(z)
    return (y, state.transpose(-1, -2)) if return_final_states else y


class Mamba2(nn.Module):
    def __init__(self, d_model, d_state=128, d_conv=4, conv_init=None, expand=2, headdim=64, d_ssm=None, ngroups=1,
                 A_init_range=(1, 16), D_has_hdim=False, rmsnorm=True, norm_before_gate=False, dt_min=0.001, dt_max=0.1,
                 dt_init_floor=1e-4, dt_limit=(0.0, float("inf")), bias=False, conv_bias=True, chunk_size=256, use_mem_eff_path=False,
                 layer_idx=None, process_group=None, sequence_parallel=True, device=None, dtype=None, use_fast_path=True,
                 num_feature_maps=1):
        fk = {"device": device, "dtype": dtype}
        super().__init__()
        self.d_model, self.d_state, self.d_conv, self.expand, self.headdim = d_model, d_state, d_conv, expand, headdim
        self.process_group, self.sequence_parallel = process_group, sequence_parallel
        self.d_inner = expand * d_model
        self.d_ssm = self.d_inner if d_ssm is None else d_ssm
        self.ngroups = ngroups
        assert self.d_ssm % headdim == 0
        self.nheads = self.d_ssm // headdim
        self.D_has_hdim, self.rmsnorm, self.norm_before_gate, self.dt_limit = D_has_hdim, rmsnorm, norm_before_gate, tuple(dt_limit)
        self.activation, self.chunk_size, self.layer_idx = "silu", chunk_size, layer_idx
        self.in_proj = nn.Linear(d_model, 2 * self.d_inner + 2 * ngroups * d_state + self.nheads, bias=bias, **fk)
        conv_dim = self.d_ssm + 2 * ngroups * d_state
        self.conv1d = nn.Conv1d(conv_dim, conv_dim, bias=conv_bias, kernel_size=d_conv, groups=conv_dim, padding=d_conv - 1, **fk)
        if conv_init is not None:
            nn.init.uniform_(self.conv1d.weight, -conv_init, conv_init)
        self.act = nn.SiLU()
        dt = torch.exp(torch.rand(self.nheads, **fk) * (math.log(dt_max) - math.log(dt_min)) + math.log(dt_min)).clamp(min=dt_init_floor)
        self.dt_bias = nn.Parameter(dt + torch.log(-torch.expm1(-dt)))
        self.dt_bias._no_weight_decay = True
        assert 0 < A_init_range[0] <= A_init_range[1]
        self.A_log = nn.Parameter(torch.log(torch.empty(self.nheads, dtype=torch.float32, device=device).uniform_(*A_init_range)))
        self.A_log._no_weight_decay = True
        self.D = nn.Parameter(torch.ones(self.d_ssm if D_has_hdim else self.nheads, device=device))
        self.D._no_weight_decay = True
        if rmsnorm:
            self.norm = RMSNormGated(self.d_ssm, eps=1e-5, norm_before_gate=norm_before_gate, group_size=self.d_ssm // ngroups, **fk)
        self.out_proj = nn.Linear(self.d_inner, d_model, bias=bias, **fk)

    def forward(self, u, seqlen=None, seq_idx=None, cu_seqlens=None, inference_params=None):
        flat = seqlen is not None
        if flat:
            u = u.view(-1, seqlen, u.shape[-1])
        b, L, _ = u.shape
        zxbcdt = self.in_proj(u)
        gs = self.ngroups * self.d_state
        d_mlp = (zxbcdt.shape[-1] - 2 * self.d_ssm - 2 * gs - self.nheads) // 2
        z0, x0, z, xBC, dt = torch.split(zxbcdt, [d_mlp, d_mlp, self.d_ssm, self.d_ssm + 2 * gs, self.nheads], dim=-1)
        xBC = self.act(self.conv1d(xBC.transpose(1, 2))[..., :L].transpose(1, 2))
        x, B, C = torch.split(xBC, [self.d_ssm, gs, gs], dim=-1)
        D = self.D.view(self.nheads, self.headdim) if self.D_has_hdim else self.D
        y = mamba_chunk_scan_combined(
            x.unflatten(-1, (self.nheads, self.headdim)), dt, -torch.exp(self.A_log.float()),
            B.unflatten(-1, (self.ngroups, self.d_state)), C.unflatten(-1, (self.ngroups, self.d_state)), chunk_size=self.chunk_size, D=D,
            z=None if self.rmsnorm else z.unflatten(-1, (self.nheads, self.headdim)), dt_bias=self.dt_bias, dt_softplus=True,
            dt_limit=self.dt_limit).flatten(-2)
        if self.rmsnorm:
            y = self.norm(y, z)
        if d_mlp > 0:
            y = torch.cat([F.silu(z0) * x0, y], dim=-1)
        out = self.out_proj(y.to(u.dtype))
        return out.flatten(0, 1) if flat else out

    def state_size(self, sequence_length: int = 2048):
        return 2 * self.d_model * self.d_state


class Mamba2Block(_AddNormMixerBlock):
    def __init__(self, config, norm_cls=RMSNorm, fused_add_norm: bool = False, residual_in_fp32: bool = False, use_fast_path: bool = True,
                 layer_idx: int = None, **kwargs):
        super().__init__()
        self.fused_add_norm, self.mlp = fused_add_norm, None
        self._setup(norm_cls(config.d_model), Mamba2(config.d_model, use_fast_path=use_fast_path, **config.sequence_mixer.kwargs),
                    residual_in_fp32)
