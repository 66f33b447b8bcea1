"""S6 (Mamba-1) selective-scan language model: pre-norm residual blocks of

``in_proj (d -> 2 d_inner) -> causal depthwise conv k=4 + SiLU -> x_proj -> (dt_rank, B, C) -> dt_proj + softplus
-> selective scan (A = -exp(A_log), D skip) -> * silu(z) -> out_proj``.

Block structure, parameter names and initialisation follow the reference mixers
(zoology/mixers/mamba.py:21-198; src/heuristic_secrets/models/backbone.py:1100-1246 ``SSMMixer``): ``A_log = log(1..N)``
per channel, ``D = 1``, ``dt_proj.bias`` such that softplus(bias) is log-uniform in [1e-3, 1e-1]. The LM wrapper (token
embedding, tied head, final norm) follows zoology/model.py:218-263. Projections run on the tcgen05 GEMM and the scan on
the S6 kernels when the model lives on a GPU.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops.causal_conv import causal_conv1d_silu
from ..ops.norm_act import rms_norm_act, rms_norm_act_skip
from ..ops.linear import linear, linear_pair, linear_tee
from ..ops.selective_scan import selective_scan


@dataclass
class S6Config:
    vocab_size: int = 256
    d_model: int = 1024
    n_layers: int = 24
    expand: int = 2
    d_state: int = 16
    d_conv: int = 4
    dt_rank: int | None = None
    chunk_size: int = 64
    dt_min: float = 1e-3
    dt_max: float = 1e-1
    tie_embeddings: bool = True

    @property
    def d_inner(self) -> int:
        return self.expand * self.d_model

    @property
    def rank(self) -> int:
        return self.dt_rank if self.dt_rank is not None else math.ceil(self.d_model / 16)


class RMSNorm(nn.Module):
    def __init__(self, d: int, eps: float = 1e-5):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(d))

    def forward(self, x):
        if x.is_cuda:  # one kernel forward, one backward
            return rms_norm_act(x, self.weight, self.eps)
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)).to(x.dtype) * self.weight.to(x.dtype)


class S6Mixer(nn.Module):
    def __init__(self, cfg: S6Config):
        super().__init__()
        self.cfg = cfg
        di, n, r = cfg.d_inner, cfg.d_state, cfg.rank
        self.in_proj = nn.Linear(cfg.d_model, 2 * di, bias=False)
        self.conv1d = nn.Conv1d(di, di, cfg.d_conv, groups=di, padding=cfg.d_conv - 1, bias=True)
        self.x_proj = nn.Linear(di, r + 2 * n, bias=False)
        self.dt_proj = nn.Linear(r, di, bias=True)
        std = r ** -0.5
        nn.init.uniform_(self.dt_proj.weight, -std, std)
        dt = torch.exp(torch.rand(di) * (math.log(cfg.dt_max) - math.log(cfg.dt_min)) + math.log(cfg.dt_min)).clamp(min=1e-4)
        with torch.no_grad():
            self.dt_proj.bias.copy_(dt + torch.log(-torch.expm1(-dt)))  # inverse softplus
        self.A_log = nn.Parameter(torch.log(torch.arange(1, n + 1, dtype=torch.float32)).repeat(di, 1))
        self.D = nn.Parameter(torch.ones(di))
        self.out_proj = nn.Linear(di, cfg.d_model, bias=False)

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:  # (B, L, d_model)
        """``residual`` (the block's skip connection) is added in the epilogue of the output projection."""
        cfg = self.cfg
        L = x.shape[1]
        # the two halves of in_proj as two GEMMs on row ranges of its weight (one autograd node): the scan needs x and the
        # gate z as separate contiguous tensors, and one wide GEMM would cost a strided-to-contiguous copy of each half in
        # the forward and a concatenation of their gradients in the backward
        di = cfg.d_inner
        xi, z = linear_pair(x, self.in_proj.weight, di)
        xi = causal_conv1d_silu(xi, self.conv1d.weight, self.conv1d.bias)
        dbc, xi = linear_tee(xi, self.x_proj.weight)   # the scan's gradient of xi is added in x_proj's backward GEMM
        dt, Bm, Cm = torch.split(dbc, [cfg.rank, cfg.d_state, cfg.d_state], dim=-1)
        y = selective_scan(xi.contiguous(), linear(dt, self.dt_proj.weight), -torch.exp(self.A_log.float()), Bm, Cm, self.D,
                           z, delta_bias=self.dt_proj.bias, delta_softplus=True)
        return linear(y, self.out_proj.weight, residual=residual)


class S6Block(nn.Module):
    def __init__(self, cfg: S6Config):
        super().__init__()
        self.norm = RMSNorm(cfg.d_model)
        self.mixer = S6Mixer(cfg)

    def forward(self, x):
        if x.is_cuda:   # the skip's gradient joins the norm's inside the norm's backward kernel
            h, skip = rms_norm_act_skip(x, self.norm.weight, self.norm.eps)
            return self.mixer(h, residual=skip)
        return self.mixer(self.norm(x), residual=x)


class S6LM(nn.Module):
    def __init__(self, cfg: S6Config | None = None, **kw):
        super().__init__()
        self.cfg = cfg = cfg or S6Config(**kw)
        self.embedding = nn.Embedding(cfg.vocab_size, cfg.d_model)
        self.layers = nn.ModuleList([S6Block(cfg) for _ in range(cfg.n_layers)])
        self.norm_f = RMSNorm(cfg.d_model)
        self.lm_head = nn.Linear(cfg.d_model, cfg.vocab_size, bias=False)
        if cfg.tie_embeddings:
            self.lm_head.weight = self.embedding.weight
        nn.init.normal_(self.embedding.weight, std=0.02)
        for name, p in self.named_parameters():
            if name.endswith("out_proj.weight"):
                nn.init.normal_(p, std=0.02 / math.sqrt(2 * cfg.n_layers))

    def forward(self, ids: torch.Tensor, targets: torch.Tensor | None = None):
        x = self.embedding(ids)
        for layer in self.layers:
            x = layer(x)
        logits = linear(self.norm_f(x), self.lm_head.weight)
        if targets is None:
            return logits
        return F.cross_entropy(logits.float().view(-1, logits.shape[-1]), targets.reshape(-1), ignore_index=-100)
