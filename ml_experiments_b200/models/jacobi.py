"""MIMO Jacobi SSM: an iterated diffusion-style state-space operator.

State ``H: (B, R, L, N)`` for ``R`` input groups; every iteration recomputes input / output maps ``B, C`` from the
sequence, injects ``B * X_r``, diffuses the state along the sequence with a depthwise 3-tap convolution and blends with
a trapezoidal rule ``H <- alpha * H + beta * H_prev + gamma * inject``; the readout is ``act(out_proj(C * H))``.
Follows the 1-D case of the reference's ``MIMOJacobiSSM_ND`` (src/heuristic_secrets/models/scatter_attention.py:1316-1499)
with its default options; the N-D and rope-per-iteration options are not reproduced.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F


class MIMOJacobiSSM(nn.Module):
    def __init__(self, channels: int, n_state: int = 16, n_groups: int = 4, n_iters: int = 12, diffuse_se: bool = False,
                 diff_inject: bool = False, diff_readout: bool = False, bc_norm: bool = False, relu2: bool = False):
        super().__init__()
        self.channels, self.n_state, self.n_groups, self.n_iters = channels, n_state, n_groups, n_iters
        self.act = (lambda t: F.relu(t).square()) if relu2 else F.silu
        self.in_proj = nn.Linear(channels, n_groups)
        self.b_proj = nn.Linear(channels, n_groups * n_state)
        self.c_proj = nn.Linear(channels, n_groups * n_state)
        self.diffuse = nn.Conv1d(n_groups * n_state, n_groups * n_state, 3, padding=1, groups=n_groups * n_state, bias=False)
        with torch.no_grad():
            self.diffuse.weight.copy_(torch.tensor([0.25, 0.5, 0.25]).view(1, 1, 3).expand_as(self.diffuse.weight))
        self.log_dt = nn.Parameter(torch.zeros(n_groups))
        self.lam = nn.Parameter(torch.zeros(n_groups))
        self.out_proj = nn.Linear(n_groups * n_state, channels)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        Bsz, L, _ = x.shape
        R, N = self.n_groups, self.n_state
        xr = self.in_proj(x)                                                  # (B, L, R)
        Bm = self.act(self.b_proj(x)).view(Bsz, L, R, N)
        Cm = self.act(self.c_proj(x)).view(Bsz, L, R, N)
        dt = F.softplus(self.log_dt).view(1, 1, R, 1)
        lam = torch.sigmoid(self.lam).view(1, 1, R, 1)
        alpha = torch.exp(-dt)
        beta, gamma = (1 - lam) * dt * alpha, lam * dt
        inject = Bm * xr.unsqueeze(-1)
        H = torch.zeros_like(inject)
        prev = torch.zeros_like(inject)
        for _ in range(self.n_iters):
            Hd = self.diffuse(H.reshape(Bsz, L, R * N).transpose(1, 2)).transpose(1, 2).reshape(Bsz, L, R, N)
            H, prev = alpha * Hd + beta * prev + gamma * inject, inject
        return self.act(self.out_proj((Cm * H).reshape(Bsz, L, R * N)))
