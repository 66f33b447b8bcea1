"""MIMO Jacobi SSM: an iterated diffusion-style state-space operator on ``(B, *spatial, C)`` grids.

State ``H: (B, R, *spatial, N)`` for ``R`` input groups of ``N`` states. Iteration ``i`` recomputes the input / output
maps ``B, C = act(Linear(x) + bias)`` (optionally RMS-normed), rotates them by ``theta(x) * (i + 1)`` (interleaved-pair
rotary), injects ``B * X_r``, diffuses the state over the grid with a depthwise 3-tap convolution (optionally followed by
squeeze-excite) and blends with a trapezoidal rule ``H <- alpha H + (1 - lambda) alpha inject_prev + lambda inject``
with data-dependent decay ``alpha`` and ``lambda``; the readout is ``act(out_proj(C * H))``. ``diff_inject`` /
``diff_readout`` split the state in halves and mix sum and difference. Follows ``MIMOJacobiSSM_ND`` of the reference
(src/heuristic_secrets/models/scatter_attention.py:1316-1499). ``init_state`` / ``step`` run one iteration at a time,
which the reference's layer-wise Ripple models call (:1659, 1727, 1800, 1878) but its SSM never defined.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F


def _relu_squared(x):
    return F.relu(x).square()


class _RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x):
        return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + self.eps) * self.weight


class _SqueezeExcite(nn.Module):
    def __init__(self, channels: int, reduction: int = 4, relu2: bool = False):
        super().__init__()
        hidden = max(channels // reduction, 8)
        self.fc1 = nn.Linear(channels, hidden, bias=False)
        self.fc2 = nn.Linear(hidden, channels, bias=False)
        self.act = _relu_squared if relu2 else F.silu

    def forward(self, x):
        scale = torch.sigmoid(self.fc2(self.act(self.fc1(x.mean(dim=tuple(range(1, x.dim() - 1)))))))
        return x * scale.view(x.shape[0], *([1] * (x.dim() - 2)), -1)


def _rotate_pairs(x, theta):
    x1, x2 = x[..., 0::2], x[..., 1::2]
    cos, sin = theta.cos(), theta.sin()
    return torch.stack((x1 * cos - x2 * sin, x1 * sin + x2 * cos), dim=-1).flatten(-2)


class MIMOJacobiSSM_ND(nn.Module):
    def __init__(self, dim: int, state_dim: int = 64, mimo_rank: int = 4, ndim: int = 2, n_iters: int = 12, diffuse_se: bool = False,
                 diff_inject: bool = False, diff_readout: bool = False, bc_norm: bool = False, relu2: bool = False):
        super().__init__()
        self.D, self.N, self.R, self.ndim, self.n_iters = dim, state_dim, mimo_rank, ndim, n_iters
        self.diff_inject, self.diff_readout, self.bc_norm = diff_inject, diff_readout, bc_norm
        self.act = _relu_squared if relu2 else F.silu
        self.to_B = nn.Linear(dim, state_dim * mimo_rank)
        self.to_C = nn.Linear(dim, state_dim * mimo_rank)
        self.to_X = nn.Linear(dim, mimo_rank)
        self.to_decay = nn.Linear(dim, state_dim)
        self.to_theta = nn.Linear(dim, state_dim // 2)
        self.to_lambda = nn.Linear(dim, 1)
        self.B_bias = nn.Parameter(torch.ones(state_dim * mimo_rank))
        self.C_bias = nn.Parameter(torch.ones(state_dim * mimo_rank))
        if diff_inject:
            self.inject_lambda = nn.Parameter(torch.tensor(0.5))
        if diff_readout:
            self.readout_lambda = nn.Parameter(torch.tensor(0.5))
        if bc_norm:
            self.b_norm, self.c_norm = _RMSNorm(state_dim), _RMSNorm(state_dim)
        self.diffuse = (nn.Conv1d, nn.Conv2d, nn.Conv3d)[ndim - 1](state_dim, state_dim, kernel_size=3, padding=1, groups=state_dim)
        self.diffuse_se = _SqueezeExcite(state_dim, relu2=relu2) if diffuse_se else None
        self.out_proj = nn.Linear(state_dim * mimo_rank, dim)

    def init_state(self, x):
        """``(H, previous injection)``; both zero."""
        H = torch.zeros(x.shape[0], self.R, *x.shape[1:-1], self.N, device=x.device, dtype=x.dtype)
        return H, None

    def _project(self, x):
        """Everything ``_maps`` computes that does not depend on the iteration (the input does not change between
        iterations, so the five projections are evaluated once per call instead of once per iteration)."""
        B, spatial = x.shape[0], tuple(x.shape[1:-1])
        nd = len(spatial)
        to_br = (0, nd + 2) + tuple(range(1, nd + 1)) + (nd + 1,)  # (B, *sp, N, R) -> (B, R, *sp, N)
        Bm = self.act(self.to_B(x) + self.B_bias).view(B, *spatial, self.N, self.R).permute(*to_br)
        Cm = self.act(self.to_C(x) + self.C_bias).view(B, *spatial, self.N, self.R).permute(*to_br)
        if self.bc_norm:
            Bm, Cm = self.b_norm(Bm), self.c_norm(Cm)
        xr = self.act(self.to_X(x)).movedim(-1, 1).unsqueeze(-1)  # (B, R, *sp, 1)
        return Bm, Cm, self.to_theta(x).unsqueeze(1), xr, torch.sigmoid(self.to_decay(x)).unsqueeze(1), torch.sigmoid(self.to_lambda(x)).unsqueeze(1)

    def _maps(self, x, it: int, proj=None):
        Bm, Cm, theta, xr, alpha, gamma = self._project(x) if proj is None else proj
        theta = theta * (it + 1)
        Bm, Cm = _rotate_pairs(Bm, theta), _rotate_pairs(Cm, theta)
        if self.diff_inject:
            h = self.N // 2
            i1, i2 = Bm[..., :h] * xr, Bm[..., h:] * xr
            inject = torch.cat([i1 - self.inject_lambda * i2, i1 + self.inject_lambda * i2], dim=-1)
        else:
            inject = Bm * xr
        return inject, alpha, gamma, Cm

    def _diffuse_state(self, H):
        B, spatial = H.shape[0], tuple(H.shape[2:-1])
        flat = self.diffuse(H.reshape(B * self.R, *spatial, self.N).movedim(-1, 1)).movedim(1, -1)
        if self.diffuse_se is not None:
            flat = self.diffuse_se(flat)
        return flat.reshape(H.shape)

    def _readout(self, H, Cm):
        B, spatial = H.shape[0], tuple(H.shape[2:-1])
        if self.diff_readout:
            h = self.N // 2
            g1, g2 = Cm[..., :h] * H[..., :h], Cm[..., h:] * H[..., h:]
            gated = torch.cat([g1 - self.readout_lambda * g2, g1 + self.readout_lambda * g2], dim=-1)
        else:
            gated = Cm * H
        return self.act(self.out_proj(gated.movedim(1, -2).reshape(B, *spatial, self.R * self.N)))

    def _iterate(self, x, H, prev, it: int, proj=None):
        inject, alpha, gamma, Cm = self._maps(x, it, proj)
        H = self._diffuse_state(H)
        H = alpha * H + inject if prev is None else alpha * H + (1.0 - gamma) * alpha * prev + gamma * inject
        return H, inject, Cm

    def step(self, x, state, it: int):
        """One iteration driven by ``x``: returns ``((H, injection), readout)``."""
        H, prev = state
        H, inject, Cm = self._iterate(x, H, prev, it)
        return (H, inject), self._readout(H, Cm)

    def forward(self, x):
        proj = self._project(x)
        if x.is_cuda and self.ndim == 1 and x.dim() == 3 and self.diffuse_se is None:
            # 1-D grids without the squeeze-excite (a global mean per iteration) run every iteration in one kernel
            from ..ops.jacobi_iter import jacobi_iterate, kernel_supported
            if kernel_supported(self.N, self.n_iters):
                Bm, Cm, theta, xr, alpha, gamma = proj
                gated = jacobi_iterate(Bm, Cm, theta.squeeze(1), xr.squeeze(-1), alpha.squeeze(1), gamma.squeeze(1).squeeze(-1),
                                       self.diffuse.weight, self.diffuse.bias, self.inject_lambda if self.diff_inject else None,
                                       self.readout_lambda if self.diff_readout else None, self.n_iters)
                return self.act(self.out_proj(gated))
        H, prev = self.init_state(x)
        Cm = None
        for it in range(self.n_iters):
            H, prev, Cm = self._iterate(x, H, prev, it, proj)
        return self._readout(H, Cm)


class MIMOJacobiSSM(MIMOJacobiSSM_ND):
    def __init__(self, dim: int, state_dim: int = 64, mimo_rank: int = 4, n_iters: int = 12, diffuse_se: bool = False,
                 diff_inject: bool = False, diff_readout: bool = False, bc_norm: bool = False, relu2: bool = False):
        super().__init__(dim, state_dim, mimo_rank, ndim=1, n_iters=n_iters, diffuse_se=diffuse_se, diff_inject=diff_inject,
                         diff_readout=diff_readout, bc_norm=bc_norm, relu2=relu2)


class MIMOJacobiBlock_ND(nn.Module):
    """``x + ssm(norm(x))`` (scatter_attention.py:1502-1529)."""

    def __init__(self, dim: int, state_dim: int = 64, mimo_rank: int = 4, ndim: int = 2, n_iters: int = 12, eps: float = 1e-6):
        super().__init__()
        self.norm = _RMSNorm(dim, eps)
        self.ssm = MIMOJacobiSSM_ND(dim, state_dim, mimo_rank, ndim, n_iters)

    def forward(self, x):
        return x + self.ssm(self.norm(x))


class MIMOJacobiBlock(MIMOJacobiBlock_ND):
    def __init__(self, dim: int, state_dim: int = 64, mimo_rank: int = 4, n_iters: int = 12, eps: float = 1e-6):
        super().__init__(dim, state_dim, mimo_rank, ndim=1, n_iters=n_iters, eps=eps)
