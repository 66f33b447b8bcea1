"""All iterations of the MIMO-Jacobi state update and its gated readout as one kernel (forward and backward).

``jacobi_iterate`` takes the iteration-independent maps of :class:`ml_experiments_b200.models.jacobi.MIMOJacobiSSM_ND`
(1-D grids) and returns ``rot(C, n theta) * H_n`` in the ``[batch, L, R * N]`` layout of the output projection. On CUDA
it runs ``csrc/scan/jacobi.cu`` (state of a sequence window resident in shared memory for all iterations; the backward
walks the saved per-iteration states in reverse); elsewhere, and for shapes the kernel does not take, the plain PyTorch
loop :func:`jacobi_iterate_torch`, which is also the oracle of the GPU test. Counterpart of the reference's per-iteration
operator chain (src/heuristic_secrets/models/scatter_attention.py:1416-1482) and its Triton step / rotation kernels
(triton_scatter.py:582-667).
"""
from __future__ import annotations

import os

import torch
import torch.nn.functional as F

_THREADS, _BWD_ITEMS = 512, 2


def kernel_supported(N: int, n_iters: int) -> bool:
    """State sizes 16 / 32 / 64 / 128; the backward window (``2 * 512 / (N / 4)`` positions) must keep a quarter of its
    width after ``n_iters - 1`` halo positions on each side (mirrors ``jacobi_supported`` of the extension)."""
    if N not in (16, 32, 64, 128) or n_iters < 1:
        return False
    w = _THREADS // (N // 4) * _BWD_ITEMS
    return w - 2 * (n_iters - 1) >= w // 4


def _rotate_pairs(x, theta):
    x1, x2 = x[..., 0::2], x[..., 1::2]
    cos, sin = theta.cos(), theta.sin()
    return torch.stack((x1 * cos - x2 * sin, x1 * sin + x2 * cos), dim=-1).flatten(-2)


def _mix(v, lam):
    h = v.shape[-1] // 2
    a, b = v[..., :h], v[..., h:]
    return torch.cat([a - lam * b, a + lam * b], dim=-1)


def jacobi_iterate_torch(Bm, Cm, theta, xr, alpha, gamma, conv_w, conv_b, inj_lambda, ro_lambda, n_iters: int):
    """``Bm, Cm: [b, R, L, N]``, ``theta: [b, L, N/2]``, ``xr: [b, R, L]``, ``alpha: [b, L, N]``, ``gamma: [b, L]``,
    ``conv_w: [N, 3]`` (taps at l-1, l, l+1), ``conv_b: [N]``; returns ``[b, L, R * N]``."""
    b, R, L, N = Bm.shape
    H = torch.zeros_like(Bm)
    prev = None
    th, al, gm, x = theta.unsqueeze(1), alpha.unsqueeze(1), gamma.view(b, 1, L, 1), xr.unsqueeze(-1)
    for it in range(n_iters):
        inj = _rotate_pairs(Bm, th * (it + 1)) * x
        if inj_lambda is not None:
            inj = _mix(inj, inj_lambda)
        flat = F.conv1d(H.reshape(b * R, L, N).transpose(1, 2), conv_w.view(N, 1, 3), conv_b, padding=1, groups=N).transpose(1, 2)
        H = flat.reshape(b, R, L, N)
        H = al * H + inj if prev is None else al * H + (1.0 - gm) * al * prev + gm * inj
        prev = inj
    g = _rotate_pairs(Cm, th * n_iters) * H
    if ro_lambda is not None:
        g = _mix(g, ro_lambda)
    return g.permute(0, 2, 1, 3).reshape(b, L, R * N)


class _JacobiFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, Bm, Cm, theta, xr, alpha, gamma, conv_w, conv_b, inj_lambda, ro_lambda, n_iters):
        from .runtime import add_launches, ops

        b, R, L, N = Bm.shape
        f = lambda t: None if t is None else t.detach().float()
        args = [f(Bm), f(Cm), f(theta).contiguous(), f(xr), f(alpha).contiguous(), f(gamma).contiguous().view(b, L),
                f(conv_w).contiguous().view(N, 3), f(conv_b).contiguous(), f(inj_lambda), f(ro_lambda)]
        need_grad = any(t is not None and t.requires_grad for t in (Bm, Cm, theta, xr, alpha, gamma, conv_w, conv_b, inj_lambda, ro_lambda))
        gated = torch.empty(b, L, R * N, device=Bm.device, dtype=torch.float32)
        Hs = torch.empty(n_iters, b, R, L, N, device=Bm.device, dtype=torch.float32) if need_grad else None
        ops().jacobi_fwd(*args, n_iters, gated, Hs)
        add_launches(1)
        if need_grad:
            ctx.save_for_backward(Hs, *[a for a in args if a is not None])
            ctx.has = (inj_lambda is not None, ro_lambda is not None)
            ctx.n_iters = n_iters
            ctx.dtypes = [None if t is None else t.dtype for t in (Bm, Cm, theta, xr, alpha, gamma, conv_w, conv_b, inj_lambda, ro_lambda)]
            ctx.shapes = (gamma.shape, conv_w.shape)
        return gated.to(Bm.dtype)

    @staticmethod
    def backward(ctx, dgated):
        from .runtime import add_launches, ops

        Hs, *rest = ctx.saved_tensors
        Bm, Cm, theta, xr, alpha, gamma, conv_w, conv_b = rest[:8]
        extra = list(rest[8:])
        inj_lambda = extra.pop(0) if ctx.has[0] else None
        ro_lambda = extra.pop(0) if ctx.has[1] else None
        b, R, L, N = Bm.shape
        dev = Bm.device
        new = lambda *s: torch.empty(*s, device=dev, dtype=torch.float32)
        dBm, dCm, dtheta, dxr = new(b, R, L, N), new(b, R, L, N), new(b, L, N // 2), new(b, R, L)
        dalpha, dgamma = new(b, L, N), new(b, L)
        small = torch.zeros(4 * N + 2, device=dev, dtype=torch.float32)      # taps, bias, the two mix weights: atomic sums
        dcw, dcb, dlam = small[:3 * N].view(N, 3), small[3 * N:4 * N], small[4 * N:]
        ops().jacobi_bwd(dgated.float().contiguous(), Hs, Bm, Cm, theta, xr, alpha, gamma, conv_w, conv_b, inj_lambda, ro_lambda,
                         ctx.n_iters, dBm, dCm, dtheta, dxr, dalpha, dgamma, dcw, dcb, dlam)
        add_launches(1)
        gshape, wshape = ctx.shapes
        outs = [dBm, dCm, dtheta, dxr, dalpha, dgamma.view(gshape), dcw.reshape(wshape), dcb,
                dlam[0].reshape(()) if ctx.has[0] else None, dlam[1].reshape(()) if ctx.has[1] else None]
        outs = [None if (o is None or dt is None) else o.to(dt) for o, dt in zip(outs, ctx.dtypes)]
        return (*outs, None)


def jacobi_iterate(Bm, Cm, theta, xr, alpha, gamma, conv_w, conv_b, inj_lambda=None, ro_lambda=None, n_iters: int = 12):
    """See :func:`jacobi_iterate_torch` for the shapes. ``B200_JACOBI_KERNEL=0`` forces the PyTorch loop."""
    use = (Bm.is_cuda and kernel_supported(Bm.shape[-1], n_iters) and os.environ.get("B200_JACOBI_KERNEL", "1") == "1")
    if not use:
        return jacobi_iterate_torch(Bm, Cm, theta, xr, alpha, gamma.reshape(Bm.shape[0], -1), conv_w.reshape(-1, 3), conv_b, inj_lambda, ro_lambda, n_iters)
    return _JacobiFn.apply(Bm, Cm, theta, xr, alpha, gamma, conv_w, conv_b, inj_lambda, ro_lambda, n_iters)
