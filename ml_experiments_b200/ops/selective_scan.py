"""S6 selective scan: CUDA kernels (tiles of 16 steps, state 16) with autograd, plus the plain-torch restatement.

Interface mirrors ``selective_scan_fn`` / ``selective_scan_ref`` of the reference
(zoology/mixers/mamba_ssm/ops/selective_scan_interface.py:19-157) but channel-last: ``u, delta, z`` are ``[B, L, Din]``,
``A`` is ``[Din, N]``, ``B, C`` are ``[B, L, N]`` (input-dependent, shared over channels), ``D`` is ``[Din]``.
``delta_softplus`` and ``delta_bias`` are applied before the kernel.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .runtime import ops

TILE = 16     # time steps per tile and per state checkpoint of the kernels (SUB in csrc/scan/s6_scan.cu)


def selective_scan_ref(u, delta, A, B, C, D=None, z=None, delta_bias=None, delta_softplus=False):
    """Sequential fp32 oracle (any device)."""
    dtype_in = u.dtype
    u, delta = u.float(), delta.float()
    if delta_bias is not None:
        delta = delta + delta_bias.float()
    if delta_softplus:
        delta = F.softplus(delta)
    Bf, Cf, Af = B.float(), C.float(), A.float()
    bsz, L, din = u.shape
    h = u.new_zeros(bsz, din, Af.shape[1])
    ys = []
    for t in range(L):
        dA = torch.exp(delta[:, t, :, None] * Af[None])
        h = dA * h + delta[:, t, :, None] * Bf[:, t, None, :] * u[:, t, :, None]
        ys.append((h * Cf[:, t, None, :]).sum(-1))
    y = torch.stack(ys, 1)
    if D is not None:
        y = y + u * D.float()
    if z is not None:
        y = y * F.silu(z.float())
    return y.to(dtype_in)


def set_states_per_thread(fwd: int = 2, bwd: int = 4, device="cuda") -> None:
    """States of a channel held per thread (2 or 4) by the forward and the backward scan kernel: 4 runs four warps per
    32-channel block, 2 runs eight (more warps per SM to hide the latency of the recurrence, more shared-memory
    traffic). The state checkpoints have one layout for both, so the two choices are independent."""
    ops().s6_set_states_per_thread(int(fwd), int(bwd), torch.empty(0, device=device))


class _S6Scan(torch.autograd.Function):
    """CUDA path: softplus / bias / gate and their backward all run inside the two kernels."""

    @staticmethod
    def forward(ctx, u, delta, A, B, C, D, z, delta_bias, delta_softplus):
        o = ops()
        bsz, L, din = u.shape
        n = A.shape[1]
        u16 = u.to(torch.bfloat16).contiguous()
        z16 = None if z is None else z.to(torch.bfloat16).contiguous()
        d32 = (delta if delta.dtype == torch.bfloat16 else delta.float()).contiguous()  # raw step, bf16 or fp32
        A32 = A.float().contiguous()
        B32, C32 = B.float().contiguous(), C.float().contiguous()
        D32 = None if D is None else D.float().contiguous()
        b32 = None if delta_bias is None else delta_bias.float().contiguous()
        need_grad = any(t is not None and t.requires_grad for t in (u, delta, A, B, C, D, z, delta_bias))
        state = torch.empty(bsz, (L + TILE - 1) // TILE, 4, din, 4, dtype=torch.float32, device=u.device) if need_grad else None
        y_pre = torch.empty_like(u16) if (need_grad and z16 is not None) else None
        out = torch.empty_like(u16)
        o.s6_scan_fwd(u16, d32, b32, bool(delta_softplus), A32, B32, C32, D32, z16, y_pre, out, state)
        ctx.save_for_backward(u16, d32, b32, A32, B32, C32, D32, z16, y_pre, state)
        ctx.softplus = bool(delta_softplus)
        ctx.dtypes = tuple(None if t is None else t.dtype for t in (u, delta, A, B, C, D, z, delta_bias))
        return out.to(u.dtype)

    @staticmethod
    def backward(ctx, dout):
        o = ops()
        u16, d32, b32, A32, B32, C32, D32, z16, y_pre, state = ctx.saved_tensors
        bsz, L, din = u16.shape
        n = A32.shape[1]
        dev = u16.device
        du = torch.empty_like(u16)
        ddelta = torch.empty_like(d32)
        dA = torch.zeros_like(A32)
        dBp = torch.empty(bsz, (din + 31) // 32, L, n, dtype=torch.float32, device=dev)
        dCp = torch.empty_like(dBp)
        dD = None if D32 is None else torch.zeros_like(D32)
        dz = None if z16 is None else torch.empty_like(z16)
        dbias = None if b32 is None else torch.zeros_like(b32)
        o.s6_scan_bwd(u16, d32, b32, ctx.softplus, A32, B32, C32, D32, z16, y_pre, dout.to(torch.bfloat16).contiguous(), state,
                      du, ddelta, dA, dBp, dCp, dD, dz, dbias)
        t = ctx.dtypes
        cast = lambda g, dt: None if g is None else g.to(dt)
        return (cast(du, t[0]), cast(ddelta, t[1]), cast(dA, t[2]), cast(dBp.sum(1), t[3]), cast(dCp.sum(1), t[4]), cast(dD, t[5]),
                cast(dz, t[6]), cast(dbias, t[7]), None)


def selective_scan(u, delta, A, B, C, D=None, z=None, delta_bias=None, delta_softplus=False):
    """Differentiable S6 scan; CUDA kernels when ``u`` is on a GPU and ``N == 16``, the oracle otherwise."""
    if not u.is_cuda or A.shape[1] != 16:
        return selective_scan_ref(u, delta, A, B, C, D, z, delta_bias, delta_softplus)
    return _S6Scan.apply(u, delta, A, B, C, D, z, delta_bias, delta_softplus)


def selective_state_update(state, x, dt, A, B, C, D=None, z=None, dt_bias=None, dt_softplus: bool = False):
    """One decode step of the S6 recurrence, in place on ``state [B, Din, N]`` (the ``selective_state_update`` Triton
    kernel of the reference, zoology/mixers/mamba_ssm/ops/triton/selective_state_update.py): ``x, dt, z [B, Din]``,
    ``A [Din, N]``, ``B, C [B, N]``, ``D, dt_bias [Din]``. Returns ``y [B, Din]``. A handful of fused elementwise
    kernels; one token per sequence is launch-bound, not bandwidth-bound."""
    dt = dt.float()
    if dt_bias is not None:
        dt = dt + dt_bias.float()
    if dt_softplus:
        dt = F.softplus(dt)
    dA = torch.exp(dt.unsqueeze(-1) * A.float())
    dBx = (dt * x.float()).unsqueeze(-1) * B.float().unsqueeze(1)
    state.copy_(state.float() * dA + dBx)
    y = (state.float() * C.float().unsqueeze(1)).sum(-1)
    if D is not None:
        y = y + x.float() * D.float()
    if z is not None:
        y = y * F.silu(z.float())
    return y.to(x.dtype)


def causal_conv1d_update(x, conv_state, weight, bias=None, activation: str | None = None):
    """One decode step of a causal depthwise conv: ``x [B, C]``, ``conv_state [B, C, K]`` (shifted in place),
    ``weight [C, K]``."""
    conv_state.copy_(torch.roll(conv_state, shifts=-1, dims=-1))
    conv_state[:, :, -1] = x
    y = (conv_state.float() * weight.float()).sum(-1)
    if bias is not None:
        y = y + bias.float()
    return (F.silu(y) if activation in ("silu", "swish") else y).to(x.dtype)
