"""S6 selective scan: CUDA kernels (chunk 64, state 16) with autograd, plus the plain-torch restatement.

Interface mirrors ``selective_scan_fn`` / ``selective_scan_ref`` of the reference
(zoology/mixers/mamba_ssm/ops/selective_scan_interface.py:19-157) but channel-last: ``u, delta, z`` are ``[B, L, Din]``,
``A`` is ``[Din, N]``, ``B, C`` are ``[B, L, N]`` (input-dependent, shared over channels), ``D`` is ``[Din]``.
``delta_softplus`` and ``delta_bias`` are applied before the kernel.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .runtime import ops


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


class _S6Scan(torch.autograd.Function):
    @staticmethod
    def forward(ctx, u, delta, A, B, C, D, z):
        o = ops()
        bsz, L, din = u.shape
        n = A.shape[1]
        u16 = u.to(torch.bfloat16).contiguous()
        z16 = None if z is None else z.to(torch.bfloat16).contiguous()
        d32, A32 = delta.float().contiguous(), A.float().contiguous()
        B32, C32 = B.float().contiguous(), C.float().contiguous()
        D32 = None if D is None else D.float().contiguous()
        nch = (L + 63) // 64
        state = torch.empty(bsz, nch, din, n, dtype=torch.float32, device=u.device)
        y_pre = torch.empty_like(u16)
        out = torch.empty_like(u16)
        o.s6_scan_fwd(u16, d32, A32, B32, C32, D32, z16, y_pre, out, state)
        ctx.save_for_backward(u16, d32, A32, B32, C32, D32, z16, y_pre, state)
        ctx.dtypes = (u.dtype, delta.dtype, A.dtype, B.dtype, C.dtype, None if D is None else D.dtype,
                      None if z is None else z.dtype)
        return out.to(u.dtype)

    @staticmethod
    def backward(ctx, dout):
        o = ops()
        u16, d32, A32, B32, C32, D32, z16, y_pre, state = ctx.saved_tensors
        bsz, L, din = u16.shape
        n = A32.shape[1]
        dout = dout.float()
        dz = None
        if z16 is not None:
            zf = z16.float()
            sig = torch.sigmoid(zf)
            dz = dout * y_pre.float() * (sig * (1 + zf * (1 - sig)))
            dy = (dout * zf * sig).to(torch.bfloat16).contiguous()
        else:
            dy = dout.to(torch.bfloat16).contiguous()
        nblk = (din + 15) // 16
        du = torch.empty_like(u16)
        ddelta = torch.empty_like(d32)
        dA = torch.zeros_like(A32)
        dBp = torch.empty(bsz, nblk, L, n, dtype=torch.float32, device=u16.device)
        dCp = torch.empty_like(dBp)
        dD = None if D32 is None else torch.zeros_like(D32)
        o.s6_scan_bwd(u16, d32, A32, B32, C32, D32, dy, state, du, ddelta, dA, dBp, dCp, dD)
        t = ctx.dtypes
        return (du.to(t[0]), ddelta.to(t[1]), dA.to(t[2]), dBp.sum(1).to(t[3]), dCp.sum(1).to(t[4]),
                None if dD is None else dD.to(t[5]), None if dz is None else dz.to(t[6]))


def selective_scan(u, delta, A, B, C, D=None, z=None, delta_bias=None, delta_softplus=False):
    """Differentiable S6 scan; CUDA kernels when ``u`` is on a GPU and ``N == 16``, the oracle otherwise."""
    if not u.is_cuda or A.shape[1] != 16:
        return selective_scan_ref(u, delta, A, B, C, D, z, delta_bias, delta_softplus)
    if delta_bias is not None:
        delta = delta + delta_bias
    if delta_softplus:
        delta = F.softplus(delta.float())
    return _S6Scan.apply(u, delta, A, B, C, D, z)
