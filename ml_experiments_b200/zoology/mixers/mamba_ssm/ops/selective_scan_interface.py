"""``selective_scan_fn`` / ``selective_scan_ref`` / ``mamba_inner_fn`` / ``mamba_inner_ref`` with the reference's
channel-first signatures (zoology/mixers/mamba_ssm/ops/selective_scan_interface.py:82-157,311-360):
``u, delta, z [batch, dim, L]``, ``A [dim, dstate]``, ``B, C [batch, dstate, L]`` (or ``[batch, 1, dstate, L]``),
``D, delta_bias [dim]``. The work is done by :mod:`ml_experiments_b200.ops.selective_scan` on channel-last views."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from ml_experiments_b200.ops.causal_conv import causal_conv1d_silu
from ml_experiments_b200.ops.selective_scan import selective_scan as _scan_cl
from ml_experiments_b200.ops.selective_scan import selective_scan_ref as _scan_ref_cl


def _bc_channel_last(t: torch.Tensor) -> torch.Tensor:
    if t.dim() == 4:
        if t.shape[1] != 1:
            raise NotImplementedError("selective scan: grouped B / C (more than one group) is not supported")
        t = t[:, 0]
    return t.transpose(1, 2)


def _last_state(u, delta, A, B, delta_bias, delta_softplus):
    """State after the last step, ``[batch, dim, dstate]`` (only computed when the caller asks for it)."""
    d = delta.float() + (0 if delta_bias is None else delta_bias.float()[None, :, None])
    d = F.softplus(d) if delta_softplus else d
    Bc = _bc_channel_last(B).float()                                   # [b, L, n]
    h = u.new_zeros(u.shape[0], u.shape[1], A.shape[1], dtype=torch.float32)
    for t in range(u.shape[2]):
        h = torch.exp(d[:, :, t, None] * A.float()) * h + (d[:, :, t] * u[:, :, t].float()).unsqueeze(-1) * Bc[:, t, None, :]
    return h


def _run(scan, u, delta, A, B, C, D, z, delta_bias, delta_softplus, return_last_state):
    cl = lambda t: None if t is None else t.transpose(1, 2).contiguous()
    y = scan(cl(u), cl(delta), A, _bc_channel_last(B).contiguous(), _bc_channel_last(C).contiguous(), D, cl(z), delta_bias, delta_softplus)
    y = y.transpose(1, 2)
    return (y, _last_state(u, delta, A, B, delta_bias, delta_softplus)) if return_last_state else y


def selective_scan_fn(u, delta, A, B, C, D=None, z=None, delta_bias=None, delta_softplus=False, return_last_state=False):
    return _run(_scan_cl, u, delta, A, B, C, D, z, delta_bias, delta_softplus, return_last_state)


def selective_scan_ref(u, delta, A, B, C, D=None, z=None, delta_bias=None, delta_softplus=False, return_last_state=False):
    return _run(_scan_ref_cl, u, delta, A, B, C, D, z, delta_bias, delta_softplus, return_last_state)


def mamba_inner_ref(xz, conv1d_weight, conv1d_bias, x_proj_weight, delta_proj_weight, out_proj_weight, out_proj_bias, A, B=None, C=None,
                    D=None, delta_bias=None, B_proj_bias=None, C_proj_bias=None, delta_softplus=True, _scan=_scan_ref_cl):
    """The whole inner block of the S6 mixer from the in-projection's output ``xz [batch, 2 dim, L]``: causal depthwise
    convolution + SiLU, ``x_proj`` to (delta rank, B, C), ``delta_proj``, selective scan gated by ``z``, ``out_proj``.
    ``B`` / ``C`` given -> input-independent (``[batch, dstate, L]``)."""
    x, z = (t.transpose(1, 2) for t in xz.chunk(2, dim=1))                       # channel-last views [b, L, dim]
    x = causal_conv1d_silu(x.contiguous(), conv1d_weight, conv1d_bias)
    n, r = A.shape[-1], delta_proj_weight.shape[1]
    x_dbl = F.linear(x, x_proj_weight)
    delta = F.linear(x_dbl[..., :r], delta_proj_weight)
    Bc = x_dbl[..., r:r + n] + (0 if B_proj_bias is None else B_proj_bias.to(x_dbl.dtype)) if B is None else _bc_channel_last(B)
    Cc = x_dbl[..., -n:] + (0 if C_proj_bias is None else C_proj_bias.to(x_dbl.dtype)) if C is None else _bc_channel_last(C)
    y = _scan(x, delta.contiguous(), A, Bc.contiguous(), Cc.contiguous(), D, z.contiguous(), delta_bias, True)
    return F.linear(y, out_proj_weight, out_proj_bias)


def mamba_inner_fn(*args, **kwargs):
    return mamba_inner_ref(*args, _scan=_scan_cl, **kwargs)


class SelectiveScanFn:
    """The reference exposes ``autograd.Function`` classes; here differentiation goes through the operators, so ``apply``
    is the function."""
    apply = staticmethod(selective_scan_fn)


class MambaInnerFn:
    apply = staticmethod(mamba_inner_fn)
