"""Chunked state-space-duality scan and the fused Mamba-2 inner block with the reference's names and layouts
(zoology/mixers/mamba_ssm/ops/triton/ssd_combined.py:563-985): ``x [b, l, h, p]``, ``dt [b, l, h]``, ``A [h]``,
``B, C [b, l, g, n]``, ``D [h]`` or ``[h, p]``, ``z`` like ``x``. The scan itself is
:func:`ml_experiments_b200.ops.ssd_scan.ssd_chunk_scan` (tcgen05 kernel on CUDA, batched-GEMM formulation elsewhere)."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from ml_experiments_b200.ops.causal_conv import causal_conv1d_silu
from ....mamba2 import mamba_chunk_scan_combined
from .layernorm_gated import rmsnorm_fn


def mamba_chunk_scan(x, dt, A, B, C, chunk_size, D=None, z=None, dt_bias=None, dt_softplus=False):
    return mamba_chunk_scan_combined(x, dt, A, B, C, chunk_size, D=D, z=z, dt_bias=dt_bias, dt_softplus=dt_softplus)


def ssd_selective_scan(x, dt, A, B, C, D=None, z=None, dt_bias=None, dt_softplus=False, dt_limit=(0.0, float("inf"))):
    """Step-by-step oracle of the same recurrence (fp32): ``S <- exp(dt A) S + dt B x^T``, ``y = C S (+ D x) (* silu(z))``."""
    b, l, h, p = x.shape
    g, n = B.shape[2], B.shape[3]
    dtf = dt.float() + (0 if dt_bias is None else dt_bias.float())
    dtf = F.softplus(dtf) if dt_softplus else dtf
    if dt_limit != (0.0, float("inf")):
        dtf = dtf.clamp(*dt_limit)
    Bh, Ch = (t.float().repeat_interleave(h // g, dim=2) for t in (B, C))
    S = x.new_zeros(b, h, p, n, dtype=torch.float32)
    ys = []
    for t in range(l):
        S = torch.exp(dtf[:, t] * A.float())[..., None, None] * S + (dtf[:, t, :, None] * x[:, t].float())[..., None] * Bh[:, t, :, None, :]
        ys.append(torch.einsum("bhpn,bhn->bhp", S, Ch[:, t]))
    y = torch.stack(ys, 1)
    if D is not None:
        y = y + x.float() * (D.float().view(h, -1) if D.dim() > 0 else D.float())
    if z is not None:
        y = y * F.silu(z.float())
    return y.to(x.dtype)


def ssd_chunk_scan_combined_ref(x, dt, A, B, C, chunk_size, D=None, z=None, dt_bias=None, dt_softplus=False):
    """The chunked formulation in plain PyTorch on every device (the kernel's own oracle)."""
    from ml_experiments_b200.ops import ssd_scan as S

    b, l, h, p = x.shape
    dtf = dt.float() + (0 if dt_bias is None else dt_bias.float())
    dtf = F.softplus(dtf) if dt_softplus else dtf
    g = B.shape[2]
    Bh, Ch = (t if g in (1, h) else t.repeat_interleave(h // g, dim=2) for t in (B, C))
    y = S._ssd_chunk_scan_torch(x.float(), Bh.float(), Ch.float(), dtf * A.float(), dtf, chunk=min(chunk_size, 128))
    if D is not None:
        y = y + x.float() * (D.float().view(h, -1) if D.dim() > 0 else D.float())
    if z is not None:
        y = y * F.silu(z.float())
    return y.to(x.dtype)


def _split_block(zxbcdt, conv1d_weight, conv1d_bias, dt_bias, A, D, headdim, ngroups):
    nheads = D.shape[0]
    headdim = D.shape[1] if D.dim() == 2 else headdim
    if headdim is None:
        raise ValueError("headdim is needed when D has one entry per head")
    dim = nheads * headdim
    dstate = (zxbcdt.shape[-1] - 2 * dim - nheads) // ngroups // 2
    z, xBC, dt = torch.split(zxbcdt, [dim, dim + 2 * ngroups * dstate, nheads], dim=-1)
    w = conv1d_weight if conv1d_weight.dim() == 3 else conv1d_weight.unsqueeze(1)
    xBC = causal_conv1d_silu(xBC.contiguous(), w, conv1d_bias)
    x, B, C = torch.split(xBC, [dim, ngroups * dstate, ngroups * dstate], dim=-1)
    b, l = zxbcdt.shape[:2]
    return (z.reshape(b, l, nheads, headdim), x.reshape(b, l, nheads, headdim), B.reshape(b, l, ngroups, dstate),
            C.reshape(b, l, ngroups, dstate), dt)


def _finish(out, z, rmsnorm_weight, rmsnorm_eps, outproj_weight, outproj_bias, norm_before_gate):
    out = out.flatten(-2)
    if rmsnorm_weight is not None:
        out = rmsnorm_fn(out, rmsnorm_weight, None, z=z.flatten(-2), eps=rmsnorm_eps, norm_before_gate=norm_before_gate)
    return out if outproj_weight is None else F.linear(out, outproj_weight, outproj_bias)


def mamba_split_conv1d_scan_combined(zxbcdt, conv1d_weight, conv1d_bias, dt_bias, A, D, chunk_size, initial_states=None, seq_idx=None,
                                     dt_limit=(0.0, float("inf")), return_final_states=False, activation="silu", rmsnorm_weight=None,
                                     rmsnorm_eps=1e-6, outproj_weight=None, outproj_bias=None, headdim=None, ngroups=1, norm_before_gate=True):
    """The Mamba-2 inner block from the in-projection's output ``zxbcdt [b, l, 2 dim + 2 g n + h]``: split, causal
    depthwise convolution + SiLU on (x, B, C), chunked scan with softplus(dt + dt_bias), gate (inside the scan when
    there is no norm, inside the gated RMSNorm otherwise), output projection."""
    if seq_idx is not None:
        raise NotImplementedError("seq_idx (packed sequences) is not supported by this scan")
    if activation not in ("silu", "swish"):
        raise NotImplementedError("only the SiLU activation is fused with the convolution")
    z, x, B, C, dt = _split_block(zxbcdt, conv1d_weight, conv1d_bias, dt_bias, A, D, headdim, ngroups)
    res = mamba_chunk_scan_combined(x, dt, A, B, C, chunk_size, D=D, z=z if rmsnorm_weight is None else None, dt_bias=dt_bias, dt_softplus=True,
                                    dt_limit=dt_limit, return_final_states=return_final_states, initial_states=initial_states)
    y, state = res if return_final_states else (res, None)
    out = _finish(y, z, rmsnorm_weight, rmsnorm_eps, outproj_weight, outproj_bias, norm_before_gate)
    return (out, state) if return_final_states else out


def mamba_split_conv1d_scan_ref(zxbcdt, conv1d_weight, conv1d_bias, dt_bias, A, D, chunk_size, dt_limit=(0.0, float("inf")), activation="silu",
                                rmsnorm_weight=None, rmsnorm_eps=1e-6, outproj_weight=None, outproj_bias=None, headdim=None, ngroups=1,
                                norm_before_gate=True):
    z, x, B, C, dt = _split_block(zxbcdt, conv1d_weight, conv1d_bias, dt_bias, A, D, headdim, ngroups)
    y = ssd_selective_scan(x, dt.to(x.dtype), A, B, C, D=D.float(), z=z if rmsnorm_weight is None else None, dt_bias=dt_bias, dt_softplus=True,
                           dt_limit=dt_limit)
    return _finish(y, z, rmsnorm_weight, rmsnorm_eps, outproj_weight, outproj_bias, norm_before_gate)


__all__ = ["mamba_chunk_scan", "mamba_chunk_scan_combined", "mamba_split_conv1d_scan_combined", "mamba_split_conv1d_scan_ref",
           "ssd_chunk_scan_combined_ref", "ssd_selective_scan"]
