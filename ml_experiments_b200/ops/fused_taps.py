"""Telephone attention and adaptive local convolution with the tap formulas evaluated inside the gather kernels
(``csrc/gather/fused_taps.cu``): the ``[B, L, H, S]`` position / weight tensors of the unfused composition never exist,
so the whole sequence is processed in one launch, without chunking or recomputation. The PyTorch restatements below
build those tensors and call :func:`~ml_experiments_b200.ops.gather_conv.gather_conv_ref`; they are the CPU path and the
oracle of the kernels. Tap formulas: src/heuristic_secrets/models/telephone_attention.py:124-180 and
adaptive_local_conv.py:75-169 of the reference.
"""
from __future__ import annotations

import torch

from .gather_conv import gather_conv_ref
from .runtime import ops


def _lerp_table(table, norm_pos):
    K = table.shape[-1]
    idx = norm_pos.clamp(0, 1) * (K - 1)
    lo = idx.detach().long().clamp(0, K - 2)
    w_hi = idx - lo.to(idx.dtype)
    return table.gather(-1, lo) * (1 - w_hi) + table.gather(-1, lo + 1) * w_hi


def telephone_taps(freq, phase, kern, expo, half: int, max_rec: float, L: int, start: int = 0):
    """Positions and weights ``[B, n, H, 2*half+1]`` for query rows ``start .. start+n``."""
    n = freq.shape[1]
    s_off = torch.arange(-half, half + 1, device=freq.device, dtype=torch.float32)
    rel = s_off.view(1, 1, 1, -1) * freq.unsqueeze(-1)
    centers = torch.arange(start, start + n, device=freq.device, dtype=torch.float32).view(1, n, 1, 1)
    pos = centers + rel + phase.unsqueeze(-1)
    valid = ((pos >= 0) & (pos < L)).float()
    power = (1.0 + rel.abs() / L).pow(-expo.view(expo.shape[0], n, 1, 1))
    return pos, _lerp_table(kern, rel.abs() / max_rec) * power * valid


def telephone_gather_ref(x, freq, phase, kern, expo, num_heads: int, half: int, max_rec: float):
    pos, wgt = telephone_taps(freq.float(), phase.float(), kern.float(), expo.float(), half, max_rec, x.shape[1])
    return gather_conv_ref(x, pos, wgt, num_heads)


def alc_taps(half_w, center, kern, half: int, L: int):
    s_off = torch.arange(-half, half + 1, device=half_w.device, dtype=torch.float32)
    rel = s_off.abs().view(1, 1, 1, -1) / half_w.unsqueeze(-1)
    pos = torch.arange(L, device=half_w.device, dtype=torch.float32).view(1, L, 1, 1) + center.unsqueeze(-1) + s_off.view(1, 1, 1, -1)
    valid = ((pos >= 0) & (pos < L)).float()
    wgt = (_lerp_table(kern, rel).clamp(min=0) + 1.0) * torch.exp(-rel * rel) * valid
    return pos, wgt / wgt.sum(-1, keepdim=True).clamp(min=1.0)


def alc_gather_ref(x, half_w, center, kern, num_heads: int, half: int):
    pos, wgt = alc_taps(half_w.float(), center.float(), kern.float(), half, x.shape[1])
    return gather_conv_ref(x, pos, wgt, num_heads)


class _Telephone(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, freq, phase, kern, expo, H, half, max_rec):
        x16 = x.to(torch.bfloat16).contiguous()
        f, p, k, e = (t.float().contiguous() for t in (freq, phase, kern, expo))
        out = torch.empty_like(x16)
        ops().tele_fused_fwd(x16, f, p, k, e, out, H, half, max_rec)
        ctx.save_for_backward(x16, f, p, k, e)
        ctx.cfg, ctx.dt = (H, half, max_rec), (x.dtype, freq.dtype, phase.dtype, kern.dtype, expo.dtype)
        return out.to(x.dtype)

    @staticmethod
    def backward(ctx, dout):
        x16, f, p, k, e = ctx.saved_tensors
        H, half, max_rec = ctx.cfg
        dx = torch.zeros(x16.shape, dtype=torch.float32, device=x16.device)
        df, dp, de_h = torch.empty_like(f), torch.empty_like(p), torch.empty_like(f)
        dk = torch.empty_like(k)
        ops().tele_fused_bwd(x16, f, p, k, e, dout.to(torch.bfloat16).contiguous(), dx, df, dp, dk, de_h, H, half, max_rec)
        de = de_h.view(*f.shape[:2], -1).sum(-1).view(e.shape)
        d = ctx.dt
        return dx.to(d[0]), df.to(d[1]), dp.to(d[2]), dk.to(d[3]), de.to(d[4]), None, None, None


class _AdaptiveLocal(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, half_w, center, kern, H, half):
        x16 = x.to(torch.bfloat16).contiguous()
        w, c, k = (t.float().contiguous() for t in (half_w, center, kern))
        out = torch.empty_like(x16)
        ops().alc_fused_fwd(x16, w, c, k, out, H, half)
        ctx.save_for_backward(x16, w, c, k)
        ctx.cfg, ctx.dt = (H, half), (x.dtype, half_w.dtype, center.dtype, kern.dtype)
        return out.to(x.dtype)

    @staticmethod
    def backward(ctx, dout):
        x16, w, c, k = ctx.saved_tensors
        H, half = ctx.cfg
        dx = torch.zeros(x16.shape, dtype=torch.float32, device=x16.device)
        dw, dc, dk = torch.empty_like(w), torch.empty_like(c), torch.empty_like(k)
        ops().alc_fused_bwd(x16, w, c, k, dout.to(torch.bfloat16).contiguous(), dx, dw, dc, dk, H, half)
        d = ctx.dt
        return dx.to(d[0]), dw.to(d[1]), dc.to(d[2]), dk.to(d[3]), None, None


def _fusable(x, kern, num_heads):
    return x.is_cuda and x.shape[-1] // num_heads in (8, 16, 32, 64, 128) and 2 <= kern.shape[-1] <= 64


def telephone_gather(x, freq, phase, kern, expo, num_heads: int, half: int, max_rec: float):
    """``x [B, L, C]``; ``freq, phase [B, L, H]``; ``kern [B, L, H, K]``; ``expo [B, L, 1]`` -> ``[B, L, C]``."""
    if _fusable(x, kern, num_heads):
        return _Telephone.apply(x, freq, phase, kern, expo, num_heads, int(half), float(max_rec))
    return telephone_gather_ref(x, freq, phase, kern, expo, num_heads, half, max_rec)


def adaptive_local_gather(x, half_w, center, kern, num_heads: int, half: int):
    """``x [B, L, C]``; ``half_w, center [B, L, H]``; ``kern [B, L, H, K]`` -> ``[B, L, C]``."""
    if _fusable(x, kern, num_heads) and half <= 64:
        return _AdaptiveLocal.apply(x, half_w, center, kern, num_heads, int(half))
    return alc_gather_ref(x, half_w, center, kern, num_heads, half)
