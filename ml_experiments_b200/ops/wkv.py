"""RWKV time-mixing operators with autograd: WKV-4 (per-channel exponential moving softmax) and WKV-5 (linear attention
with a per-key-channel decay and a bonus for the current token).

CUDA kernels on a GPU (``csrc/wkv/wkv.cu``); the differentiable sequential restatements below are the CPU path and the
test oracle. Parameterisation follows the reference wrappers (zoology/mixers/rwkv.py:47-100, rwkv5.py:53-101):
``wkv4`` takes the raw ``time_decay`` (the decay is ``-exp(time_decay)``), ``wkv5`` takes the raw ``time_decay`` of
shape ``[H, N]`` (the decay factor is ``exp(-exp(time_decay))``) -- the chain rule through those maps is applied here.
"""
from __future__ import annotations

import torch

from .runtime import ops


def wkv4_ref(time_decay, u, k, v):
    """``k, v [B, T, C]``; sequential, numerically stabilised by the running maximum exponent."""
    w = -torch.exp(time_decay.float())
    u, k, v = u.float(), k.float(), v.float()
    B, T, C = k.shape
    p = k.new_zeros(B, C)
    q = k.new_zeros(B, C)
    o = k.new_full((B, C), -1e38)
    ys = []
    for t in range(T):
        kt, vt = k[:, t], v[:, t]
        no = torch.maximum(o, u + kt)
        a, e = torch.exp(o - no), torch.exp(u + kt - no)
        ys.append((a * p + e * vt) / (a * q + e))
        no = torch.maximum(w + o, kt)
        a, e = torch.exp(w + o - no), torch.exp(kt - no)
        p, q, o = a * p + e * vt, a * q + e, no
    return torch.stack(ys, 1)


def wkv5_ref(r, k, v, time_decay, u):
    """``r, k, v [B, T, H*N]``, ``time_decay, u [H, N]``."""
    H, N = time_decay.shape
    B, T, C = r.shape
    w = torch.exp(-torch.exp(time_decay.float())).view(1, H, N, 1)
    uu = u.float().view(1, H, N, 1)
    rf, kf, vf = (t.float().view(B, T, H, N) for t in (r, k, v))
    S = rf.new_zeros(B, H, N, N)
    ys = []
    for t in range(T):
        kv = kf[:, t].unsqueeze(-1) * vf[:, t].unsqueeze(-2)  # [B, H, Nk, Nv]
        ys.append(torch.einsum("bhj,bhji->bhi", rf[:, t], uu * kv + S))
        S = w * S + kv
    return torch.stack(ys, 1).reshape(B, T, C)


class _WKV4(torch.autograd.Function):
    @staticmethod
    def forward(ctx, time_decay, u, k, v):
        io = torch.bfloat16 if k.dtype == torch.bfloat16 else torch.float32
        w = (-torch.exp(time_decay.float())).contiguous()
        uf, kc, vc = u.float().contiguous(), k.to(io).contiguous(), v.to(io).contiguous()
        y = torch.empty_like(kc)
        ops().wkv4_fwd(kc, vc, w, uf, y)
        ctx.save_for_backward(w, uf, kc, vc)
        ctx.dtypes = (time_decay.dtype, u.dtype, k.dtype, v.dtype)
        return y.to(k.dtype)

    @staticmethod
    def backward(ctx, gy):
        w, uf, kc, vc = ctx.saved_tensors
        B, T, C = kc.shape
        gk, gv = torch.empty_like(kc), torch.empty_like(vc)
        gw = torch.empty(B, C, dtype=torch.float32, device=kc.device)
        gu = torch.empty_like(gw)
        scratch = torch.empty(3, B, T, C, dtype=torch.float32, device=kc.device)
        ops().wkv4_bwd(kc, vc, w, uf, gy.to(kc.dtype).contiguous(), gk, gv, gw, gu, scratch)
        t = ctx.dtypes
        # w = -exp(time_decay): d w / d time_decay = w
        return (gw.sum(0) * w).to(t[0]), gu.sum(0).to(t[1]), gk.to(t[2]), gv.to(t[3])


class _WKV5(torch.autograd.Function):
    @staticmethod
    def forward(ctx, r, k, v, time_decay, u):
        io = torch.bfloat16 if r.dtype == torch.bfloat16 else torch.float32
        ew = -torch.exp(time_decay.float())
        w = torch.exp(ew).contiguous()
        uf = u.float().contiguous()
        rc, kc, vc = (t.to(io).contiguous() for t in (r, k, v))
        y = torch.empty_like(rc)
        ops().wkv5_fwd(rc, kc, vc, w, uf, y)
        ctx.save_for_backward(rc, kc, vc, w, ew, uf)
        ctx.dtypes = (r.dtype, k.dtype, v.dtype, time_decay.dtype, u.dtype)
        return y.to(r.dtype)

    @staticmethod
    def backward(ctx, gy):
        rc, kc, vc, w, ew, uf = ctx.saved_tensors
        B, T, C = rc.shape
        gr, gk, gv = torch.empty_like(rc), torch.empty_like(kc), torch.empty_like(vc)
        gw = torch.empty(B, C, dtype=torch.float32, device=rc.device)
        gu = torch.empty_like(gw)
        ops().wkv5_bwd(rc, kc, vc, w, uf, gy.to(rc.dtype).contiguous(), gr, gk, gv, gw, gu)
        t = ctx.dtypes
        # w = exp(-exp(time_decay)): d w / d time_decay = w * (-exp(time_decay))
        g_decay = gw.sum(0).view_as(w) * w * ew
        return gr.to(t[0]), gk.to(t[1]), gv.to(t[2]), g_decay.to(t[3]), gu.sum(0).view_as(uf).to(t[4])


def wkv4(time_decay, u, k, v):
    if not k.is_cuda:
        return wkv4_ref(time_decay, u, k, v).to(k.dtype)
    return _WKV4.apply(time_decay, u, k, v)


def wkv5(r, k, v, time_decay, u):
    if not r.is_cuda or time_decay.shape[1] not in (32, 64, 128):
        return wkv5_ref(r, k, v, time_decay, u).to(r.dtype)
    return _WKV5.apply(r, k, v, time_decay, u)
