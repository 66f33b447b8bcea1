"""Block-sparse primitives of multi-resolution attention (MRA-2) with autograd, and the attention built from them.

The attention scores are computed exactly on a selected list of 32 x 32 blocks (the ``num_blocks`` highest scoring blocks
of a block-averaged "low resolution" score map, plus optional diagonal / first-rows priors) and, in ``"full"`` mode,
approximated by the low-resolution scores everywhere else. Follows zoology/mixers/mra/attention.py:17-146 and
autograd_function.py:13-61 of the reference; the CUDA kernels are ``csrc/mra/mra.cu``, the index arithmetic is shared
with the PyTorch restatements used on the CPU and as oracle. Block tensors are ``[B, n, 32(query), 32(key)]``.
"""
from __future__ import annotations

import math

import torch

from .runtime import ops

BS = 32


def _split(indices, kbn):
    return torch.div(indices, kbn, rounding_mode="floor").long(), (indices % kbn).long()


def sddmm_ref(Q, K, indices):
    B, Lk = K.shape[0], K.shape[1]
    qb, kb = _split(indices, Lk // BS)
    bi = torch.arange(B, device=Q.device)[:, None]
    Qb = Q.view(B, -1, BS, Q.shape[-1])[bi, qb]
    Kb = K.view(B, -1, BS, K.shape[-1])[bi, kb]
    return Qb @ Kb.transpose(-1, -2)


def spmm_ref(P, indices, V, Lq, Lk, transposed=False):
    B, D = V.shape[0], V.shape[-1]
    qb, kb = _split(indices, Lk // BS)
    bi = torch.arange(B, device=V.device)[:, None]
    if transposed:
        src, dst, Ldst, Pm = qb, kb, Lk, P.transpose(-1, -2)
    else:
        src, dst, Ldst, Pm = kb, qb, Lq, P
    contrib = Pm @ V.view(B, -1, BS, D)[bi, src]                       # [B, n, 32, D]
    out = V.new_zeros(B * (Ldst // BS), BS * D)
    out.index_add_(0, (dst + bi * (Ldst // BS)).reshape(-1), contrib.reshape(-1, BS * D))
    return out.view(B, Ldst, D)


def rowmax_ref(S, indices, Lq, Lk):
    B = S.shape[0]
    qb, _ = _split(indices, Lk // BS)
    bi = torch.arange(B, device=S.device)[:, None]
    m = S.new_full((B * (Lq // BS), BS), float("-inf"))
    m.index_reduce_(0, (qb + bi * (Lq // BS)).reshape(-1), S.amax(dim=-1).reshape(-1, BS), "amax")
    return m.view(B, Lq)


def _cuda_ok(*ts):
    return all(t.is_cuda and t.dtype == torch.float32 for t in ts) and ts[0].shape[-1] % 4 == 0 and ts[0].shape[-1] <= 256


def _sddmm(Q, K, indices):
    if _cuda_ok(Q, K):
        S = torch.empty(Q.shape[0], indices.shape[1], BS, BS, device=Q.device, dtype=torch.float32)
        ops().mra_sddmm(Q.contiguous(), K.contiguous(), indices.int().contiguous(), S)
        return S
    return sddmm_ref(Q, K, indices)


def _spmm(P, indices, V, Lq, Lk, transposed=False):
    if _cuda_ok(V) and P.is_cuda:
        out = torch.zeros(V.shape[0], Lk if transposed else Lq, V.shape[-1], device=V.device, dtype=torch.float32)
        ops().mra_spmm(P.contiguous(), indices.int().contiguous(), V.contiguous(), out, Lq, Lk, transposed)
        return out
    return spmm_ref(P, indices, V, Lq, Lk, transposed)


class SampledDenseMM(torch.autograd.Function):
    """``S[b, n] = Q_block(qb) @ K_block(kb)^T`` on the listed blocks."""

    @staticmethod
    def forward(ctx, Q, K, indices):
        ctx.save_for_backward(Q, K, indices)
        return _sddmm(Q, K, indices)

    @staticmethod
    def backward(ctx, g):
        Q, K, indices = ctx.saved_tensors
        Lq, Lk = Q.shape[1], K.shape[1]
        g = g.contiguous()
        return _spmm(g, indices, K, Lq, Lk), _spmm(g, indices, Q, Lq, Lk, transposed=True), None


class SparseDenseMM(torch.autograd.Function):
    """``out[q rows] += P[b, n] @ V_block(kb)``."""

    @staticmethod
    def forward(ctx, P, indices, V, Lq):
        ctx.save_for_backward(P, indices, V)
        ctx.Lq = Lq
        return _spmm(P, indices, V, Lq, V.shape[1])

    @staticmethod
    def backward(ctx, g):
        P, indices, V = ctx.saved_tensors
        g = g.contiguous()
        return _sddmm(g, V, indices), None, _spmm(P, indices, g, ctx.Lq, V.shape[1], transposed=True), None


def sparse_row_max(S, indices, Lq, Lk):
    """Per query row, the maximum over its listed blocks (``-inf`` for rows with none); no gradient (it only shifts)."""
    S = S.detach()
    if S.is_cuda and S.dtype == torch.float32:
        m = torch.full((S.shape[0], Lq), float("-inf"), device=S.device, dtype=torch.float32)
        ops().mra_rowmax(S.contiguous(), indices.int().contiguous(), m, Lk)
        return m
    return rowmax_ref(S, indices, Lq, Lk)


def sparse_row_sum(P, indices, Lq, Lk):
    B = P.shape[0]
    qb, _ = _split(indices, Lk // BS)
    bi = torch.arange(B, device=P.device)[:, None]
    out = P.new_zeros(B * (Lq // BS), BS)
    return out.index_add(0, (qb + bi * (Lq // BS)).reshape(-1), P.sum(dim=-1).reshape(-1, BS)).view(B, Lq)


def low_resolution_logit(Q, K, V=None):
    B, L, D = Q.shape
    pool = lambda t: t.view(B, L // BS, BS, D).mean(dim=-2)
    logit = pool(Q) @ pool(K).transpose(-1, -2) / math.sqrt(D)
    return logit, logit.amax(dim=-1, keepdim=True), (pool(V) if V is not None else None)


def select_blocks(logit, num_blocks, approx_mode, first_n_blocks=0, diagonal_n_blocks=0, causal=False):
    """Top-``num_blocks`` entries of the (prior-boosted) block score map -> flat indices and, in full mode, their mask."""
    B, nb, _ = logit.shape
    logit = logit.clone()
    if diagonal_n_blocks > 0:
        off = diagonal_n_blocks // 2
        ones = torch.ones(nb, nb, device=logit.device)
        logit += torch.tril(torch.triu(ones, diagonal=-off), diagonal=off)[None] * 5e3
    if first_n_blocks > 0:
        logit[:, :first_n_blocks, :] += 5e3
        logit[:, :, :first_n_blocks] += 5e3
    if causal:  # blocks strictly above the diagonal can never be visible
        logit = logit.masked_fill(torch.ones(nb, nb, device=logit.device, dtype=torch.bool).triu(1)[None], float("-inf"))
    top = torch.topk(logit.reshape(B, -1), num_blocks, dim=-1, largest=True, sorted=False)
    mask = (logit >= top.values.min(dim=-1).values[:, None, None]).float() if approx_mode == "full" else None
    return top.indices, mask


def mra2_attention(Q, K, V, num_blocks, approx_mode="full", initial_prior_first_n_blocks=0, initial_prior_diagonal_n_blocks=0,
                   causal=False):
    """``Q, K, V [B, H, L, D]`` (``L`` a multiple of 32) -> ``[B, H, L, D]``. ``causal`` adds the token-level causal mask
    inside the listed blocks and restricts the low-resolution part to strictly earlier blocks (an extension: the
    reference attends in both directions)."""
    Bh, H, L, D = Q.shape
    mb, nb = Bh * H, L // BS
    Q, K, V = (t.reshape(mb, L, D).float() for t in (Q, K, V))
    if approx_mode == "full":
        low, low_max, V_hat = low_resolution_logit(Q, K, V)
    elif approx_mode == "sparse":
        with torch.no_grad():
            low, low_max, V_hat = low_resolution_logit(Q, K)
    else:
        raise ValueError(approx_mode)
    with torch.no_grad():
        indices, hi_mask = select_blocks(low - low_max, min(num_blocks, nb * nb), approx_mode, initial_prior_first_n_blocks,
                                         initial_prior_diagonal_n_blocks, causal)
    S = SampledDenseMM.apply(Q, K, indices) / math.sqrt(D)
    if causal:
        qb, kb = _split(indices, nb)
        i = torch.arange(BS, device=Q.device)
        visible = (qb[..., None, None] * BS + i[:, None]) >= (kb[..., None, None] * BS + i[None, :])
        S = S.masked_fill(~visible, -1e4)
    row_max = sparse_row_max(S, indices, L, L)
    row_max = torch.where(torch.isfinite(row_max), row_max, torch.zeros_like(row_max))
    qb, _ = _split(indices, nb)
    S = S - row_max.view(mb, nb, BS)[torch.arange(mb, device=Q.device)[:, None], qb].unsqueeze(-1)
    P = torch.exp(S)
    hi_out = SparseDenseMM.apply(P, indices, V, L)
    hi_norm = sparse_row_sum(P, indices, L, L)
    if approx_mode == "sparse":
        out = hi_out / (hi_norm[:, :, None] + 1e-6)
    else:
        penal = 1e4 * hi_mask
        if causal:
            penal = penal + 1e4 * torch.ones(nb, nb, device=Q.device).triu(0)[None]  # only strictly earlier blocks
        low_attn = torch.exp(low - low_max - penal) * BS
        low_out = (low_attn @ V_hat).repeat_interleave(BS, dim=1)
        low_norm = low_attn.sum(dim=-1).repeat_interleave(BS, dim=1)
        corr = low_max.repeat_interleave(BS, dim=1).squeeze(-1) - row_max
        low_c, hi_c = torch.exp(corr * (corr <= 0).float()), torch.exp(-corr * (corr > 0).float())
        out = (hi_out * hi_c[:, :, None] + low_out * low_c[:, :, None]) / (hi_norm[:, :, None] * hi_c[:, :, None] + low_norm[:, :, None] * low_c[:, :, None] + 1e-6)
    return out.view(Bh, H, L, D)
