"""Document-masked causal flash attention with a block sliding window (tcgen05 kernels + torch oracle).

Replaces the FlexAttention / FlashAttention-3 call sites of the reference trainers
(modded-nanogpt/train_gpt.py:926,963-965; records/track_1_short/2025-01-26_BatchSize: ``flex_attention`` with a
document-causal ``BlockMask`` of 128-token blocks). Mask semantics: query ``i`` attends key ``j`` iff ``j <= i``, both
tokens belong to the same document, and ``block(j) > block(i) - window_blocks`` with 128-token blocks.
"""
from __future__ import annotations

import torch

from .runtime import ops, status


def doc_bounds_from_starts(is_start: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Per-token ``(doc_start, doc_end)`` (int32) from a boolean "this token begins a document" vector.

    Token 0 always begins a document.
    """
    t = is_start.numel()
    pos = torch.arange(t, device=is_start.device, dtype=torch.int64)
    starts = is_start.clone().bool()
    starts[0] = True
    start_pos = torch.where(starts, pos, torch.zeros_like(pos))
    doc_start = torch.cummax(start_pos, 0).values
    # end = next start strictly after the token (or T)
    nxt = torch.where(starts, pos, torch.full_like(pos, t))
    rev = torch.flip(torch.cummin(torch.flip(nxt, [0]), 0).values, [0])  # next start at or after i
    doc_end = torch.cat([rev[1:], rev.new_full((1,), t)])
    return doc_start.to(torch.int32), doc_end.to(torch.int32)


def doc_bounds_from_tokens(tokens: torch.Tensor, bos: int) -> tuple[torch.Tensor, torch.Tensor]:
    """``doc_bounds_from_starts(tokens == bos)``; one kernel on a GPU instead of two scans and a dozen elementwise ops."""
    if not tokens.is_cuda:
        return doc_bounds_from_starts(tokens == bos)
    t = tokens.numel()
    doc_start = torch.empty(t, dtype=torch.int32, device=tokens.device)
    doc_end = torch.empty(t, dtype=torch.int32, device=tokens.device)
    ops().doc_bounds(tokens.to(torch.int64).contiguous(), int(bos), doc_start, doc_end)
    return doc_start, doc_end


def attention_mask(doc_start: torch.Tensor, window_blocks: int) -> torch.Tensor:
    """Dense boolean [T, T] mask with the kernel's semantics (for oracles and small tests)."""
    t = doc_start.numel()
    i = torch.arange(t, device=doc_start.device)
    causal = i[:, None] >= i[None, :]
    same_doc = i[None, :] >= doc_start.to(torch.int64)[:, None]
    m = causal & same_doc
    if window_blocks > 0:
        m &= (i[None, :] // 128) > (i[:, None] // 128 - window_blocks)
    return m


def attention_reference(q, k, v, doc_start, scale: float, window_blocks: int = 0) -> torch.Tensor:
    """fp32 dense oracle: q, k, v are [T, H, D]."""
    m = attention_mask(doc_start, window_blocks)
    qf, kf, vf = (x.float().transpose(0, 1) for x in (q, k, v))  # [H, T, D]
    s = (qf @ kf.transpose(1, 2)) * scale
    s = s.masked_fill(~m[None], float("-inf"))
    p = torch.softmax(s, dim=-1)
    return (p @ vf).transpose(0, 1)


class _FlashAttn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, doc_start, doc_end, scale, window_blocks):
        t, h, d = q.shape
        o = torch.empty(t, h, d, dtype=torch.bfloat16, device=q.device)
        lse = torch.empty(h, t, dtype=torch.float32, device=q.device)
        ops().attn_fwd(q, k, v, o, lse, doc_start, doc_end, scale, window_blocks, status(q.device))
        ctx.save_for_backward(q, k, v, o, lse, doc_start, doc_end)
        ctx.scale, ctx.window_blocks = scale, window_blocks
        return o

    @staticmethod
    def backward(ctx, d_o):
        q, k, v, o, lse, doc_start, doc_end = ctx.saved_tensors
        dq, dk, dv = flash_attention_backward(q, k, v, o, d_o, lse, doc_start, doc_end, ctx.scale, ctx.window_blocks)
        return dq.to(torch.bfloat16), dk, dv, None, None, None, None


def flash_attention_forward(q, k, v, doc_start, doc_end, scale: float, window_blocks: int = 0):
    """Returns ``(o, lse)``; ``q, k, v`` are bf16 [T, H, D] views whose heads are contiguous."""
    t, h, d = q.shape
    o = torch.empty(t, h, d, dtype=torch.bfloat16, device=q.device)
    lse = torch.empty(h, t, dtype=torch.float32, device=q.device)
    ops().attn_fwd(q, k, v, o, lse, doc_start, doc_end, scale, window_blocks, status(q.device))
    return o, lse


def flash_attention_backward(q, k, v, o, d_o, lse, doc_start, doc_end, scale: float, window_blocks: int = 0,
                             dq_acc: torch.Tensor | None = None):
    """Returns ``(dq fp32, dk bf16, dv bf16)``. ``dq_acc`` (fp32, zeroed) may be supplied to reuse a buffer."""
    t, h, d = q.shape
    if dq_acc is None:
        dq_acc = torch.zeros(t, h, d, dtype=torch.float32, device=q.device)
    dk = torch.empty(t, h, d, dtype=torch.bfloat16, device=q.device)   # every row is written by its key tile's CTA
    dv = torch.empty(t, h, d, dtype=torch.bfloat16, device=q.device)
    delta = torch.empty(h, t, dtype=torch.float32, device=q.device)
    if d_o.stride(2) != 1 or d_o.stride(1) != d:
        d_o = d_o.contiguous()
    ops().attn_bwd(q, k, v, o, d_o, lse, delta, dq_acc, dk, dv, doc_start, doc_end, scale, window_blocks,
                   status(q.device))
    return dq_acc, dk, dv


def flash_attention(q, k, v, doc_start, doc_end, scale: float, window_blocks: int = 0) -> torch.Tensor:
    """Differentiable attention on [T, H, D] bf16 tensors (CUDA); falls back to the dense oracle on CPU."""
    if not q.is_cuda:
        return attention_reference(q, k, v, doc_start, scale, window_blocks).to(q.dtype)
    return _FlashAttn.apply(q, k, v, doc_start, doc_end, float(scale), int(window_blocks))


def differential_flash_attention(q1, k1, q2, k2, v, scale: float | None = None):
    """Both score streams of causal differential attention in ONE launch of the flash kernel.

    ``q1, k1, q2, k2 [B, L, H, d]`` and the shared values ``v [B, L, H, dv]`` -> ``(o1, o2)``, each ``[B, L, H, dv]``
    with ``o_i = softmax(q_i k_i^T * scale, causal) v``. The two streams become ``2 H`` heads of one call: the narrower
    q / k head dimension is zero-padded to the kernel's head size (zeros do not change a dot product), every batch
    element is one document of the packed token stream, and the values are laid out once per stream. Gradients flow
    through the kernel's backward; the padding and the stacking are plain autograd ops.
    """
    B, L, H, d = q1.shape
    dv = v.shape[-1]
    scale = float(scale) if scale is not None else d ** -0.5
    D = 64 if max(d, dv) <= 64 else 128
    if max(d, dv) > 128:
        raise ValueError("differential_flash_attention: head dimensions up to 128")
    T = B * L
    bf = torch.bfloat16

    def pad(t, w):
        t = t.reshape(T, H, w).to(bf)
        return t if w == D else torch.nn.functional.pad(t, (0, D - w))

    q = torch.cat([pad(q1, d), pad(q2, d)], 1).contiguous()          # [T, 2H, D]
    k = torch.cat([pad(k1, d), pad(k2, d)], 1).contiguous()
    vv = pad(v, dv)
    vv = torch.cat([vv, vv], 1).contiguous()
    pos = torch.arange(T, device=q.device, dtype=torch.int32)
    start = pos // L * L
    o = flash_attention(q, k, vv, start, start + L, scale)            # [T, 2H, D]
    o = o[..., :dv].reshape(B, L, 2, H, dv)
    return o[:, :, 0], o[:, :, 1]
