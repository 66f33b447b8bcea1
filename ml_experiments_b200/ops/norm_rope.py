"""RMS norm over the head dimension fused with the rotary map of the current speedrun GPT (one kernel forward, one
backward): ``y = f1 * n + f2 * flip_pairs(n)`` with ``n = rms_norm(x)``; see ``csrc/fused/norm_rope.cu``. The eager
form is ``F.rms_norm`` + ``Yarn.rotary`` (modded-nanogpt/train_gpt.py: ``norm``, ``Yarn.rotary``)."""
from __future__ import annotations

import torch
import torch.nn.functional as F


def norm_rotary_ref(x, f1, f2, eps=None):
    """``x [B, T, H, D]``; tables ``[>= T, D]`` or, for the paired-head layout, ``[>= T, 2 D]`` (head ``h`` reads columns
    ``(h % 2) * D`` onwards, which is what rotating the ``[B, T, H/2, 2 D]`` view does)."""
    B, T, H, D = x.shape
    n = F.rms_norm(x, (D,), eps=eps)
    W = f1.shape[1]
    if W == 2 * D:
        n = n.reshape(B, T, H // 2, 2 * D)
    a, b = f1[None, :T, None, :].to(x.dtype), f2[None, :T, None, :].to(x.dtype)
    flip = n.reshape(*n.shape[:-1], n.shape[-1] // 2, 2).flip(-1).reshape(n.shape)
    return (a * n + b * flip).reshape(B, T, H, D)


class _NormRotary(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, f1, f2, eps):
        from .runtime import add_launches, ops

        B, T, H, D = x.shape
        y = torch.empty(B, T, H, D, dtype=torch.bfloat16, device=x.device)
        rstd = torch.empty(B * T * H, dtype=torch.float32, device=x.device)
        ops().norm_rope_fwd(x, f1, f2, y, rstd, eps)
        add_launches(1)
        ctx.save_for_backward(x, f1, f2, rstd)
        return y

    @staticmethod
    def backward(ctx, dy):
        from .runtime import add_launches, ops

        x, f1, f2, rstd = ctx.saved_tensors
        dx = torch.empty(x.shape, dtype=torch.bfloat16, device=x.device)
        ops().norm_rope_bwd(x, f1, f2, rstd, dy.contiguous(), dx)
        add_launches(1)
        return dx, None, None, None


def norm_rotary(x: torch.Tensor, f1: torch.Tensor, f2: torch.Tensor, eps: float | None = None) -> torch.Tensor:
    """Kernel path for bf16 CUDA inputs with ``D`` in {64, 128} whose last dim is dense (``x`` may be the q or k slice
    of a fused projection); the eager composition otherwise."""
    ok = (x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 4 and x.shape[-1] in (64, 128) and x.stride(-1) == 1
          and (x.shape[0] == 1 or x.stride(0) == x.shape[1] * x.stride(1))
          and f1.dtype == torch.bfloat16 and f1.is_contiguous() and f2.is_contiguous())
    if not ok:
        return norm_rotary_ref(x, f1, f2, eps)
    return _NormRotary.apply(x, f1, f2, float(torch.finfo(x.dtype).eps if eps is None else eps))
