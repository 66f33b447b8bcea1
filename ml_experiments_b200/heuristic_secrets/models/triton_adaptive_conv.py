"""``heuristic_secrets.models.triton_adaptive_conv`` (reference: src/heuristic_secrets/models/triton_adaptive_conv.py).

The reference's Triton programs behind these names are CUDA kernels of this package; the functions keep the reference's
argument order and fall back to the PyTorch restatements off CUDA, so ``HAS_TRITON`` stays a statement about "is there
a fused kernel path", not about the Triton package.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from ...models.ripple_ops import AdaptiveLocalConv, SqueezeExcite1D
from ...ops.fused_taps import adaptive_local_gather
from ...ops.linear import linear
from ...ops.norm_act import rms_norm_act

HAS_TRITON = True


def triton_linear(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None = None) -> torch.Tensor:
    """``x [M, K] @ w [N, K].T (+ b)`` on the tcgen05 GEMM."""
    return linear(x, w, b)


def triton_rmsnorm(x: torch.Tensor, gamma: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return rms_norm_act(x, gamma, eps)


def triton_silu(x: torch.Tensor) -> torch.Tensor:
    return F.silu(x)


def triton_adaptive_conv(v, half_win, center_off, kernel, half_window_max):
    """``v [B, L, C]``; ``half_win, center_off [B, L, H]``; ``kernel [B, L, H, K]``: every position mixes the rows within its
    own window (centre offset, half width) with weights read from its kernel table. Whole sequence, one launch."""
    return adaptive_local_gather(v, half_win, center_off, kernel, half_win.shape[-1], int(half_window_max))


class TritonAdaptiveLocalConv(AdaptiveLocalConv):
    """:class:`AdaptiveLocalConv` under the reference's fused-variant name and argument order."""

    def __init__(self, channels: int, num_heads: int = 8, max_kernel_size: int = 64, min_window: float = 1.0, chunk_size: int = 1024,
                 scale_power: float = 0.421875):
        super().__init__(channels, num_heads, max_kernel_size, min_window, scale_power, chunk_size)


__all__ = ["HAS_TRITON", "SqueezeExcite1D", "TritonAdaptiveLocalConv", "triton_adaptive_conv", "triton_linear", "triton_rmsnorm", "triton_silu"]
