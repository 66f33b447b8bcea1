"""``heuristic_secrets.models.triton_telephone`` (reference: src/heuristic_secrets/models/triton_telephone.py): the
telephone operator's fused entry points on this package's CUDA kernels, with the reference's names and argument order."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from ...models.ripple_ops import TelephoneAttentionND
from ...ops.fused_taps import telephone_gather
from ...ops.linear import linear
from ...ops.norm_act import rms_norm_act

HAS_TRITON = True


def triton_linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    return linear(x, w)


def triton_linear_silu(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return F.silu(linear(x, w, b))


def triton_silu(x: torch.Tensor) -> torch.Tensor:
    return F.silu(x)


def triton_rmsnorm_silu(x: torch.Tensor, gamma: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """Weighted RMSNorm and SiLU in one kernel."""
    return rms_norm_act(x, gamma, eps, "silu")


def triton_linear_rmsnorm_silu(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, gamma: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return rms_norm_act(linear(x, w, b), gamma, eps, "silu")


def triton_telephone_attn(x, freq, phase, kernel, exponent, half_s, max_receptive, chunk_start: int = 0, seq_len: int | None = None):
    """``x [B, L, C]`` (the whole sequence); ``freq, phase [B, Lc, H]``, ``kernel [B, Lc, H, K]``, ``exponent [B, Lc, 1]`` for
    the ``Lc`` query positions starting at ``chunk_start``. Returns ``[B, Lc, C]``. The kernel of this package takes the
    whole sequence in one launch; a proper chunk is embedded into full-length parameter tensors and cut out again."""
    B, L, _ = x.shape
    Lc = freq.shape[1]
    H = freq.shape[-1]
    if chunk_start == 0 and Lc == L:
        return telephone_gather(x, freq, phase, kernel, exponent, H, int(half_s), float(max_receptive))

    def full(t, fill=0.0):
        out = t.new_full((B, L) + tuple(t.shape[2:]), fill)
        out[:, chunk_start:chunk_start + Lc] = t
        return out

    y = telephone_gather(x, full(freq, 1.0), full(phase), full(kernel), full(exponent, 1.0), H, int(half_s), float(max_receptive))
    return y[:, chunk_start:chunk_start + Lc]


def triton_telephone_attn_with_decay(x, freq, phase, kernel, exponent, half_s, max_receptive, chunk_start: int = 0, seq_len: int | None = None):
    return triton_telephone_attn(x, freq, phase, kernel, exponent, half_s, max_receptive, chunk_start, seq_len)


class TritonTelephoneAttention(TelephoneAttentionND):
    """1-D :class:`TelephoneAttentionND` under the reference's fused-variant name (``max_samples`` of that variant fixed the
    tap count; here it follows the sequence length as in the rank-generic class)."""

    def __init__(self, channels: int, num_heads: int = 8, max_samples: int = 32, max_freq: float = 16.0, min_freq: float = 1.0,
                 max_kernel_size: int = 64, chunk_size: int = 1024):
        super().__init__(channels, ndim=1, num_heads=num_heads, max_freq=max_freq, min_freq=min_freq, max_kernel_size=max_kernel_size,
                         chunk_size=chunk_size)
        self.max_samples = max_samples


__all__ = ["HAS_TRITON", "TritonTelephoneAttention", "triton_linear", "triton_linear_rmsnorm_silu", "triton_linear_silu", "triton_rmsnorm_silu",
           "triton_silu", "triton_telephone_attn", "triton_telephone_attn_with_decay"]
