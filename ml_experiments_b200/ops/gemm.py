"""tcgen05/TMEM GEMM front end.

``gemm(a, b)`` computes ``epilogue(a @ b.T)`` on the fifth-generation tensor cores. Each operand may be given
K-major (``[rows, K]``, the default) or MN-major (``[K, rows]``, flag ``a_mn`` / ``b_mn``), which lets the three
products of a linear layer run on the stored tensors without a transpose pass:

* forward      ``y  = x @ W.T``   -> ``gemm(x, W)``
* data grad    ``dx = dy @ W``    -> ``gemm(dy, W, b_mn=True)``
* weight grad  ``dW = dy.T @ x``  -> ``gemm(dy, x, a_mn=True, b_mn=True)``

Counterpart of the cuBLAS / ``torch._scaled_mm`` / Triton ``tl.dot`` call sites of the reference
(modded-nanogpt/train_gpt.py:45-137,171-189,950,969; modded-nanogpt/triton_kernels.py:54-391).
"""
from __future__ import annotations

import torch

from .runtime import ops, status

EPI_NONE, EPI_RELU2, EPI_AXPBY, EPI_RELU2_BWD = 0, 1, 2, 3


def _overlap(x: torch.Tensor, y: torch.Tensor) -> bool:
    """True when the memory spans of two tensors intersect (conservative for strided views)."""
    if x.numel() == 0 or y.numel() == 0 or x.device != y.device:
        return False
    span = lambda t: (t.data_ptr(), t.data_ptr() + (sum((n - 1) * abs(st) for n, st in zip(t.shape, t.stride())) + 1) * t.element_size())
    (x0, x1), (y0, y1) = span(x), span(y)
    return x0 < y1 and y0 < x1


def gemm(a: torch.Tensor, b: torch.Tensor, *, out: torch.Tensor | None = None, out_dtype=None,
         a_mn: bool = False, b_mn: bool = False, epilogue: int = EPI_NONE, aux: torch.Tensor | None = None,
         alpha: float = 1.0, beta: float = 0.0, split_k: int = 1, accumulate: bool = False) -> torch.Tensor:
    """``out = epilogue(alpha * a @ b.T [+ beta * aux])``; 2-D or batched 3-D operands, bf16 or fp8 inputs."""
    m = a.shape[-1] if a_mn else a.shape[-2]
    n = b.shape[-1] if b_mn else b.shape[-2]
    if out is None:
        if out_dtype is None:
            out_dtype = torch.float32 if (split_k > 1 or accumulate) else torch.bfloat16
        out = torch.empty(*a.shape[:-2], m, n, dtype=out_dtype, device=a.device)
    elif _overlap(out, a) or _overlap(out, b):
        # an output tile is stored while other CTAs still read the operand panels: the result would depend on timing
        raise ValueError("gemm: `out` must not alias an operand")
    ops().gemm(a, b, out, aux, a_mn, b_mn, epilogue, alpha, beta, split_k, accumulate, status(a.device))
    return out


def auto_split_k(m: int, n: int, k: int, sms: int = 148) -> int:
    """Split factor that fills the machine when the output has fewer tiles than there are SMs."""
    bn = 256 if n > 128 else 128
    tiles = ((m + 127) // 128) * ((n + bn - 1) // bn)
    if tiles >= sms or k < 1024:
        return 1
    s = max(1, sms // tiles)
    return max(1, min(s, k // 512))
