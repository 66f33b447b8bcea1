"""Newton-Schulz / Polar-Express orthogonalisation on the tcgen05 GEMM.

Each iteration is three batched GEMMs with the polynomial folded into their epilogues
(``A = X·Xᵀ``, ``B = b·A + c·A·A``, ``X ← a·X + B·X``); tall matrices are handled through the operand-majorness flags
(``A = Xᵀ·X``, ``X ← a·X + X·B``) so no transposed copy is ever made. Counterparts in the reference:
``zeropower_via_newtonschulz5`` (records/track_1_short/2025-01-26_BatchSize/...txt:110-133) and ``polar_express`` with
the Triton ``XXT`` / ``ba_plus_cAA`` kernels (modded-nanogpt/train_gpt.py:143-195, triton_kernels.py:54-254).
"""
from __future__ import annotations

import torch

from . import gemm as G

NS5_COEFFS = [(3.4445, -4.7750, 2.0315)] * 5

# Per-iteration coefficients of the "Polar Express" schedule (Amsel et al., 2025), safety factor 1.01 folded in.
POLAR_EXPRESS_COEFFS = [
    (8.156554524902461, -22.48329292557795, 15.878769915207462),
    (4.042929935166739, -2.808917465908714, 0.5000178451051316),
    (3.8916678022926607, -2.772484153217685, 0.5060648178503393),
    (3.285753657755655, -2.3681294933425376, 0.46449024233003106),
    (2.3465413258596377, -1.7097828382687081, 0.42323551169305323),
]


def newton_schulz_torch(G_: torch.Tensor, coeffs=NS5_COEFFS, eps: float = 1e-7, norm_scale: float = 1.0) -> torch.Tensor:
    """Plain-torch restatement (any device); input of any float dtype, result bf16 (as the reference computes it)."""
    X = G_.bfloat16()
    tall = G_.size(-2) > G_.size(-1)
    if tall:
        X = X.mT
    X = X / (X.norm(dim=(-2, -1), keepdim=True) * norm_scale + eps)
    for a, b, c in coeffs:
        A = X @ X.mT
        B = b * A + c * A @ A
        X = a * X + B @ X
    return X.mT if tall else X


def newton_schulz_(X: torch.Tensor, coeffs=NS5_COEFFS, work: dict | None = None) -> torch.Tensor:
    """Orthogonalises the batch ``X [B, r, c]`` (bf16, CUDA, already divided by its Frobenius norm).

    Returns a tensor holding the result: the ping-pong buffer kept in ``work`` after an odd number of iterations, ``X``
    itself after an even number. ``X`` is overwritten either way. The ping-pong buffer of a ``work`` dict never changes
    identity, so a caller that passes the same ``X`` every step never meets a GEMM whose output aliases its operand
    (handing the buffers back swapped would make the second call run ``X <- a X + B X`` in place: tiles of ``X`` that
    other CTAs still have to read would be overwritten)."""
    assert X.is_cuda and X.dtype == torch.bfloat16 and X.dim() == 3
    bsz, r, c = X.shape
    wide = r <= c
    n = min(r, c)
    work = {} if work is None else work
    key = (bsz, r, c)
    bufs = work.get(key)
    if bufs is None:
        bufs = (torch.empty(bsz, n, n, dtype=torch.bfloat16, device=X.device),
                torch.empty(bsz, n, n, dtype=torch.bfloat16, device=X.device), torch.empty_like(X))
        work[key] = bufs
    A, Bm, X2 = bufs
    assert X2.data_ptr() != X.data_ptr(), "newton_schulz_: X must not be the work dict's own ping-pong buffer"
    for a_, b_, c_ in coeffs:
        if wide:
            G.gemm(X, X, out=A)
        else:
            G.gemm(X, X, a_mn=True, b_mn=True, out=A)
        G.gemm(A, A, out=Bm, epilogue=G.EPI_AXPBY, aux=A, alpha=c_, beta=b_)
        if wide:
            G.gemm(Bm, X, b_mn=True, out=X2, epilogue=G.EPI_AXPBY, aux=X, alpha=1.0, beta=a_)
        else:
            G.gemm(X, Bm, out=X2, epilogue=G.EPI_AXPBY, aux=X, alpha=1.0, beta=a_)
        X, X2 = X2, X
    return X


class GraphedNewtonSchulz:
    """The Newton-Schulz iteration of one stack captured once as a CUDA graph and replayed every step.

    One orthogonalisation is 15 dependent GEMM launches on small matrices; issued one by one, the host cost of each
    launch (argument checks, tensor-map encoding, the launch itself) is of the order of the kernel's run time. The
    stack ``X`` is a persistent buffer (the optimizer writes the normalised update into it every step), the work
    buffers and coefficients never change, so the whole chain is static: it is captured after one eager warm-up on
    placeholder data and replayed with a single graph launch on whatever stream is current. Independent stacks
    replayed on different streams run side by side, which matters because a single small GEMM does not fill 148 SMs.

    ``X`` is overwritten by the iteration (ping-pong with a work buffer); the result is :attr:`out`.
    """

    def __init__(self, X: torch.Tensor, coeffs=NS5_COEFFS):
        from . import runtime

        assert X.is_cuda and X.dtype == torch.bfloat16 and X.dim() == 3 and X.is_contiguous()
        self.X, self.coeffs = X, [tuple(c) for c in coeffs]
        self._work: dict = {}
        keep = X.clone()
        side = torch.cuda.Stream(X.device)
        side.wait_stream(torch.cuda.current_stream(X.device))
        with torch.cuda.stream(side):
            X.normal_(0, 1.0 / max(X.shape[-1], X.shape[-2]) ** 0.5)          # placeholder with a sane spectrum
            newton_schulz_(X, self.coeffs, self._work)                        # eager warm-up: kernels get configured
            n0 = runtime.launch_count()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=side, capture_error_mode="thread_local"):
                self.out = newton_schulz_(X, self.coeffs, self._work)
            self.launches = runtime.launch_count() - n0
            X.copy_(keep)
        torch.cuda.current_stream(X.device).wait_stream(side)

    def __call__(self) -> torch.Tensor:
        from . import runtime

        self.graph.replay()
        runtime.add_launches(self.launches)
        return self.out
