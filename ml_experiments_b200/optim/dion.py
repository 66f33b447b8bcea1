"""Dion: distributed orthonormalised updates by low-rank power iteration with error feedback.

The reference repository contains no Dion; this follows the published algorithm (Ahn, Xu, Abreu, Langford, "Dion:
Distributed Orthonormalized Updates", 2025, Algorithm 1/3). Per matrix ``W (m x n)`` with momentum ``M`` and right
basis ``Q (n x r)``, ``r = rank_fraction * min(m, n)``:

    B = M + G                      (G is this rank's local gradient in the data-parallel variant)
    P = B Q              -> mean over ranks            (m x r)
    P = orthonormalise(P)                              (Newton-Schulz on the GEMM kernel; Cholesky-QR / Householder QR)
    R = Bᵀ P             -> mean over ranks            (n x r)
    M = B - (1 - mu) P Rᵀ                              (error feedback: what the low-rank step missed stays in M)
    Q = R with unit-norm columns
    W = (1 - lr * wd) W - lr * sqrt(m / n) * P Qᵀ

Only ``P`` and ``R`` (``(m + n) r`` numbers instead of ``m n``) cross the network. Matrices of equal shape are stacked
and processed as batches: the products run on the tcgen05 GEMM (bf16 operands, fp32 accumulation) and the two means
use the peer-memory all-reduce kernel when a :class:`~ml_experiments_b200.parallel.symm.SymmWorld` is given, NCCL when
only a process group exists, nothing for a single process.

Orthonormalisation on CUDA defaults to ``ortho="ns"``: five Polar-Express Newton-Schulz iterations on the stacked
``m x r`` blocks, i.e. 15 batched tcgen05 GEMMs with no factorisation, no library call and no host synchronisation
(Cholesky-QR has to read back whether the factorisation succeeded). The columns come out orthonormal up to the
iteration's tolerance (singular values within a few percent of 1); what the slightly inexact projector misses stays in
the momentum through the error-feedback line. ``"cholqr"`` and ``"qr"`` remain for CPU runs and exact comparisons.
"""
from __future__ import annotations

from collections import defaultdict

import torch
import torch.distributed as dist

from ..ops import gemm as G


def orthonormalize(P: torch.Tensor, method: str = "cholqr") -> torch.Tensor:
    """Orthonormal basis of the column space of each ``P[b] (m x r)`` (fp32)."""
    if method == "ns":
        from ..ops.newton_schulz import POLAR_EXPRESS_COEFFS, newton_schulz_, newton_schulz_torch

        scale = P.float().norm(dim=(-2, -1), keepdim=True) * 1.02 + 1e-6
        if P.is_cuda and P.dim() == 3 and all(d % 8 == 0 for d in P.shape[-2:]):
            X = (P.float() / scale).to(torch.bfloat16).contiguous()
            return newton_schulz_(X, POLAR_EXPRESS_COEFFS).float()
        return newton_schulz_torch(P, POLAR_EXPRESS_COEFFS, eps=1e-6, norm_scale=1.02).float()
    if method == "qr":
        return torch.linalg.qr(P, mode="reduced").Q
    gram = P.transpose(-1, -2) @ P
    eye = torch.eye(P.shape[-1], device=P.device, dtype=P.dtype)
    gram = gram + 1e-6 * gram.diagonal(dim1=-2, dim2=-1).mean(-1)[..., None, None].clamp(min=1e-30) * eye
    L, info = torch.linalg.cholesky_ex(gram)
    if bool((info != 0).any()):
        return torch.linalg.qr(P, mode="reduced").Q
    return torch.linalg.solve_triangular(L, P.transpose(-1, -2), upper=False).transpose(-1, -2)


def _bmm(a: torch.Tensor, b: torch.Tensor, a_t: bool = False) -> torch.Tensor:
    """``a @ b`` (or ``aᵀ @ b``) in fp32; tcgen05 GEMM on CUDA when the shapes fit its TMA constraints."""
    ok = a.is_cuda and all(d % 8 == 0 for d in (a.shape[-1], a.shape[-2], b.shape[-1], b.shape[-2]))
    if not ok:
        return (a.transpose(-1, -2) if a_t else a).float() @ b.float()
    a16, b16 = a.to(torch.bfloat16).contiguous(), b.to(torch.bfloat16).contiguous()
    # out[m, r] = sum_k A[m, k] B[k, r]: B is stored [k, r] i.e. MN-major for the "N x K" operand
    return G.gemm(a16, b16, a_mn=a_t, b_mn=True, out_dtype=torch.float32)


class Dion(torch.optim.Optimizer):
    def __init__(self, params, lr: float = 0.01, mu: float = 0.95, rank_fraction: float = 0.25, weight_decay: float = 0.0,
                 ortho: str | None = None, world=None, process_group=None, seed: int = 0):
        params = [*params]
        if ortho is None:
            ortho = "ns" if params and params[0].is_cuda else "cholqr"
        super().__init__(params, dict(lr=lr, mu=mu, rank_fraction=rank_fraction, weight_decay=weight_decay))
        self.ortho, self.world, self.group, self.seed = ortho, world, process_group, seed
        self.distributed = world is not None or (dist.is_initialized() and dist.get_world_size(process_group) > 1)
        self._groups = None

    def _build(self, params, rank_fraction):
        by_shape = defaultdict(list)
        for p in params:
            by_shape[(p.shape[-2], p.shape[-1])].append(p)
        gen = torch.Generator().manual_seed(self.seed)
        self._groups = []
        for (m, n), plist in by_shape.items():
            k = sum(p.numel() // (m * n) for p in plist)
            r = max(1, int(min(m, n) * rank_fraction))
            r = max(8, r // 8 * 8) if min(m, n) >= 8 else r
            dev = plist[0].device
            Q = torch.linalg.qr(torch.randn(k, n, r, generator=gen)).Q.to(dev)
            g = dict(m=m, n=n, r=r, k=k, plist=plist, Q=Q.float(), M=torch.zeros(k, m, n, device=dev),
                     G=torch.empty(k, m, n, device=dev))
            slot, g["gviews"] = 0, []
            for p in plist:
                c = p.numel() // (m * n)
                g["gviews"].append(g["G"][slot:slot + c].view(p.shape))
                slot += c
            if self.world is not None:
                g["P_buf"] = self.world.alloc(k * m * r, torch.float32)
                g["R_buf"] = self.world.alloc(k * n * r, torch.float32)
            self._groups.append(g)
        self._epoch = 0

    def _mean(self, t: torch.Tensor, buf=None) -> torch.Tensor:
        if not self.distributed:
            return t
        if buf is not None:
            from ..ops.runtime import ops, status
            from ..parallel.muon_dist import CH_F32_IN, CH_F32_OUT

            w, o = self.world, ops()
            self._epoch += 1
            e = 1_000_000 + self._epoch  # own epoch range on the shared fp32 channels
            flat = buf.local[: t.numel()]
            flat.copy_(t.reshape(-1))
            o.comm_signal(w.flags.ptrs, w.rank, CH_F32_IN, e, w.flags.local)
            n = (t.numel() + 4 * w.world - 1) // (4 * w.world) * (4 * w.world)
            o.allreduce_mean(buf.ptrs, w.rank, min(n, buf.local.numel() // 4 * 4), 0, w.flags.local, w.flags.ptrs, CH_F32_IN, e,
                             status(t.device))
            o.comm_wait(w.flags.local, w.world, CH_F32_OUT, e, status(t.device))
            return flat.view_as(t)        # the next all-reduce of this buffer is enqueued after every consumer of the view
        dist.all_reduce(t, op=dist.ReduceOp.AVG, group=self.group)
        return t

    @torch.no_grad()
    def step(self, closure=None):
        hp = self.param_groups[0]
        params = [p for p in hp["params"] if p.grad is not None]
        if self._groups is None:
            self._build(params, hp["rank_fraction"])
        lr, mu, wd = float(hp["lr"]), float(hp["mu"]), float(hp["weight_decay"])
        for g in self._groups:
            m, n = g["m"], g["n"]
            torch._foreach_copy_(g["gviews"], [p.grad for p in g["plist"]])     # one multi-tensor copy (and cast) into the stack
            B = g["M"].add_(g["G"])
            P = self._mean(_bmm(B, g["Q"]), g.get("P_buf"))
            P = orthonormalize(P.float(), self.ortho)
            R = self._mean(_bmm(B, P, a_t=True), g.get("R_buf"))
            B.sub_(_bmm(P, R.transpose(-1, -2).contiguous()), alpha=1 - mu)      # M <- B - (1 - mu) P Rᵀ, in place
            Qn = R / R.norm(dim=-2, keepdim=True).clamp(min=1e-8)
            g["Q"] = Qn
            upd = _bmm(P, Qn.transpose(-1, -2).contiguous())
            scale = (m / n) ** 0.5
            slot = 0
            for p in g["plist"]:
                c = p.numel() // (m * n)
                if wd:
                    p.mul_(1 - lr * wd)
                p.add_(upd[slot:slot + c].view(p.shape).to(p.dtype), alpha=-lr * scale)
                slot += c
        return None
