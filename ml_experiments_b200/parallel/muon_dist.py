"""Data-parallel Muon with sharded momentum (one process per GPU).

Work split (world size W): the hidden matrices are stacked per shape into batches padded to a multiple of W; rank k
owns a contiguous slice of every batch. One step is

1. reduce-scatter of the stacked fp32 gradients (average over ranks) into the owner's slice,
2. momentum + Nesterov + Frobenius normalisation + Newton-Schulz on the owned slice only (tcgen05 batched GEMMs),
3. all-gather of the orthogonalised bf16 updates,
4. every rank applies ``p += alpha * U`` to its full replica and refreshes the bf16 shadow used by the forward GEMMs.

The reference distributes the same math by round-robin parameter ownership with per-parameter ``all_reduce`` of the
gradients and ``all_gather_into_tensor`` of the updates
(records/track_1_short/2025-01-26_BatchSize/c44090cc-...txt:134-212,600); sharding the reduce-scatter instead moves
1/W of the gradient bytes per rank and keeps momentum state sharded. The collectives are issued through
:class:`Collectives`, which uses the fused peer-memory kernels of :mod:`ml_experiments_b200.parallel.symm` when they
are available and NCCL otherwise.
"""
from __future__ import annotations

from collections import defaultdict

import torch
import torch.distributed as dist

from ..ops.newton_schulz import NS5_COEFFS, newton_schulz_
from ..ops.runtime import ops
from ..utils.shadow import get_shadow_buffer, set_shadow


class GradSync:
    """Averages the gradients of everything that is not a Muon matrix (embeddings, head, scalars) over the ranks."""

    def __init__(self, model, muon_params, rank: int, world_size: int, group=None):
        self.rank, self.world, self.group = rank, world_size, group
        muon_ids = {id(p) for p in muon_params}
        self.params = [p for p in model.parameters() if id(p) not in muon_ids]
        self._small = [p for p in self.params if p.numel() < 65536]
        self._large = [p for p in self.params if p.numel() >= 65536]
        self._flat = None

    @torch.no_grad()
    def sync_non_muon_grads(self):
        works = []
        for p in self._large:
            if p.grad is not None:
                works.append(dist.all_reduce(p.grad, op=dist.ReduceOp.AVG, group=self.group, async_op=True))
        small = [p for p in self._small if p.grad is not None]
        if small:
            flat = torch.cat([p.grad.reshape(-1).float() for p in small])
            dist.all_reduce(flat, op=dist.ReduceOp.AVG, group=self.group)
            off = 0
            for p in small:
                n = p.numel()
                p.grad.copy_(flat[off:off + n].view_as(p.grad))
                off += n
        for w in works:
            w.wait()


class DistMuon(torch.optim.Optimizer):
    def __init__(self, params, comm: GradSync, lr: float = 0.02, momentum: float = 0.95, nesterov: bool = True,
                 ns_steps: int = 5):
        params = [*params]
        super().__init__(params, dict(lr=lr, momentum=momentum, nesterov=nesterov, ns_steps=ns_steps))
        self.rank, self.world, self.group = comm.rank, comm.world, comm.group
        self._work: dict = {}
        self._groups = None

    def _build(self, params):
        W = self.world
        by_shape = defaultdict(list)
        for p in params:
            r, c = p.shape[-2], p.shape[-1]
            by_shape[(r, c)].append((p, p.numel() // (r * c)))
        groups = []
        for (r, c), plist in by_shape.items():
            total = sum(n for _, n in plist)
            padded = (total + W - 1) // W * W
            per = padded // W
            dev = plist[0][0].device
            groups.append(dict(
                r=r, c=c, plist=plist, total=total, per=per,
                g_full=torch.zeros(padded, r, c, dtype=torch.float32, device=dev),
                g_shard=torch.empty(per, r, c, dtype=torch.float32, device=dev),
                mom=torch.zeros(per, r, c, dtype=torch.float32, device=dev),
                u_shard=torch.empty(per, r, c, dtype=torch.bfloat16, device=dev),
                u_full=torch.empty(padded, r, c, dtype=torch.bfloat16, device=dev),
                sumsq=torch.zeros(per, dtype=torch.float32, device=dev)))
        self._groups = groups

    @torch.no_grad()
    def step(self, closure=None):
        group = self.param_groups[0]
        params = [p for p in group["params"] if p.grad is not None]
        if self._groups is None:
            self._build(params)
        o = ops()
        mu, nesterov, lr = float(group["momentum"]), bool(group["nesterov"]), float(group["lr"])
        coeffs = [NS5_COEFFS[0]] * group["ns_steps"]
        # 1. stack gradients and launch every reduce-scatter
        works = []
        for g in self._groups:
            views, srcs, slot = [], [], 0
            for p, nmat in g["plist"]:
                views.append(g["g_full"][slot:slot + nmat].view(p.shape))
                srcs.append(p.grad if p.grad.dtype == torch.float32 else p.grad.float())
                slot += nmat
            torch._foreach_copy_(views, srcs)
            works.append(dist.reduce_scatter_tensor(g["g_shard"], g["g_full"], op=dist.ReduceOp.AVG, group=self.group,
                                                    async_op=True))
        # 2. owner-side momentum + Newton-Schulz, 3. all-gather of the bf16 updates
        gathers = []
        for g, w in zip(self._groups, works):
            w.wait()
            per = g["per"]
            g["sumsq"].zero_()
            for j in range(per):
                o.muon_momentum(g["g_shard"][j], g["mom"][j], g["u_shard"][j], g["sumsq"][j:j + 1], mu, nesterov, 1.0)
                o.scale_by_inv_norm(g["u_shard"][j], g["sumsq"][j:j + 1], 1e-7)
            u = newton_schulz_(g["u_shard"], coeffs, self._work)
            gathers.append(dist.all_gather_into_tensor(g["u_full"], u.contiguous(), group=self.group, async_op=True))
        # 4. apply on every replica
        for g, w in zip(self._groups, gathers):
            w.wait()
            alpha = -lr * max(1.0, g["r"] / g["c"]) ** 0.5
            slot = 0
            for p, nmat in g["plist"]:
                upd = g["u_full"][slot:slot + nmat].view(p.shape)
                sh = get_shadow_buffer(p, torch.bfloat16)
                if sh is None:
                    sh = torch.empty(p.shape, dtype=torch.bfloat16, device=p.device)
                o.axpy_bf16_to_f32(p, upd, sh, alpha)
                set_shadow(p, sh)
                slot += nmat
        return None
