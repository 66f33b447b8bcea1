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

import os

from ..ops.newton_schulz import NS5_COEFFS, GraphedNewtonSchulz, newton_schulz_
from ..ops.runtime import ops
from ..utils.shadow import get_shadow_buffer, mark_modified, set_shadow


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


def _momentum_shards(groups) -> dict:
    return {f"mom_{g['r']}x{g['c']}": g["mom"].detach().clone() for g in groups}


def _load_momentum(groups, shard: dict) -> None:
    for g in groups:
        t = shard.get(f"mom_{g['r']}x{g['c']}")
        if t is None:
            continue
        if tuple(t.shape) != tuple(g["mom"].shape):
            raise ValueError(f"momentum shard {tuple(t.shape)} does not fit this rank's slice {tuple(g['mom'].shape)}: "
                             "load it through utils.checkpoint.load_sharded, which re-partitions for the world size")
        g["mom"].copy_(t)


class DistMuon(torch.optim.Optimizer):
    def __init__(self, params, comm: GradSync, lr: float = 0.02, momentum: float = 0.95, nesterov: bool = True,
                 ns_steps: int = 5):
        params = [*params]
        super().__init__(params, dict(lr=lr, momentum=momentum, nesterov=nesterov, ns_steps=ns_steps))
        self.rank, self.world, self.group = comm.rank, comm.world, comm.group
        self._work: dict = {}
        self._groups = None
        self._pending_shard = None

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
        if self._pending_shard is not None:
            _load_momentum(self._groups, self._pending_shard)
            self._pending_shard = None

    # -- sharded momentum: lives in the per-shape stacks, not in ``Optimizer.state`` (one slice per rank)
    def sharded_state(self) -> dict:
        """``{"mom_{rows}x{cols}": this rank's [per, rows, cols] momentum slice}`` (empty before the first step)."""
        return _momentum_shards(self._groups or [])

    def sharded_rows(self) -> dict:
        """Number of real (unpadded) matrices per stack, for re-partitioning under another world size."""
        return {f"mom_{g['r']}x{g['c']}": g["total"] for g in (self._groups or [])}

    def load_sharded_state(self, shard: dict) -> None:
        if self._groups is None:
            self._pending_shard = shard        # the stacks are built at the first step
        else:
            _load_momentum(self._groups, shard)

    @torch.no_grad()
    def step(self, closure=None):
        group = self.param_groups[0]
        params = [p for p in group["params"] if p.grad is not None]
        if self._groups is None:
            self._build(params)
        mu, nesterov, lr = float(group["momentum"]), bool(group["nesterov"]), float(group["lr"])
        coeffs = [NS5_COEFFS[0]] * group["ns_steps"]
        if not params[0].is_cuda:
            return self._step_host(mu, nesterov, lr, coeffs)
        o = ops()
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
                mark_modified(p)
                set_shadow(p, sh)
                slot += nmat
        return None


    def _step_host(self, mu, nesterov, lr, coeffs):
        """The same work split in plain torch for CPU tensors (gloo ranks): what the host-side logic (ownership,
        padding, sharded momentum, checkpoints) is tested with where no GPU is present."""
        from ..ops.newton_schulz import newton_schulz_torch

        for g in self._groups:
            slot = 0
            for p, nmat in g["plist"]:
                g["g_full"][slot:slot + nmat].view(p.shape).copy_(p.grad.float())
                slot += nmat
            if self.world > 1:
                # gloo has no reduce-scatter: all-reduce the stack and keep the owned slice
                dist.all_reduce(g["g_full"], op=dist.ReduceOp.SUM, group=self.group)
                g["g_full"].div_(self.world)
            per = g["per"]
            mine = g["g_full"][self.rank * per:(self.rank + 1) * per]
            g["mom"].lerp_(mine, 1 - mu)
            u = mine.lerp(g["mom"], mu) if nesterov else g["mom"]
            g["u_shard"].copy_(newton_schulz_torch(u, coeffs))
            if self.world > 1:
                parts = [torch.empty_like(g["u_shard"]) for _ in range(self.world)]
                dist.all_gather(parts, g["u_shard"].contiguous(), group=self.group)
                g["u_full"].copy_(torch.cat(parts, 0))
            else:
                g["u_full"].copy_(g["u_shard"])
            alpha = -lr * max(1.0, g["r"] / g["c"]) ** 0.5
            slot = 0
            for p, nmat in g["plist"]:
                p.add_(g["u_full"][slot:slot + nmat].view(p.shape).to(p.dtype), alpha=alpha)
                mark_modified(p)
                slot += nmat
        return None


# ======================================================================================================================
# Fused path: the same work split, with both collectives done by this package's kernels over peer memory
# ======================================================================================================================
CH_GRADS, CH_AG, CH_B16_IN, CH_B16_OUT, CH_F32_IN, CH_F32_OUT = 0, 1, 2, 3, 4, 5
CH_AG_GROUP0, MAX_CONCURRENT_GROUPS = 12, 4     # one "pushed" channel per shape group when the groups run concurrently


class MuonShardEngine:
    """Banked Muon state of one rank plus the three phases of a fused step.

    * ``publish_grads``   : gradients -> this rank's symmetric fp32 stack, then "ready" flag to every peer;
    * ``reduce_ns_push``  : per shape group, one kernel reduce-scatters the owned slice straight out of the peers'
      stacks into the momentum update / bf16 cast, Newton-Schulz runs on the slice, one kernel stores the
      result into every peer's update buffer and raises the "pushed" flag;
    * ``apply``           : waits for every rank's push, then ``p += alpha * U`` on the banked fp32 masters and
      refreshes the banked bf16 copies in the same kernel.

    Master weights and their bf16 copies live in per-shape banks; the ``nn.Parameter`` objects are views into them.
    """

    def __init__(self, params, world, alloc=None):
        from ..utils.shadow import set_shadow as _set

        self.w = world
        self.params = [*params]
        alloc = alloc or world.alloc
        W = world.world
        by_shape = defaultdict(list)
        for p in self.params:
            r, c = p.shape[-2], p.shape[-1]
            by_shape[(r, c)].append((p, p.numel() // (r * c)))
        self.groups = []
        dev = self.params[0].device
        for (r, c), plist in by_shape.items():
            total = sum(n for _, n in plist)
            padded = (total + W - 1) // W * W
            per = padded // W
            g = dict(r=r, c=c, plist=plist, total=total, per=per, padded=padded, mat=r * c)
            g["g_full"] = alloc(padded * r * c, torch.float32)
            g["u_full"] = alloc(padded * r * c, torch.bfloat16)
            g["g_full"].local.zero_()
            g["p_stack"] = torch.zeros(padded, r, c, dtype=torch.float32, device=dev)
            slot = 0
            with torch.no_grad():
                for p, nmat in plist:
                    view = g["p_stack"][slot:slot + nmat].view(p.shape)
                    view.copy_(p.detach())
                    p.data = view
                    slot += nmat
            g["sh_stack"] = g["p_stack"].to(torch.bfloat16)
            slot = 0
            for p, nmat in plist:
                _set(p, g["sh_stack"][slot:slot + nmat].view(p.shape))
                slot += nmat
            g["mom"] = torch.zeros(per, r, c, dtype=torch.float32, device=dev)
            g["u_shard"] = torch.empty(per, r, c, dtype=torch.bfloat16, device=dev)
            g["sumsq"] = torch.zeros(per, dtype=torch.float32, device=dev)
            self.groups.append(g)
        self._work: dict = {}
        self._step = 0
        self._streams = None
        self._concurrent = False

    def grad_views(self) -> dict:
        """``{id(param): fp32 view}`` of this rank's peer-mapped gradient stacks: a backward that writes a matrix's
        gradient there (and makes the view ``p.grad``) needs no copy in :meth:`publish_grads`. Safe to overwrite once
        :meth:`apply` of the previous step has returned: every peer has pushed by then, and a peer pushes after its
        last read of these stacks."""
        out = {}
        for g in self.groups:
            flat, slot = g["g_full"].local.view(g["padded"], g["r"], g["c"]), 0
            for p, nmat in g["plist"]:
                out[id(p)] = flat[slot:slot + nmat].view(p.shape)
                slot += nmat
        return out

    @torch.no_grad()
    def publish_grads(self):
        from ..ops.runtime import status

        o = ops()
        for g in self.groups:
            views, srcs, slot = [], [], 0
            flat = g["g_full"].local.view(g["padded"], g["r"], g["c"])
            for p, nmat in g["plist"]:
                if p.grad is not None:
                    view = flat[slot:slot + nmat].view(p.shape)
                    if p.grad.data_ptr() != view.data_ptr():      # not written in place by the producing kernel
                        views.append(view)
                        srcs.append(p.grad if p.grad.dtype == torch.float32 else p.grad.float())
                slot += nmat
            if views:
                torch._foreach_copy_(views, srcs)
        self._step += 1
        o.comm_signal(self.w.flags.ptrs, self.w.rank, CH_GRADS, self._step, self.w.flags.local)
        self._status = status(self.params[0].device)

    @torch.no_grad()
    def reduce_ns_push(self, mu: float, nesterov: bool, coeffs):
        """Every shape group is an independent chain (reduce-scatter + momentum -> normalise -> Newton-Schulz -> push)
        and runs on its own stream, so that the link-bound collectives of one group overlap the GEMMs of another and
        small GEMMs of different groups share the machine. The 15 GEMMs of a group are one CUDA-graph launch
        (``B200_NS_GRAPH=0`` issues them one by one)."""
        o = ops()
        w = self.w
        ng = len(self.groups)
        use_graph = os.environ.get("B200_NS_GRAPH", "1") == "1"
        # concurrent groups need a flag channel each: a group that finishes early must not satisfy (or later undo) the
        # wait for another group's push
        concurrent = 1 < ng <= MAX_CONCURRENT_GROUPS and os.environ.get("B200_MUON_STREAMS", "1") == "1"
        self._concurrent = concurrent
        cur = torch.cuda.current_stream()
        if self._streams is None:
            self._streams = [torch.cuda.Stream() for _ in self.groups]
        fork = torch.cuda.Event()
        fork.record(cur)
        for gi, g in enumerate(self.groups):
            st = self._streams[gi] if concurrent else cur
            with torch.cuda.stream(st):
                if st is not cur:
                    st.wait_event(fork)
                per, mat = g["per"], g["mat"]
                g["sumsq"].zero_()
                o.muon_rs_momentum(g["g_full"].ptrs, w.rank * per * mat, per, mat, g["mom"], g["u_shard"], g["sumsq"], mu,
                                   nesterov, w.flags.local, CH_GRADS, self._step, self._status)
                o.stack_scale_by_inv_norm(g["u_shard"], g["sumsq"], per, mat, 1e-7)
                key = tuple(tuple(c) for c in coeffs)
                if use_graph:
                    if g.get("ns_key") != key:
                        g["ns"], g["ns_key"] = GraphedNewtonSchulz(g["u_shard"], coeffs), key
                    u = g["ns"]()
                else:
                    u = newton_schulz_(g["u_shard"], coeffs, self._work)
                if concurrent:
                    o.ag_push(u.contiguous(), g["u_full"].ptrs, w.rank, w.rank * per * mat, w.flags.ptrs, CH_AG_GROUP0 + gi,
                              self._step, gi + 1)
                else:
                    o.ag_push(u.contiguous(), g["u_full"].ptrs, w.rank, w.rank * per * mat, w.flags.ptrs, CH_AG,
                              (self._step - 1) * ng + gi + 1, 0)
        if concurrent:
            for st in self._streams:
                cur.wait_stream(st)

    @torch.no_grad()
    def apply(self, lr: float):
        o = ops()
        w = self.w
        ng = len(self.groups)
        for gi, g in enumerate(self.groups):
            alpha = -lr * max(1.0, g["r"] / g["c"]) ** 0.5
            ch, ep = (CH_AG_GROUP0 + gi, self._step) if self._concurrent else (CH_AG, (self._step - 1) * ng + gi + 1)
            o.ag_wait_apply(g["p_stack"], g["u_full"].local, g["sh_stack"], alpha, w.world, w.flags.local, ch, ep, self._status)
            slot = 0
            for p, nmat in g["plist"]:
                mark_modified(p)
                set_shadow(p, g["sh_stack"][slot:slot + nmat].view(p.shape))
                slot += nmat


class FusedDistMuon(torch.optim.Optimizer):
    """Muon whose reduce-scatter and all-gather are fused into its own kernels over NVLink peer memory."""

    def __init__(self, params, world, lr: float = 0.02, momentum: float = 0.95, nesterov: bool = True, ns_steps: int = 5):
        params = [*params]
        super().__init__(params, dict(lr=lr, momentum=momentum, nesterov=nesterov, ns_steps=ns_steps))
        self.engine = MuonShardEngine(params, world)

    def grad_views(self) -> dict:
        return self.engine.grad_views()

    def sharded_state(self) -> dict:
        return _momentum_shards(self.engine.groups)

    def sharded_rows(self) -> dict:
        return {f"mom_{g['r']}x{g['c']}": g["total"] for g in self.engine.groups}

    def load_sharded_state(self, shard: dict) -> None:
        _load_momentum(self.engine.groups, shard)

    @torch.no_grad()
    def step(self, closure=None):
        g = self.param_groups[0]
        self.engine.publish_grads()
        self.engine.reduce_ns_push(float(g["momentum"]), bool(g["nesterov"]), [NS5_COEFFS[0]] * g["ns_steps"])
        self.engine.apply(float(g["lr"]))
        return None


class FusedGradSync:
    """Mean all-reduce of the non-Muon gradients (embeddings, head, scalars) by the two-shot peer-memory kernel.

    Gradients are packed into one bf16 and one fp32 symmetric bucket, reduced in place (each rank reduces 1/W of the
    bucket out of all peers and stores the scaled result into every peer), and ``p.grad`` is re-pointed at the bucket
    views, so nothing is copied back."""

    def __init__(self, model, muon_params, world, alloc=None):
        self.w = world
        alloc = alloc or world.alloc
        muon_ids = {id(p) for p in muon_params}
        self.params = [p for p in model.parameters() if id(p) not in muon_ids]
        self.p16 = [p for p in self.params if p.dtype == torch.bfloat16]
        self.p32 = [p for p in self.params if p.dtype != torch.bfloat16]

        def pad(n, m):
            return (n + m - 1) // m * m

        self.n16 = pad(sum(pad(p.numel(), 8) for p in self.p16), 8 * world.world) if self.p16 else 0
        self.n32 = pad(sum(pad(p.numel(), 4) for p in self.p32), 4 * world.world) if self.p32 else 0
        self.b16 = alloc(max(self.n16, 8), torch.bfloat16)
        self.b32 = alloc(max(self.n32, 4), torch.float32)
        self.b16.local.zero_()
        self.b32.local.zero_()
        self.views16, off = [], 0
        for p in self.p16:
            self.views16.append(self.b16.local[off:off + p.numel()].view(p.shape))
            off += pad(p.numel(), 8)
        self.views32, off = [], 0
        for p in self.p32:
            self.views32.append(self.b32.local[off:off + p.numel()].view(p.shape))
            off += pad(p.numel(), 4)
        self._step = 0

    @torch.no_grad()
    def publish(self):
        from ..ops.runtime import status

        o = ops()
        for plist, views in ((self.p16, self.views16), (self.p32, self.views32)):
            pairs = [(v, p.grad) for p, v in zip(plist, views) if p.grad is not None]
            if pairs:
                torch._foreach_copy_([a for a, _ in pairs], [b if b.dtype == a.dtype else b.to(a.dtype) for a, b in pairs])
        self._step += 1
        self._status = status(self.w.flags.local.device)
        o.comm_signal(self.w.flags.ptrs, self.w.rank, CH_B16_IN, self._step, self.w.flags.local)
        o.comm_signal(self.w.flags.ptrs, self.w.rank, CH_F32_IN, self._step, self.w.flags.local)

    @torch.no_grad()
    def reduce(self):
        o = ops()
        w = self.w
        if self.n16:
            o.allreduce_mean(self.b16.ptrs, w.rank, self.n16, 1, w.flags.local, w.flags.ptrs, CH_B16_IN, self._step, self._status)
        if self.n32:
            o.allreduce_mean(self.b32.ptrs, w.rank, self.n32, 0, w.flags.local, w.flags.ptrs, CH_F32_IN, self._step, self._status)

    @torch.no_grad()
    def wait(self):
        """Device-side wait until every peer has stored its reduced slice into this rank's buckets."""
        o = ops()
        w = self.w
        if self.n16:
            o.comm_wait(w.flags.local, w.world, CH_B16_OUT, self._step, self._status)
        if self.n32:
            o.comm_wait(w.flags.local, w.world, CH_F32_OUT, self._step, self._status)

    @torch.no_grad()
    def adopt(self):
        """Point ``p.grad`` at the reduced bucket views (host-side only)."""
        for plist, views in ((self.p16, self.views16), (self.p32, self.views32)):
            for p, v in zip(plist, views):
                if p.grad is not None:
                    p.grad = v

    def finish(self):
        self.wait()
        self.adopt()

    def sync_non_muon_grads(self):
        self.publish()
        self.reduce()
        self.finish()

    # -- overlapped form: the link-bound all-reduce runs on a side stream while the caller's stream does other work
    def start_async(self):
        """Publish on the current stream, then reduce + wait on a side stream. The signals every peer waits for are
        all enqueued before the fork, so no kernel of either stream waits on work queued behind a waiting kernel."""
        self.publish()
        cur = torch.cuda.current_stream()
        if getattr(self, "_side", None) is None:
            self._side = torch.cuda.Stream()
        self._side.wait_stream(cur)
        with torch.cuda.stream(self._side):
            self.reduce()
            self.wait()

    def join_async(self):
        torch.cuda.current_stream().wait_stream(self._side)
        self.adopt()
