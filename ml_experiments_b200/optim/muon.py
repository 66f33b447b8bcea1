"""Muon: momentum orthogonalised by Newton-Schulz (classic modded-nanogpt semantics).

Reference: ``Muon`` in records/track_1_short/2025-01-26_BatchSize/c44090cc-...txt:134-212 — fp32 momentum ``lerp``,
Nesterov mix, 5 quintic Newton-Schulz steps in bf16 on the (batched) 2-D update, update scale
``max(1, rows/cols)**0.5``. There the work is distributed by round-robin parameter ownership followed by
``all_gather_into_tensor``; here the single-process path stacks all equally shaped matrices into one batch and runs
the three GEMMs of each iteration on the tcgen05 kernel, and the multi-GPU path lives in
:mod:`ml_experiments_b200.parallel.muon_dist`.
"""
from __future__ import annotations

from collections import defaultdict

import torch

import os

from ..ops.newton_schulz import NS5_COEFFS, GraphedNewtonSchulz, newton_schulz_, newton_schulz_torch
from ..ops.runtime import ops
from ..utils.shadow import get_shadow_buffer, mark_modified, set_shadow


class Muon(torch.optim.Optimizer):
    def __init__(self, params, lr: float = 0.02, momentum: float = 0.95, nesterov: bool = True, ns_steps: int = 5,
                 rank: int = 0, world_size: int = 1):
        self.rank, self.world_size = rank, world_size
        defaults = dict(lr=lr, momentum=momentum, nesterov=nesterov, ns_steps=ns_steps)
        params = [*params]
        assert all(isinstance(p, torch.Tensor) for p in params)
        super().__init__(params, defaults)
        self._work: dict = {}
        self._stacks: dict = {}
        self._pending_shard = None
        self._streams: list = []

    # ------------------------------------------------------------------------------------------ torch path
    @torch.no_grad()
    def _step_torch(self, group):
        coeffs = NS5_COEFFS[: group["ns_steps"]] if group["ns_steps"] <= 5 else [NS5_COEFFS[0]] * group["ns_steps"]
        for p in group["params"]:
            if p.grad is None:
                continue
            g = p.grad.float()
            st = self.state[p]
            if "momentum_buffer" not in st:
                st["momentum_buffer"] = torch.zeros_like(g)
            buf = st["momentum_buffer"]
            buf.lerp_(g, 1 - group["momentum"])
            g = g.lerp(buf, group["momentum"]) if group["nesterov"] else buf
            u = newton_schulz_torch(g, coeffs)
            p.add_(u.to(p.dtype), alpha=-group["lr"] * max(1, p.size(-2) / p.size(-1)) ** 0.5)

    # ------------------------------------------------------------------------------------------ fused path
    def _slots(self, params):
        """Groups parameters by matrix shape; every 2-D slice of a parameter gets one slot of a stacked buffer."""
        key = tuple(id(p) for p in params)
        ent = self._stacks.get(key)
        if ent is not None:
            return ent
        by_shape = defaultdict(list)
        for p in params:
            r, c = p.shape[-2], p.shape[-1]
            nmat = p.numel() // (r * c)
            by_shape[(r, c)].append((p, nmat))
        out = []
        for (r, c), plist in by_shape.items():
            total = sum(n for _, n in plist)
            dev = plist[0][0].device
            ent = dict(r=r, c=c, plist=plist, total=total,
                       stack=torch.empty(total, r, c, dtype=torch.bfloat16, device=dev),       # normalised updates (NS input)
                       grads=torch.empty(total, r, c, dtype=torch.float32, device=dev),        # gradients, stacked
                       mom=torch.zeros(total, r, c, dtype=torch.float32, device=dev),          # momentum, stacked
                       sumsq=torch.zeros(total, dtype=torch.float32, device=dev))
            slot, ent["gviews"], ent["mviews"] = 0, [], []
            for p, nmat in plist:
                ent["gviews"].append(ent["grads"][slot:slot + nmat].view(p.shape))
                ent["mviews"].append(ent["mom"][slot:slot + nmat].view(p.shape))
                slot += nmat
            out.append(ent)
        self._stacks[key] = out
        return out

    @torch.no_grad()
    def _step_fused(self, group):
        """All matrices of one shape are one stack: one copy of the gradients into it, one momentum + sum-of-squares
        launch, one normalisation, one batched Newton-Schulz; only the weight update runs per parameter."""
        o = ops()
        mu, nesterov, lr = float(group["momentum"]), bool(group["nesterov"]), float(group["lr"])
        coeffs = [NS5_COEFFS[0]] * group["ns_steps"]
        params = [p for p in group["params"] if p.grad is not None]
        ents = self._slots(params)
        # every shape stack is an independent chain: on its own stream, with its 15 GEMMs replayed as one CUDA graph,
        # the small Newton-Schulz products of different shapes share the machine instead of running one after another
        use_graph = os.environ.get("B200_NS_GRAPH", "1") == "1"
        cur = torch.cuda.current_stream()
        side = len(ents) > 1 and os.environ.get("B200_MUON_STREAMS", "1") == "1"
        if side and len(self._streams) < len(ents):
            self._streams = [torch.cuda.Stream() for _ in ents]
        fork = torch.cuda.Event()
        fork.record(cur)
        for ei, ent in enumerate(ents):
            st = self._streams[ei] if side else cur
            with torch.cuda.stream(st):
                if side:
                    st.wait_event(fork)
                self._step_stack(ent, o, mu, nesterov, lr, coeffs, use_graph)
        if side:
            for st in self._streams[: len(ents)]:
                cur.wait_stream(st)
        self._pending_shard = None

    def _step_stack(self, ent, o, mu, nesterov, lr, coeffs, use_graph):
        r, c, plist = ent["r"], ent["c"], ent["plist"]
        for (p, _), mv in zip(plist, ent["mviews"]):
            st = self.state[p]
            cur = st.get("momentum_buffer")
            if cur is None or cur.data_ptr() != mv.data_ptr():
                if cur is not None:            # a buffer restored from a checkpoint: move it into the stack
                    mv.copy_(cur.view(mv.shape))
                st["momentum_buffer"] = mv
        if self._pending_shard is not None:
            t = self._pending_shard.get(f"mom_{r}x{c}")
            if t is not None:
                ent["mom"].copy_(t[: ent["total"]])
        # gradients the producing GEMM already wrote into their slot of the stack (see `grad_views`) need no copy
        pairs = [(gv, p.grad) for (p, _), gv in zip(plist, ent["gviews"]) if p.grad.data_ptr() != gv.data_ptr()]
        if pairs:
            torch._foreach_copy_([a for a, _ in pairs], [b for _, b in pairs])
        ent["sumsq"].zero_()
        o.muon_momentum(ent["grads"], ent["mom"], ent["stack"], ent["sumsq"], mu, nesterov, 1.0)
        o.stack_scale_by_inv_norm(ent["stack"], ent["sumsq"], ent["total"], r * c, 1e-7)
        key = tuple(coeffs)
        if use_graph:
            if ent.get("ns_key") != key:
                ent["ns"], ent["ns_key"] = GraphedNewtonSchulz(ent["stack"], coeffs), key
            u = ent["ns"]()
        else:
            u = newton_schulz_(ent["stack"], coeffs, self._work)
        alpha = -lr * max(1.0, r / c) ** 0.5
        slot = 0
        for p, nmat in plist:
            upd = u[slot:slot + nmat].view(p.shape)
            if p.dtype == torch.float32:
                sh = get_shadow_buffer(p, torch.bfloat16)
                if sh is None:
                    sh = torch.empty(p.shape, dtype=torch.bfloat16, device=p.device)
                o.axpy_bf16_to_f32(p, upd, sh, alpha)
                mark_modified(p)
                set_shadow(p, sh)
            else:
                p.add_(upd.to(p.dtype), alpha=alpha)
            slot += nmat

    def grad_views(self) -> dict:
        """``{id(param): fp32 view}`` of the stacked gradient buffers of the fused step. A backward that writes a
        matrix's gradient into its view (and makes that view ``p.grad``) saves the step's copy of all gradients into
        the stacks."""
        out = {}
        for group in self.param_groups:
            params = list(group["params"])
            if not params or not all(p.is_cuda and p.is_contiguous() and p.dim() >= 2 for p in params):
                continue
            for ent in self._slots(params):
                for (p, _), gv in zip(ent["plist"], ent["gviews"]):
                    out[id(p)] = gv
        return out

    # -- the same checkpoint interface as the distributed forms (parallel/muon_dist.py): per-shape momentum stacks
    def sharded_state(self) -> dict:
        out = {}
        for ents in self._stacks.values():
            for ent in ents:
                out[f"mom_{ent['r']}x{ent['c']}"] = ent["mom"].detach().clone()
        return out

    def sharded_rows(self) -> dict:
        return {f"mom_{e['r']}x{e['c']}": e["total"] for ents in self._stacks.values() for e in ents}

    def load_sharded_state(self, shard: dict) -> None:
        """Momentum stacks saved by any of the Muon forms (re-partitioned for one rank); applied at the next step."""
        self._pending_shard = dict(shard)

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            ps = [p for p in group["params"] if p.grad is not None]
            if not ps:
                continue
            if all(p.is_cuda and p.is_contiguous() for p in ps):
                self._step_fused(group)
            else:
                self._step_torch(group)
        return loss
