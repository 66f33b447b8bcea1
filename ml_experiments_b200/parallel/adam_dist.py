"""Adam with ZeRO-style sharded state whose reduce-scatter and all-gather are fused into the update kernel.

Counterpart of the reference's sharded Adam paths: ``DistAdam`` (modded-nanogpt/train_gpt_medium.py:715-833: gradient
reduce-scatter from backward hooks, update of the owned rows, ``all_gather_into_tensor`` of the parameters) and the
``sharded`` Adam entries of ``NorMuonAndAdam`` (modded-nanogpt/train_gpt.py:461-478,654-691). There the three phases
are two NCCL collectives around a compiled elementwise update; here they are ONE kernel per parameter segment
(``csrc/comm/comm.cu::adam_shard_kernel``): the owner of a slice sums the peers' gradients by NVLink loads, updates its
fp32 moments (which exist only on the owner: 1/W of the optimizer state per GPU) and stores the new parameters straight
into every rank's replica.

Layout: per dtype one symmetric *gradient* bucket and one symmetric *parameter* bucket; every ``nn.Parameter`` handed
to this class becomes a view into the parameter bucket, and :attr:`grad_views` offers the matching views of the
gradient bucket so that backward kernels can write gradients where the collective reads them (no packing copy).
Parameters with fewer than ``pack_below`` elements that share dtype and learning-rate group are packed into one
segment.
"""
from __future__ import annotations

import torch

from ..ops.runtime import ops, status
from ..utils.shadow import mark_modified

CH_ADAM, CH_ADAM_EARLY = 8, 10       # (inputs ready, outputs written) = (c, c + 1); the early pair serves segments launched
                                     # on a side stream during backward, whose order relative to the others is not fixed


def _pad(n: int, m: int) -> int:
    return (n + m - 1) // m * m


class _Segment:
    __slots__ = ("dtype", "code", "vec", "off", "numel", "per", "group", "params", "m", "v", "step", "early")


class ShardedAdam:
    """``groups``: ``[dict(params=[...], lr=...), ...]`` as for ``torch.optim.Adam``. ``world``: a
    :class:`~ml_experiments_b200.parallel.symm.SymmWorld` (or one rank of a ``VirtualWorld`` with ``alloc`` given)."""

    def __init__(self, groups, world, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0, alloc=None,
                 pack_below: int = 65536, max_blocks: int = 0):
        self.w = world
        self.betas, self.eps, self.weight_decay = betas, eps, weight_decay
        self.max_blocks = max_blocks
        alloc = alloc or world.alloc
        W = world.world
        self.param_groups = [dict(g) for g in groups]
        for g in self.param_groups:
            g["params"] = list(g["params"])
        # ---- segments
        self.segments: list[_Segment] = []
        sizes = {torch.float32: 0, torch.bfloat16: 0}
        for gi, g in enumerate(self.param_groups):
            small: dict = {}
            for p in g["params"]:
                assert p.dtype in sizes, f"ShardedAdam: fp32 or bf16 parameters, got {p.dtype}"
                if p.numel() < pack_below:
                    small.setdefault(p.dtype, []).append(p)
                else:
                    self.segments.append(self._segment(p.dtype, [p], gi, W, sizes))
            for dtype, plist in small.items():
                self.segments.append(self._segment(dtype, plist, gi, W, sizes))
        # ---- symmetric buckets; parameters and gradient slots become views
        self.pbuf, self.gbuf = {}, {}
        for dtype, n in sizes.items():
            if n:
                self.pbuf[dtype] = alloc(n, dtype)
                self.gbuf[dtype] = alloc(n, dtype)
                self.pbuf[dtype].local.zero_()
                self.gbuf[dtype].local.zero_()
        self.grad_views: dict[int, torch.Tensor] = {}
        dev = world.flags.local.device
        for s in self.segments:
            off = s.off
            vec = s.vec
            with torch.no_grad():
                for p in s.params:
                    view = self.pbuf[s.dtype].local[off:off + p.numel()].view(p.shape)
                    view.copy_(p.detach())
                    p.data = view
                    self.grad_views[id(p)] = self.gbuf[s.dtype].local[off:off + p.numel()].view(p.shape)
                    off += _pad(p.numel(), vec)
            s.m = torch.zeros(s.per, dtype=torch.float32, device=dev)
            s.v = torch.zeros(s.per, dtype=torch.float32, device=dev)
            s.step = 0
            s.early = False
        self._epoch = {CH_ADAM: 0, CH_ADAM_EARLY: 0}
        self._pending: dict[int, int] = {}          # channel -> last epoch launched and not yet waited for
        self._launched: set[int] = set()
        self._side = None
        for p in self.all_params():
            mark_modified(p)

    @staticmethod
    def _segment(dtype, plist, gi, W, sizes) -> _Segment:
        s = _Segment()
        s.dtype, s.code, s.vec = dtype, (1 if dtype == torch.bfloat16 else 0), (8 if dtype == torch.bfloat16 else 4)
        s.params, s.group = plist, gi
        s.numel = _pad(sum(_pad(p.numel(), s.vec) for p in plist), s.vec * W)
        s.per = s.numel // W
        s.off = sizes[dtype]
        sizes[dtype] += s.numel
        return s

    # ------------------------------------------------------------------------------------------
    def all_params(self):
        return [p for s in self.segments for p in s.params]

    def segment_of(self, p) -> int:
        for i, s in enumerate(self.segments):
            if any(q is p for q in s.params):
                return i
        raise KeyError("parameter is not managed by this optimizer")

    def _stage_grads(self, s: _Segment) -> None:
        """Gradients that were not written into their bucket view by the producer are copied there now."""
        pairs = [(self.grad_views[id(p)], p.grad) for p in s.params
                 if p.grad is not None and p.grad.data_ptr() != self.grad_views[id(p)].data_ptr()]
        if pairs:
            torch._foreach_copy_([a for a, _ in pairs], [b if b.dtype == a.dtype else b.to(a.dtype) for a, b in pairs])

    @torch.no_grad()
    def publish(self, index: int, early: bool = False) -> None:
        """First half of :meth:`launch`: gradients of the segment are in place, tell every peer."""
        s = self.segments[index]
        w = self.w
        self._stage_grads(s)
        ch = CH_ADAM_EARLY if early else CH_ADAM
        self._epoch[ch] += 1
        ops().comm_signal(w.flags.ptrs, w.rank, ch, self._epoch[ch], w.flags.local)
        s.early = early

    @torch.no_grad()
    def reduce(self, index: int) -> None:
        """Second half of :meth:`launch`: the fused kernel (waits for every rank's :meth:`publish` of the segment)."""
        s = self.segments[index]
        w = self.w
        ch = CH_ADAM_EARLY if s.early else CH_ADAM
        e = self._epoch[ch]
        g = self.param_groups[s.group]
        b1, b2 = g.get("betas", self.betas)
        s.step += 1
        lo = s.off + w.rank * s.per
        ops().adam_shard(self.gbuf[s.dtype].ptrs, self.pbuf[s.dtype].ptrs, w.rank, lo, lo + s.per, s.code, s.m, s.v,
                         float(g["lr"]), b1, b2, g.get("eps", self.eps), g.get("weight_decay", self.weight_decay),
                         1 - b1 ** s.step, 1 - b2 ** s.step, w.flags.local, w.flags.ptrs, ch, e,
                         status(w.flags.local.device), self.max_blocks)
        self._pending[ch] = e
        self._launched.add(index)

    def launch(self, index: int, early: bool = False) -> None:
        """Enqueues the fused reduce-scatter + Adam + all-gather of one segment on the current stream. Segments that
        share a channel pair (all ``early`` ones; all others) must be launched in the same order on every rank."""
        self.publish(index, early)
        self.reduce(index)

    @torch.no_grad()
    def step(self, closure=None) -> None:
        """Launches every segment that was not launched early in this step, then waits (on the device) until every
        rank's slices have arrived, so that the next forward reads complete parameters."""
        for i, s in enumerate(self.segments):
            if i not in self._launched:
                self.launch(i)
        self.finish()

    @torch.no_grad()
    def finish(self) -> None:
        w = self.w
        o = ops()
        st = status(w.flags.local.device)
        for ch, e in self._pending.items():
            o.comm_wait(w.flags.local, w.world, ch + 1, e, st)
        self._pending.clear()
        self._launched.clear()
        for p in self.all_params():
            mark_modified(p)          # low-precision copies held by the forward (fp8 head) are stale now
            p.grad = None

    def zero_grad(self, set_to_none: bool = True) -> None:
        for p in self.all_params():
            p.grad = None

    # ------------------------------------------------------------------------------------------ checkpoints
    def state_dict(self) -> dict:
        """Replicated part only (step counters, hyper-parameters); the moments are per-rank: :meth:`sharded_state`."""
        return {"steps": [s.step for s in self.segments],
                "param_groups": [{k: v for k, v in g.items() if k != "params"} for g in self.param_groups]}

    def load_state_dict(self, sd: dict) -> None:
        for s, n in zip(self.segments, sd.get("steps", [])):
            s.step = int(n)
        for g, saved in zip(self.param_groups, sd.get("param_groups", [])):
            g.update({k: v for k, v in saved.items() if k != "params"})

    def sharded_state(self) -> dict:
        out = {}
        for i, s in enumerate(self.segments):
            out[f"adam_m_{i}"], out[f"adam_v_{i}"] = s.m.detach().clone(), s.v.detach().clone()
        return out

    def sharded_rows(self) -> dict:
        return {f"adam_{k}_{i}": s.numel for i, s in enumerate(self.segments) for k in ("m", "v")}

    def load_sharded_state(self, shard: dict) -> None:
        for i, s in enumerate(self.segments):
            for name, dst in ((f"adam_m_{i}", s.m), (f"adam_v_{i}", s.v)):
                t = shard.get(name)
                if t is None:
                    continue
                n = min(t.numel(), dst.numel())
                dst.zero_()
                dst[:n].copy_(t.reshape(-1)[:n])
