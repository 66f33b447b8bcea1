"""Data-parallel wrapper with bucketed gradient averaging overlapped with the backward pass.

API of ``torch.nn.parallel.DistributedDataParallel`` as the reference's older trainers use it
(modded-nanogpt/records/track_1_short/2024-10-10_Muon/train_gpt2.py:383,497: ``DDP(model)``, ``model.no_sync()``) and the
hook-driven overlap of the reference's ``DistAdam`` (modded-nanogpt/train_gpt_medium.py:743-767).

Parameters are broadcast from rank 0 at construction. Gradients are packed into buckets (filled in reverse parameter
order, the order in which backward produces them). A ``post_accumulate_grad`` hook copies each gradient into its
bucket; when a bucket is complete its all-reduce starts on a side stream while backward continues:

* CUDA with symmetric memory: the bucket *is* a peer-mapped buffer and the mean all-reduce is this package's
  two-shot peer-memory kernel (sum over peers, 1/W scale and dtype handling fused), or with ``use_nvls`` its
  NVSwitch-multicast variant (``multimem.ld_reduce`` / ``multimem.st``: the sum is formed inside the switch);
* otherwise (CPU / gloo, or no peer access): ``dist.all_reduce`` on the flat bucket.

``finish()`` (called automatically by ``step`` hooks of optimizers created through :meth:`wrap_optimizer`, or by hand)
waits for all buckets and re-points every ``p.grad`` at its averaged bucket view.
"""
from __future__ import annotations

import contextlib
import os

import torch
import torch.distributed as dist
import torch.nn as nn

CH_IN, CH_OUT = 6, 7


class _Bucket:
    def __init__(self, params, dtype, device, world=None):
        self.params = params
        self.dtype = dtype
        vec = 8 if dtype == torch.bfloat16 else 4
        W = world.world if world is not None else 1
        offs, n = [], 0
        for p in params:
            offs.append(n)
            n += (p.numel() + vec - 1) // vec * vec
        self.numel = (n + vec * W - 1) // (vec * W) * (vec * W)
        self.symm = world.alloc(self.numel, dtype) if world is not None else None
        self.flat = self.symm.local if self.symm is not None else torch.zeros(self.numel, dtype=dtype, device=device)
        self.flat.zero_()
        self.views = [self.flat[o:o + p.numel()].view(p.shape) for o, p in zip(offs, params)]
        self.pending = 0
        self.work = None
        self.event = None


class DistributedDataParallel(nn.Module):
    def __init__(self, module: nn.Module, world=None, bucket_cap_mb: float = 64.0, process_group=None,
                 broadcast_parameters: bool = True, use_nvls: bool | None = None):
        super().__init__()
        # in-switch reduction (multimem) instead of peer loads; off unless asked for (argument or B200_NVLS=1)
        self.use_nvls = (os.environ.get("B200_NVLS", "0") == "1") if use_nvls is None else use_nvls
        self.module = module
        self.group = process_group
        self.world_size = dist.get_world_size(process_group) if dist.is_initialized() else 1
        self.symm_world = world
        self.require_sync = True
        self._step = 0
        params = [p for p in module.parameters() if p.requires_grad]
        self.device = params[0].device if params else torch.device("cpu")
        if broadcast_parameters and self.world_size > 1:
            for p in module.parameters():
                dist.broadcast(p.detach(), 0, group=process_group)
        cap = int(bucket_cap_mb * 1024 * 1024)
        self.buckets: list[_Bucket] = []
        cur, cur_bytes, cur_dtype = [], 0, None
        for p in reversed(params):
            gdtype = p.dtype
            if cur and (gdtype != cur_dtype or cur_bytes + p.numel() * p.element_size() > cap):
                self.buckets.append(_Bucket(cur, cur_dtype, self.device, world))
                cur, cur_bytes = [], 0
            cur.append(p)
            cur_dtype = gdtype
            cur_bytes += p.numel() * p.element_size()
        if cur:
            self.buckets.append(_Bucket(cur, cur_dtype, self.device, world))
        self._where = {}
        for bi, b in enumerate(self.buckets):
            for pi, p in enumerate(b.params):
                self._where[id(p)] = (bi, pi)
                p.register_post_accumulate_grad_hook(self._hook)
        self._comm_stream = torch.cuda.Stream(self.device) if self.device.type == "cuda" else None
        self._in_flight = False
        self._next_launch = 0
        self.launch_order: list[int] = []     # bucket indices in the order their all-reduce was enqueued (last backward)

    def forward(self, *args, **kwargs):
        return self.module(*args, **kwargs)

    @contextlib.contextmanager
    def no_sync(self):
        old, self.require_sync = self.require_sync, False
        try:
            yield
        finally:
            self.require_sync = old

    # ------------------------------------------------------------------------------------------
    def _hook(self, p: torch.Tensor):
        if not self.require_sync or self.world_size == 1:
            return
        bi, pi = self._where[id(p)]
        b = self.buckets[bi]
        if not self._in_flight:
            self._in_flight = True
            self._step += 1
            self._next_launch = 0
            for bb in self.buckets:
                bb.pending = len(bb.params)
        b.views[pi].copy_(p.grad)
        b.pending -= 1
        # Buckets are launched strictly in index order on every rank, whatever order they fill in (a parameter used by
        # every layer, listed late, gets its gradient last and would otherwise let a higher bucket go first): all
        # buckets share one pair of flag channels whose epoch grows with the bucket index, so an out-of-order launch
        # would let a peer's wait for bucket i be satisfied by bucket i+1's larger epoch.
        while self._next_launch < len(self.buckets) and self.buckets[self._next_launch].pending == 0:
            self._launch(self._next_launch)
            self._next_launch += 1

    def _launch(self, bi: int):
        b = self.buckets[bi]
        if bi == 0:
            self.launch_order = []
        self.launch_order.append(bi)
        if b.symm is not None:
            from ..ops.runtime import ops, status

            w = self.symm_world
            o = ops()
            epoch = (self._step - 1) * len(self.buckets) + bi + 1
            ready = torch.cuda.Event()
            ready.record()
            with torch.cuda.stream(self._comm_stream):
                self._comm_stream.wait_event(ready)
                o.comm_signal(w.flags.ptrs, w.rank, CH_IN, epoch, w.flags.local)
                code = 1 if b.dtype == torch.bfloat16 else 0
                if self.use_nvls and b.symm.mc_ptr:
                    o.allreduce_mean_multimem(b.symm.mc_ptr, w.world, w.rank, b.numel, code, w.flags.local, w.flags.ptrs, CH_IN, epoch,
                                              status(self.device))
                else:
                    o.allreduce_mean(b.symm.ptrs, w.rank, b.numel, code, w.flags.local, w.flags.ptrs, CH_IN, epoch, status(self.device))
                o.comm_wait(w.flags.local, w.world, CH_OUT, epoch, status(self.device))
                b.event = torch.cuda.Event()
                b.event.record()
        else:
            b.work = dist.all_reduce(b.flat, op=dist.ReduceOp.SUM, group=self.group, async_op=True)

    def finish(self):
        """Waits for every bucket of the current backward and installs the averaged gradients."""
        if not self._in_flight:
            return
        for b in self.buckets:
            if b.pending != 0:
                raise RuntimeError("DistributedDataParallel.finish(): a parameter of a bucket produced no gradient")
            if b.event is not None:
                torch.cuda.current_stream(self.device).wait_event(b.event)
                b.event = None
            if b.work is not None:
                b.work.wait()
                b.work = None
                b.flat.div_(self.world_size)
            for p, v in zip(b.params, b.views):
                p.grad = v
        self._in_flight = False

    def wrap_optimizer(self, opt: torch.optim.Optimizer) -> torch.optim.Optimizer:
        """Makes ``opt.step()`` wait for the gradient averaging first."""
        opt.register_step_pre_hook(lambda *_: self.finish())
        return opt

    def state_dict(self, *a, **k):
        return self.module.state_dict(*a, **k)

    def load_state_dict(self, *a, **k):
        return self.module.load_state_dict(*a, **k)
