"""Symmetric (peer-mapped) device buffers and epoch flags for the fused collective kernels.

``SymmWorld`` hands out buffers that every rank allocates at the same time and whose peer addresses are known on
every rank, plus one small int32 flag array per rank used by the kernels of ``csrc/comm`` for release / acquire
signalling. Allocation and handle exchange are delegated to ``torch.distributed._symmetric_memory`` (one process per
GPU); all data movement is done by this package's own kernels through the exchanged pointers.

``VirtualWorld`` builds the same objects for W *virtual* ranks inside one process on one GPU. It exists for tests of
the kernel protocol on a single device: the caller runs every rank's producer kernels before any consumer kernel, so
no kernel ever waits on something a later launch would set.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch
import torch.distributed as dist

MAX_WORLD = 16
NUM_CHANNELS = 16


@dataclass
class SymmBuffer:
    local: torch.Tensor            # this rank's buffer
    ptrs: list[int]                # address of every rank's buffer as mapped on this device
    handle: object = None          # keeps the symmetric-memory mapping alive
    mc_ptr: int = 0                # NVLink multicast (NVLS) address of the same buffer, 0 when the fabric offers none


@dataclass
class SymmWorld:
    rank: int
    world: int
    device: torch.device
    group: object = None
    flags: SymmBuffer | None = None
    _epochs: dict = field(default_factory=dict)
    _keep: list = field(default_factory=list)

    @classmethod
    def create(cls, rank: int, world: int, device, group=None) -> "SymmWorld":
        assert world <= MAX_WORLD, f"at most {MAX_WORLD} ranks"
        w = cls(rank=rank, world=world, device=torch.device(device), group=group)
        w.flags = w.alloc(NUM_CHANNELS * MAX_WORLD, torch.int32, zero=True)
        return w

    def alloc(self, numel: int, dtype: torch.dtype, zero: bool = False) -> SymmBuffer:
        import torch.distributed._symmetric_memory as symm_mem

        group = self.group if self.group is not None else dist.group.WORLD
        t = symm_mem.empty(int(numel), dtype=dtype, device=self.device)
        hdl = symm_mem.rendezvous(t, group)
        if zero:
            t.zero_()
            torch.cuda.synchronize(self.device)
            dist.barrier(group=group)
        try:
            mc = int(getattr(hdl, "multicast_ptr", 0) or 0)
        except Exception:
            mc = 0
        buf = SymmBuffer(local=t, ptrs=[int(p) for p in hdl.buffer_ptrs], handle=hdl, mc_ptr=mc)
        self._keep.append(buf)
        return buf

    def next_epoch(self, channel: int, n: int = 1) -> int:
        """Monotonic epoch counter of a channel (identical on every rank because every rank calls it equally often)."""
        e = self._epochs.get(channel, 0) + n
        self._epochs[channel] = e
        return e


class VirtualWorld:
    """W virtual ranks on one device: ``worlds[r]`` behaves like rank r's :class:`SymmWorld`."""

    def __init__(self, world: int, device="cuda"):
        self.world = world
        self.device = torch.device(device)
        self.worlds = [SymmWorld(rank=r, world=world, device=self.device) for r in range(world)]
        flags = self.alloc(NUM_CHANNELS * MAX_WORLD, torch.int32, zero=True)
        for w, f in zip(self.worlds, flags):
            w.flags = f

    def alloc(self, numel: int, dtype: torch.dtype, zero: bool = False) -> list[SymmBuffer]:
        ts = [(torch.zeros if zero else torch.empty)(int(numel), dtype=dtype, device=self.device) for _ in range(self.world)]
        ptrs = [t.data_ptr() for t in ts]
        return [SymmBuffer(local=t, ptrs=list(ptrs)) for t in ts]

    def allocator(self, rank: int):
        """Per-rank allocation callable: the k-th call of every rank returns that rank's piece of the k-th buffer."""
        if not hasattr(self, "_pool"):
            self._pool, self._count = [], [0] * self.world

        def alloc(numel: int, dtype: torch.dtype, zero: bool = False) -> SymmBuffer:
            k = self._count[rank]
            self._count[rank] += 1
            if k == len(self._pool):
                self._pool.append(self.alloc(numel, dtype, zero))
            buf = self._pool[k][rank]
            assert buf.local.numel() == int(numel) and buf.local.dtype == dtype, "ranks must allocate in the same order"
            return buf

        return alloc
