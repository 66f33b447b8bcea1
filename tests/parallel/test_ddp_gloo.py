"""DDP wrapper with two CPU ranks (gloo): bucketed averaging equals a single-process run on the concatenated batch."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from ml_experiments_b200.parallel.ddp import DistributedDataParallel as DDP

        torch.manual_seed(rank)  # different init per rank: the wrapper must broadcast rank 0's
        net = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.Tanh(), torch.nn.Linear(16, 4))
        ddp = DDP(net, bucket_cap_mb=0.0005)  # tiny cap -> several buckets
        assert len(ddp.buckets) >= 2
        opt = ddp.wrap_optimizer(torch.optim.SGD(net.parameters(), lr=0.1))
        g = torch.Generator().manual_seed(123)
        x = torch.randn(world * 4, 8, generator=g)
        y = torch.randn(world * 4, 4, generator=g)
        for step in range(3):
            xs, ys = x[rank * 4:(rank + 1) * 4], y[rank * 4:(rank + 1) * 4]
            if step == 1:  # gradient accumulation: first micro-batch without synchronisation
                with ddp.no_sync():
                    (torch.nn.functional.mse_loss(ddp(xs), ys) * 0.5).backward()
                (torch.nn.functional.mse_loss(ddp(xs), ys) * 0.5).backward()
            else:
                torch.nn.functional.mse_loss(ddp(xs), ys).backward()
            opt.step()
            opt.zero_grad(set_to_none=True)
        flat = torch.cat([p.detach().reshape(-1) for p in net.parameters()])
        if rank == 0:
            torch.save(flat, out)
        gathered = [torch.zeros_like(flat) for _ in range(world)]
        dist.all_gather(gathered, flat)
        assert all(torch.allclose(gathered[0], t, atol=1e-6) for t in gathered)
    finally:
        dist.destroy_process_group()


def test_ddp_matches_single_process(tmp_path):
    world = 2
    out = str(tmp_path / "p.pt")
    mp.spawn(_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    got = torch.load(out)
    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.Tanh(), torch.nn.Linear(16, 4))
    opt = torch.optim.SGD(net.parameters(), lr=0.1)
    g = torch.Generator().manual_seed(123)
    x = torch.randn(world * 4, 8, generator=g)
    y = torch.randn(world * 4, 4, generator=g)
    for _ in range(3):
        loss = sum(torch.nn.functional.mse_loss(net(x[r * 4:(r + 1) * 4]), y[r * 4:(r + 1) * 4]) for r in range(world)) / world
        loss.backward()
        opt.step()
        opt.zero_grad()
    want = torch.cat([p.detach().reshape(-1) for p in net.parameters()])
    assert torch.allclose(got, want, atol=1e-5), (got - want).abs().max()


class _LateScale(torch.nn.Module):
    """The parameter listed LAST (so it sits in bucket 0) is used by the first layer: its gradient arrives last and
    every other bucket is complete before bucket 0."""

    def __init__(self):
        super().__init__()
        self.a = torch.nn.Linear(8, 16)
        self.b = torch.nn.Linear(16, 4)
        self.late = torch.nn.ParameterList([torch.nn.Parameter(torch.ones(8))])   # a child registered last: listed last

    def forward(self, x):
        return self.b(torch.tanh(self.a(x * self.late[0])))


def _worker_out_of_order(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from ml_experiments_b200.parallel.ddp import DistributedDataParallel as DDP

        torch.manual_seed(0)
        net = _LateScale()
        ddp = DDP(net, bucket_cap_mb=0.00001)          # one bucket per parameter
        assert len(ddp.buckets) == 5 and ddp.buckets[0].params[0] is net.late[0]
        filled = []
        orig = ddp._launch
        ddp._launch = lambda bi: (filled.append([b.pending for b in ddp.buckets]), orig(bi))[1]
        g = torch.Generator().manual_seed(5)
        x, y = torch.randn(world * 4, 8, generator=g), torch.randn(world * 4, 4, generator=g)
        torch.nn.functional.mse_loss(ddp(x[rank * 4:(rank + 1) * 4]), y[rank * 4:(rank + 1) * 4]).backward()
        # bucket 0 was the last to fill, yet the launches went out as 0, 1, 2, ... (all at once, after it filled)
        assert ddp.launch_order == list(range(5)), ddp.launch_order
        assert filled[0] == [0] * 5, filled
        ddp.finish()
        if rank == 0:
            torch.save(torch.cat([p.grad.reshape(-1) for p in net.parameters()]), out)
    finally:
        dist.destroy_process_group()


def test_buckets_launch_in_index_order_when_they_fill_out_of_order(tmp_path):
    world = 2
    out = str(tmp_path / "g.pt")
    mp.spawn(_worker_out_of_order, args=(world, _free_port(), out), nprocs=world, join=True)
    got = torch.load(out)
    torch.manual_seed(0)
    net = _LateScale()
    g = torch.Generator().manual_seed(5)
    x, y = torch.randn(world * 4, 8, generator=g), torch.randn(world * 4, 4, generator=g)
    loss = sum(torch.nn.functional.mse_loss(net(x[r * 4:(r + 1) * 4]), y[r * 4:(r + 1) * 4]) for r in range(world)) / world
    loss.backward()
    want = torch.cat([p.grad.reshape(-1) for p in net.parameters()])
    assert torch.allclose(got, want, atol=1e-6)
