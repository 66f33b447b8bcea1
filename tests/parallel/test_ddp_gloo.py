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
