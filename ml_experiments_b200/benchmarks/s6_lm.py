"""S6 selective-scan byte LM: 24 layers, d_model 1024, expand 2, state 16, chunk 64, vocab 256,
sequence 4096, batch 8 per rank, bf16, AdamW, DDP with bucketed all-reduce overlapped with backward.

    python -m ml_experiments_b200.benchmarks.s6_lm [--layers 24 --d-model 1024 --batch 8 --seq 4096 --steps 5]
    torchrun --nproc-per-node N -m ml_experiments_b200.benchmarks.s6_lm ...
"""
from __future__ import annotations

import argparse

import torch

from ..models.s6 import S6Config, S6LM
from .common import emit, init_dist, timed_steps


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=24)
    ap.add_argument("--d-model", type=int, default=1024)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--breakdown", type=int, default=0, metavar="ROWS",
                    help="instead of timing, profile one step with torch.profiler and print the ROWS kernels with the most device time")
    a = ap.parse_args()
    rank, world, local = init_dist()
    dev = torch.device("cuda", local)
    torch.manual_seed(0)
    model = S6LM(S6Config(d_model=a.d_model, n_layers=a.layers)).to(dev).bfloat16()
    params = list(model.parameters())
    net = model
    ddp = None
    if world > 1:
        from ..parallel.ddp import DistributedDataParallel
        from ..parallel.symm import SymmWorld

        try:
            sw = SymmWorld.create(rank, world, dev)
        except Exception:
            sw = None
        net = ddp = DistributedDataParallel(model, world=sw)
    opt = torch.optim.AdamW(params, lr=3e-4, weight_decay=0.1, fused=True)
    if ddp is not None:
        ddp.wrap_optimizer(opt)
    g = torch.Generator().manual_seed(100 + rank)
    ids = torch.randint(0, 256, (a.batch, a.seq + 1), generator=g).to(dev)

    def step():
        loss = net(ids[:, :-1], ids[:, 1:])
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)

    if a.breakdown:
        from torch.profiler import ProfilerActivity, profile

        for _ in range(a.warmup):
            step()
        torch.cuda.synchronize()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            step()
            torch.cuda.synchronize()
        if rank == 0:
            ev = [e for e in prof.key_averages() if e.device_time_total > 0]
            total = sum(e.device_time_total for e in ev)
            print(f"device time per step: {total / 1e3:.2f} ms over {sum(e.count for e in ev)} launches")
            for e in sorted(ev, key=lambda e: -e.device_time_total)[: a.breakdown]:
                print(f"{100 * e.device_time_total / total:5.1f} %  {e.device_time_total / 1e3:8.3f} ms  {e.count:4d} x {e.device_time_total / e.count:9.1f} us  {e.key[:100]}")
        return
    ms = timed_steps(step, a.steps, a.warmup, world, dev)
    from ..ops.runtime import check_status

    check_status()
    emit(rank, metric="tokens/s S6 selective-scan LM", value=a.batch * a.seq * world / (ms / 1e3), unit="tokens/s",
         ms_per_step=ms, n_gpus=world, config=dict(layers=a.layers, d_model=a.d_model, batch_per_rank=a.batch, seq=a.seq,
                                                    comm="fused-p2p" if (ddp and ddp.symm_world) else ("nccl" if ddp else "none")),
         dtype="bf16", data="synthetic uniform bytes")


if __name__ == "__main__":
    main()
