"""S6 selective-scan byte LM: 24 layers, d_model 1024, expand 2, state 16, chunk 64, vocab 256,
sequence 4096, batch 8 per rank, bf16, AdamW, DDP with bucketed all-reduce overlapped with backward.

    python -m ml_experiments_b200.benchmarks.s6_lm [--layers 24 --d-model 1024 --batch 8 --seq 4096 --steps 5]
    torchrun --nproc-per-node N -m ml_experiments_b200.benchmarks.s6_lm ...
    python -m ml_experiments_b200.benchmarks.s6_lm --impl reference

``--impl reference`` stacks the reference's own S6 mixer (``zoology.mixers.mamba.Mamba``,
zoology/zoology/mixers/mamba.py:21-198) into the same byte LM (embedding, pre-norm residual blocks, tied-free head) and
times the same step. That module imports the compiled extensions ``selective_scan_cuda`` and ``causal_conv1d`` at import
time; where they are not installed the arm prints ``{"impl": "reference", "unavailable": "<the exception>"}``.
"""
from __future__ import annotations

import argparse

import torch

from .common import emit, init_dist, reference_root, timed_steps, unavailable


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
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    a = ap.parse_args()
    rank, world, local = init_dist()
    dev = torch.device("cuda", local)
    torch.manual_seed(0)
    if a.impl == "reference":
        try:
            _run_reference(a, rank, world, dev)
        except BaseException as e:      # the reference module aborts its import with ``assert 0`` when an extension is missing
            if isinstance(e, (KeyboardInterrupt, SystemExit)):
                raise
            import traceback

            traceback.print_exc()
            unavailable(rank, e)
        return
    from ..models.s6 import S6Config, S6LM

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
    from ..optim import FusedAdam          # this package's Adam kernel (decoupled weight decay), not a library optimizer

    opt = FusedAdam(params, lr=3e-4, weight_decay=0.1)
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
    emit(rank, impl="ours", metric="tokens/s S6 selective-scan LM", value=a.batch * a.seq * world / (ms / 1e3), unit="tokens/s",
         ms_per_step=ms, n_gpus=world, config=dict(layers=a.layers, d_model=a.d_model, batch_per_rank=a.batch, seq=a.seq,
                                                    comm="fused-p2p" if (ddp and ddp.symm_world) else ("nccl" if ddp else "none")),
         dtype="bf16", data="synthetic uniform bytes")


def _run_reference(a, rank, world, dev):
    import sys

    root = reference_root()
    if root is None:
        raise FileNotFoundError("no copy of the reference packages (baseline/_ref/zoology)")
    sys.path.insert(0, root)
    import importlib

    try:
        Mamba = importlib.import_module("zoology.mixers.mamba").Mamba
    except AssertionError as e:
        missing = []
        for mod in ("causal_conv1d", "selective_scan_cuda"):
            try:
                importlib.import_module(mod)
            except ImportError as ie:
                missing.append(f"{type(ie).__name__}: {ie}")
        raise ImportError("zoology.mixers.mamba cannot be imported: " + "; ".join(missing or [repr(e)])) from e
    nn = torch.nn

    class Block(nn.Module):
        def __init__(self, d, i):
            super().__init__()
            self.norm = nn.RMSNorm(d)
            self.mixer = Mamba(d_model=d, d_state=16, expand=2, layer_idx=i)

        def forward(self, x):
            return x + self.mixer(self.norm(x))

    class LM(nn.Module):
        def __init__(self, d, n, vocab=256):
            super().__init__()
            self.embed = nn.Embedding(vocab, d)
            self.blocks = nn.ModuleList(Block(d, i) for i in range(n))
            self.norm = nn.RMSNorm(d)
            self.head = nn.Linear(d, vocab, bias=False)

        def forward(self, ids, targets):
            x = self.embed(ids)
            for b in self.blocks:
                x = b(x)
            return torch.nn.functional.cross_entropy(self.head(self.norm(x)).float().flatten(0, 1), targets.flatten())

    model = LM(a.d_model, a.layers).to(dev).bfloat16()
    net = torch.nn.parallel.DistributedDataParallel(model, device_ids=[dev.index]) if world > 1 else model
    opt = torch.optim.AdamW(model.parameters(), lr=3e-4, weight_decay=0.1, fused=True)
    g = torch.Generator().manual_seed(100 + rank)
    ids = torch.randint(0, 256, (a.batch, a.seq + 1), generator=g).to(dev)

    def step():
        net(ids[:, :-1], ids[:, 1:]).backward()
        opt.step()
        opt.zero_grad(set_to_none=True)

    ms = timed_steps(step, a.steps, a.warmup, world, dev)
    emit(rank, impl="reference", metric="tokens/s S6 selective-scan LM", value=a.batch * a.seq * world / (ms / 1e3), unit="tokens/s",
         ms_per_step=ms, n_gpus=world, config=dict(layers=a.layers, d_model=a.d_model, batch_per_rank=a.batch, seq=a.seq, comm="nccl"),
         dtype="bf16", data="synthetic uniform bytes")


if __name__ == "__main__":
    main()
