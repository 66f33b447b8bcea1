"""Scatter / hierarchical-attention classifier on long sequences: 128x128 uint8 images flattened
to 16 384 tokens, 8 layers, d_model 256, 4 heads, 2 classes, batch 32 per rank, bf16 autocast, AdamW.

    python -m ml_experiments_b200.benchmarks.ripple_classifier [--batch 32 --layers 8 --side 128]
    python -m ml_experiments_b200.benchmarks.ripple_classifier --impl reference

``--impl reference`` builds the reference's own ``RippleClassifier``
(src/heuristic_secrets/models/ripple_attention.py:504-602, with its Triton kernels: ``use_triton`` stays at its
default) from a plain copy of the reference package and runs it through the same step, data, optimizer and timing;
nothing of this package's models or kernels is on that path. If the reference's code cannot run on the box the arm
prints ``{"impl": "reference", "unavailable": "<the exception>"}``.
"""
from __future__ import annotations

import argparse

import torch
import torch.nn.functional as F

from .common import emit, init_dist, reference_root, timed_steps, unavailable


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--width", type=int, default=256)
    ap.add_argument("--heads", type=int, default=4)
    ap.add_argument("--side", type=int, default=128)
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--order", default="tele,conv,lowrank")
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    a = ap.parse_args()
    rank, world, local = init_dist()
    dev = torch.device("cuda", local)
    torch.manual_seed(0)
    L = a.side * a.side
    if a.impl == "reference":
        try:
            _run_reference(a, rank, world, dev, L)
        except Exception as e:
            import traceback

            traceback.print_exc()
            unavailable(rank, e)
        return
    from ..models.ripple import RippleClassifier

    model = RippleClassifier(width=a.width, n_layers=a.layers, n_classes=2, seq_len=L, num_heads=a.heads, order=a.order,
                             embed_2d=(a.side, a.side), max_seq_len=L).to(dev)
    net, ddp = model, None
    if world > 1:
        from ..parallel.ddp import DistributedDataParallel
        from ..parallel.symm import SymmWorld

        try:
            sw = SymmWorld.create(rank, world, dev)
        except Exception:
            sw = None
        net = ddp = DistributedDataParallel(model, world=sw)
    from ..optim import FusedAdam          # this package's Adam kernel (decoupled weight decay), not a library optimizer

    opt = FusedAdam(model.parameters(), lr=3e-4, weight_decay=0.01)
    if ddp is not None:
        ddp.wrap_optimizer(opt)
    g = torch.Generator().manual_seed(7 + rank)
    x = (torch.randint(0, 256, (a.batch, a.side, a.side), generator=g).float() / 255).to(dev)
    y = (torch.rand(a.batch, generator=g) < 0.5).long().to(dev)

    def step():
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = F.cross_entropy(net(x).float(), y, label_smoothing=0.1)
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)

    ms = timed_steps(step, a.steps, a.warmup, world, dev)
    from ..ops.runtime import check_status

    check_status()
    emit(rank, impl="ours", metric="images/s Ripple classifier (16 384 tokens)", value=a.batch * world / (ms / 1e3), unit="images/s",
         tokens_per_s=a.batch * L * world / (ms / 1e3), ms_per_step=ms, n_gpus=world,
         config=dict(layers=a.layers, width=a.width, heads=a.heads, tokens=L, batch_per_rank=a.batch, order=a.order),
         dtype="bf16 autocast", data="synthetic uniform pixels, Bernoulli labels")


def _run_reference(a, rank, world, dev, L):
    """The reference's classifier, plain ``torch`` DDP when there are several ranks, same step as :func:`main`."""
    import sys

    root = reference_root()
    if root is None:
        raise FileNotFoundError("no copy of the reference package (baseline/_ref/heuristic_secrets)")
    sys.path.insert(0, root)
    from heuristic_secrets.models.ripple_attention import RippleClassifier as RefClassifier

    model = RefClassifier(width=a.width, n_layers=a.layers, n_classes=2, seq_len=L, num_heads=a.heads, order=a.order,
                          embed_2d=(a.side, a.side), max_seq_len=L).to(dev)
    net = torch.nn.parallel.DistributedDataParallel(model, device_ids=[dev.index]) if world > 1 else model
    opt = torch.optim.AdamW(model.parameters(), lr=3e-4, weight_decay=0.01, fused=True)
    g = torch.Generator().manual_seed(7 + rank)
    x = (torch.randint(0, 256, (a.batch, a.side, a.side), generator=g).float() / 255).to(dev)
    y = (torch.rand(a.batch, generator=g) < 0.5).long().to(dev)

    def step():
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = F.cross_entropy(net(x).float(), y, label_smoothing=0.1)
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)

    ms = timed_steps(step, a.steps, a.warmup, world, dev)
    emit(rank, impl="reference", metric="images/s Ripple classifier (16 384 tokens)", value=a.batch * world / (ms / 1e3),
         unit="images/s", tokens_per_s=a.batch * L * world / (ms / 1e3), ms_per_step=ms, n_gpus=world,
         config=dict(layers=a.layers, width=a.width, heads=a.heads, tokens=L, batch_per_rank=a.batch, order=a.order),
         dtype="bf16 autocast", data="synthetic uniform pixels, Bernoulli labels")


if __name__ == "__main__":
    main()
