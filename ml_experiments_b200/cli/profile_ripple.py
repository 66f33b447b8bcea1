"""Per-operator time of a Ripple model: every sub-module of every block is wrapped in a CUDA-event region and a table
of forward times by operator (telephone / conv / low-rank / attention / Jacobi / norms / MLP) is printed, together with
the whole step's forward / backward split (role of the reference's ``scripts/profile_ripple.py:38-486``, which
monkey-patches each sub-op by hand).

    python -m ml_experiments_b200.cli.profile_ripple --seq-len 16384 --width 256 --layers 8 --batch 8 --order tele,conv,lowrank
"""
from __future__ import annotations

import argparse
import json
from collections import defaultdict

import torch
import torch.nn.functional as F

from ..models.ripple import RippleAttention, RippleClassifier
from ..runtime.tracing import OpTimer, instrument_module


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--seq-len", type=int, default=4096)
    ap.add_argument("--width", type=int, default=256)
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--heads", type=int, default=4)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--order", default="tele,conv,lowrank")
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--amp", action="store_true")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args(argv)
    dev = torch.device(a.device)
    torch.manual_seed(0)
    model = RippleClassifier(width=a.width, n_layers=a.layers, n_classes=2, seq_len=a.seq_len, num_heads=a.heads, order=a.order,
                             max_seq_len=a.seq_len).to(dev)
    x, y = torch.rand(a.batch, a.seq_len, device=dev), torch.randint(0, 2, (a.batch,), device=dev)
    timer = OpTimer(dev)
    # operator level: the direct children of each RippleAttention, plus the MLP and norm of each block
    ops = {id(m) for mod in model.modules() if isinstance(mod, RippleAttention) for m in mod.children()}
    undo = instrument_module(model, timer, match=lambda name, mod: id(mod) in ops or name.endswith((".mlp", ".norm")) or name in ("embed", "head"))

    def step():
        with torch.autocast(dev.type, dtype=torch.bfloat16, enabled=a.amp):
            with timer.region("__forward__"):
                loss = F.cross_entropy(model(x).float(), y)
        with timer.region("__backward__"):
            loss.backward()
        model.zero_grad(set_to_none=True)

    step()                       # warm-up (allocations, lazy initialisation)
    timer.totals_ms()
    timer._wall.clear()
    timer.calls.clear()
    for _ in range(a.iters):
        step()
    totals = timer.totals_ms()
    undo()
    by_kind = defaultdict(float)
    for name, ms in totals.items():
        kind = name if name.startswith("__") else name.split(".")[-1] if not name.split(".")[-1].isdigit() else name.split(".")[-2]
        by_kind[kind] += ms / a.iters
    fwd = by_kind.pop("__forward__", 0.0)
    bwd = by_kind.pop("__backward__", 0.0)
    print(f"forward {fwd:.2f} ms, backward {bwd:.2f} ms per step (batch {a.batch}, {a.seq_len} tokens, {a.layers} layers)")
    for kind, ms in sorted(by_kind.items(), key=lambda kv: -kv[1]):
        print(f"  {kind:<14s} {ms:9.3f} ms  {100 * ms / max(fwd, 1e-9):5.1f}% of forward")
    out = dict(forward_ms=fwd, backward_ms=bwd, forward_by_operator=dict(by_kind))
    print(json.dumps(out))
    return out


if __name__ == "__main__":
    main()
