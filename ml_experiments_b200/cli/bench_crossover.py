"""Forward / backward time and peak memory of the long-sequence operators against full softmax attention over a sweep
of sequence lengths: where does each operator cross over (role of the reference's ``scripts/bench_crossover.py`` and
``scripts/benchmark_scatter_attention.py``, which only print).

    python -m ml_experiments_b200.cli.bench_crossover --lengths 1024,4096,16384 --width 256 --heads 4 --ops attention,tele,conv,lowrank
"""
from __future__ import annotations

import argparse
import json
import time

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..models.ripple_ops import AdaptiveLocalConv, LowRankAttention, TelephoneAttentionND
from ..models.scatter import AdaptiveConvND, HierarchicalLocalAttention, LocalAttentionND, LowRankAttentionND, SGSBAttention


class FullAttention(nn.Module):
    def __init__(self, width, heads):
        super().__init__()
        self.h, self.qkv, self.out = heads, nn.Linear(width, 3 * width), nn.Linear(width, width)

    def forward(self, x):
        B, L, C = x.shape
        q, k, v = self.qkv(x).view(B, L, 3, self.h, C // self.h).permute(2, 0, 3, 1, 4)
        return self.out(F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(B, L, C))


def make_op(name: str, width: int, heads: int, L: int, checkpoint: bool = False):
    if name == "attention":
        return FullAttention(width, heads)
    if name == "tele":
        return TelephoneAttentionND(width, ndim=1, num_heads=heads, max_seq_len=L)
    if name == "conv":
        return AdaptiveLocalConv(width, num_heads=heads)
    if name == "lowrank":
        return LowRankAttention(width, num_heads=heads)
    if name == "scatter":
        return AdaptiveConvND(width, ndim=1, num_channels=heads)
    if name == "gather":         # soft-window local attention (optionally with gradient checkpointing of its chunks)
        return LocalAttentionND(width, kernel_size=17, ndim=1, num_channels=heads, checkpoint=checkpoint)
    if name == "hier":
        return HierarchicalLocalAttention(width, window_size=17, num_channels=heads)
    if name == "sgsb":           # local attention gated by a low-rank global summary
        return SGSBAttention(width, kernel_size=17, num_channels=heads)
    if name == "lowrank_nd":     # SIREN-downsampled full attention, upsampled back
        return LowRankAttentionND(width, window_size=17, ndim=1, num_channels=heads)
    raise ValueError(name)


def measure(op, x, iters: int, warmup: int, amp: bool):
    cuda = x.is_cuda
    out_of = lambda y: y[0] if isinstance(y, tuple) else y

    def fwd():
        with torch.autocast(x.device.type, dtype=torch.bfloat16, enabled=amp):
            return out_of(op(x))

    def timed(fn):
        for _ in range(warmup):
            fn()
        if cuda:
            torch.cuda.synchronize()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(iters):
                fn()
            e.record()
            torch.cuda.synchronize()
            return s.elapsed_time(e) / iters
        t0 = time.perf_counter()
        for _ in range(iters):
            fn()
        return (time.perf_counter() - t0) * 1e3 / iters

    with torch.no_grad():
        f_ms = timed(fwd)
    if cuda:
        torch.cuda.reset_peak_memory_stats()
    fb_ms = timed(lambda: fwd().float().square().mean().backward())
    peak = torch.cuda.max_memory_allocated() / 2 ** 20 if cuda else float("nan")
    return f_ms, fb_ms - f_ms, peak


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--lengths", default="1024,4096,16384")
    ap.add_argument("--ops", default="attention,tele,conv,lowrank,scatter,gather,hier,sgsb,lowrank_nd")
    ap.add_argument("--checkpoint", action="store_true", help="gradient checkpointing inside the local-attention operator")
    ap.add_argument("--width", type=int, default=256)
    ap.add_argument("--heads", type=int, default=4)
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--amp", action="store_true")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args(argv)
    rows = []
    for L in (int(v) for v in a.lengths.split(",")):
        x = torch.randn(a.batch, L, a.width, device=a.device, requires_grad=True)
        for name in a.ops.split(","):
            torch.manual_seed(0)
            op = make_op(name, a.width, a.heads, L, a.checkpoint).to(a.device)
            try:
                f, b, mem = measure(op, x, a.iters, a.warmup, a.amp)
                row = dict(op=name, seq_len=L, fwd_ms=round(f, 3), bwd_ms=round(b, 3), peak_mib=round(mem, 1))
            except torch.OutOfMemoryError:
                row = dict(op=name, seq_len=L, error="out of memory")
                torch.cuda.empty_cache()
            rows.append(row)
            print(json.dumps(row), flush=True)
    return rows


if __name__ == "__main__":
    main()
