"""Wall-clock micro-profiles of the sequence-mixing operators (role of
zoology/analysis/paper/based_paper/based_wall_clock.py:26-60, which times Mamba-2's chunk scan at ``chunk_size=64``,
Mamba-1's selective scan at ``dstate=16``, flash attention, Based and an FFT convolution against sequence length).

Each operator is this package's own implementation, run on synthetic bf16 inputs of the reference's shapes
(``d_model = 2 * heads * head_dim`` for the Mamba operators), timed with CUDA events on the launching stream after
warm-up (host clock on a CPU); forward only, or forward + backward with ``backward=True``.

    python -m ml_experiments_b200.zoology.analysis.wall_clock --ops mamba1,mamba2,attention --seq-lens 1024,4096,16384
"""
from __future__ import annotations

import argparse
import json
import time

import torch
import torch.nn.functional as F

OPERATORS = ("mamba1", "mamba2", "attention", "gla", "long_conv")


def _inputs(op: str, batch: int, seq_len: int, heads: int, head_dim: int, dstate: int, device, dtype):
    g = torch.Generator(device=device).manual_seed(0)
    r = lambda *s, dt=dtype: torch.randn(*s, device=device, dtype=dt, generator=g)
    if op == "mamba1":
        from ...ops.selective_scan import selective_scan
        d = 2 * heads * head_dim
        u, z = r(batch, seq_len, d).requires_grad_(), r(batch, seq_len, d).requires_grad_()
        delta = r(batch, seq_len, d, dt=torch.float32).requires_grad_()
        A = (-torch.rand(d, 16, device=device, generator=g) - 0.1).requires_grad_()
        B, C = r(batch, seq_len, 16, dt=torch.float32).requires_grad_(), r(batch, seq_len, 16, dt=torch.float32).requires_grad_()
        D, bias = torch.ones(d, device=device, requires_grad=True), torch.zeros(d, device=device, requires_grad=True)
        return lambda: selective_scan(u, delta, A, B, C, D, z, delta_bias=bias, delta_softplus=True)
    if op == "mamba2":
        from ...ops.ssd_scan import ssd_chunk_scan
        h = 2 * heads
        x = r(batch, seq_len, h, head_dim).requires_grad_()
        B, C = r(batch, seq_len, h, dstate).requires_grad_(), r(batch, seq_len, h, dstate).requires_grad_()
        log_alpha = (-F.softplus(r(batch, seq_len, h, dt=torch.float32))).requires_grad_()
        gamma = torch.rand(batch, seq_len, h, device=device, generator=g).requires_grad_()
        return lambda: ssd_chunk_scan(x, B, C, log_alpha, gamma, chunk=64)
    if op == "attention":
        if device.type == "cuda" and head_dim in (64, 128):
            from ...ops.attention import flash_attention
            T = batch * seq_len
            q, k, v = (r(T, heads, head_dim).requires_grad_() for _ in range(3))
            pos = torch.arange(T, device=device, dtype=torch.int32)
            start = pos // seq_len * seq_len
            return lambda: flash_attention(q, k, v, start, start + seq_len, head_dim ** -0.5)
        q, k, v = (r(batch, heads, seq_len, head_dim).requires_grad_() for _ in range(3))
        return lambda: F.scaled_dot_product_attention(q, k, v, is_causal=True)
    if op == "gla":
        from ...ops.linear_recurrence import chunk_gla
        q, k, v = (r(batch, heads, seq_len, head_dim).requires_grad_() for _ in range(3))
        gate = F.logsigmoid(r(batch, heads, seq_len, head_dim, dt=torch.float32)).requires_grad_()
        return lambda: chunk_gla(q, k, v, gate)
    if op == "long_conv":
        d = heads * head_dim
        x = r(batch, d, seq_len, dt=torch.float32).requires_grad_()
        filt = r(d, seq_len, dt=torch.float32).requires_grad_()

        def fft_conv():
            n = 2 * seq_len
            return torch.fft.irfft(torch.fft.rfft(x, n=n) * torch.fft.rfft(filt, n=n), n=n)[..., :seq_len]
        return fft_conv
    raise ValueError(f"unknown operator {op}; available: {OPERATORS}")


def profile_operator(op: str, batch: int = 8, seq_len: int = 2048, heads: int = 16, head_dim: int = 64, dstate: int = 64,
                     backward: bool = False, iters: int = 10, warmup: int = 3, device=None) -> float:
    """Milliseconds per call."""
    device = torch.device(device or ("cuda" if torch.cuda.is_available() else "cpu"))
    dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
    fn = _inputs(op, batch, seq_len, heads, head_dim, dstate, device, dtype)

    def run():
        y = fn()
        y = y[0] if isinstance(y, tuple) else y
        if backward:
            y.float().sum().backward()

    for _ in range(warmup):
        run()
    if device.type == "cuda":
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(device)
        a.record()
        for _ in range(iters):
            run()
        b.record()
        torch.cuda.synchronize(device)
        return a.elapsed_time(b) / iters
    t = time.perf_counter()
    for _ in range(iters):
        run()
    return (time.perf_counter() - t) * 1e3 / iters


def wall_clock_table(ops=OPERATORS, seq_lens=(1024, 2048, 4096), **kw) -> list[dict]:
    rows = []
    for L in seq_lens:
        row = {"seq_len": L}
        for op in ops:
            row[op] = round(profile_operator(op, seq_len=L, **kw), 4)
        rows.append(row)
        print(json.dumps(row), flush=True)
    return rows


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--ops", default=",".join(OPERATORS))
    ap.add_argument("--seq-lens", default="1024,2048,4096")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--head-dim", type=int, default=64)
    ap.add_argument("--dstate", type=int, default=64)
    ap.add_argument("--backward", action="store_true")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--device", default=None)
    a = ap.parse_args(argv)
    return wall_clock_table(a.ops.split(","), [int(v) for v in a.seq_lens.split(",")], batch=a.batch, heads=a.heads, head_dim=a.head_dim,
                            dstate=a.dstate, backward=a.backward, iters=a.iters, device=a.device)


if __name__ == "__main__":
    main()
