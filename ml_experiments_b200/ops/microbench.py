"""Single-operator benchmark: ``python -m ml_experiments_b200.ops.microbench <op> [sizes]`` prints one JSON line.

Times one of the hand-written kernels (CUDA events on the launching stream, warm-up, L2 flushed between iterations by
writing a 256 MB buffer) and reports achieved FLOP/s or bytes/s against the measured peaks in ``MEASURED_PEAKS.json`` at
the repository root when present (6.65 TB/s and 1.59 PFLOP/s otherwise). The same command line with ``--iters 1
--warmup 0`` is what the profiler captures are taken on. The reference ships comparable sweep scripts for its own
operators (scripts/bench_crossover.py, scripts/benchmark_scatter_attention.py).
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch


def _peaks() -> dict:
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def _time(fn, iters: int, warmup: int, flush: bool = True) -> float:
    scratch = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush else None
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if flush:
            scratch.fill_(1)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        total += s.elapsed_time(e)
    return total / iters


def _doc_bounds(t: int, doc_len: int):
    idx = torch.arange(t, device="cuda", dtype=torch.int32)
    if doc_len <= 0:
        return torch.zeros_like(idx), torch.full_like(idx, t)
    start = idx // doc_len * doc_len
    return start, (start + doc_len).clamp(max=t)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("op", choices=["gemm", "attn_fwd", "attn_bwd", "softcap_ce", "s6_fwd", "s6_bwd", "gather_fwd", "gather_bwd",
                                   "newton_schulz", "ssd", "ssd_bwd", "jacobi", "jacobi_bwd", "tele_fwd", "tele_bwd", "alc_fwd", "alc_bwd", "rms_act", "rms_act_bwd"])
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--heads", type=int, default=6)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--window-blocks", type=int, default=0)
    ap.add_argument("--doc-len", type=int, default=0)
    ap.add_argument("--vocab", type=int, default=50304)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--channels", type=int, default=2048)
    ap.add_argument("--taps", type=int, default=16)
    ap.add_argument("--epilogue", default="none", choices=["none", "relu2", "axpby"])
    ap.add_argument("--ce-cache", type=int, default=1, help="softcap_ce: 1 keeps exp(z) of the row in shared memory, 0 recomputes it")
    ap.add_argument("--s6-qs", default=None, help="states per thread of the S6 forward,backward kernels, e.g. 2,4")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    a = ap.parse_args(argv)
    from . import gemm as G
    from .runtime import check_status
    dev, bf = "cuda", torch.bfloat16
    flops = bytes_ = 0.0
    if a.op == "gemm":
        x = torch.randn(a.m, a.k, device=dev, dtype=bf)
        w = torch.randn(a.n, a.k, device=dev, dtype=bf)
        out = torch.empty(a.m, a.n, device=dev, dtype=bf)
        aux = torch.randn(a.m, a.n, device=dev, dtype=bf) if a.epilogue == "axpby" else None
        epi = {"none": G.EPI_NONE, "relu2": G.EPI_RELU2, "axpby": G.EPI_AXPBY}[a.epilogue]
        fn = lambda: G.gemm(x, w, out=out, epilogue=epi, aux=aux, beta=1.0 if aux is not None else 0.0)
        flops = 2.0 * a.m * a.n * a.k
        bytes_ = 2.0 * (a.m * a.k + a.n * a.k + a.m * a.n * (2 if aux is not None else 1))
    elif a.op in ("attn_fwd", "attn_bwd"):
        from . import attention as A
        t, h, d = a.tokens, a.heads, a.head_dim
        q, k, v = (torch.randn(t, h, d, device=dev, dtype=bf) for _ in range(3))
        ds, de = _doc_bounds(t, a.doc_len)
        scale = d ** -0.5
        o, lse = A.flash_attention_forward(q, k, v, ds, de, scale, a.window_blocks)
        span = t if a.window_blocks <= 0 else min(t, a.window_blocks * 128)
        if a.doc_len > 0:
            span = min(span, a.doc_len)
        pairs = t * span / (2.0 if span == t else 1.0)  # causal: half the square, or a band
        if a.op == "attn_fwd":
            fn = lambda: A.flash_attention_forward(q, k, v, ds, de, scale, a.window_blocks)
            flops = 4.0 * pairs * h * d
        else:
            do = torch.randn_like(o)
            dq = torch.zeros(t, h, d, device=dev, dtype=torch.float32)
            fn = lambda: A.flash_attention_backward(q, k, v, o, do, lse, ds, de, scale, a.window_blocks, dq_acc=dq)
            flops = 10.0 * pairs * h * d
        bytes_ = 2.0 * 4 * t * h * d
    elif a.op == "softcap_ce":
        from . import fused as Fz
        from .runtime import ops as _ops
        _ops().softcap_ce_set_cache(bool(a.ce_cache), torch.empty(0, device=dev))
        logits = torch.randn(a.tokens, a.vocab, device=dev, dtype=bf)
        tgt = torch.randint(0, a.vocab, (a.tokens,), device=dev, dtype=torch.int64)
        grad = torch.empty_like(logits)
        fn = lambda: Fz.softcap_ce(logits, tgt, grad_out=grad)
        bytes_ = 2.0 * 2 * a.tokens * a.vocab
    elif a.op in ("s6_fwd", "s6_bwd"):
        from .selective_scan import selective_scan, set_states_per_thread
        if a.s6_qs:
            set_states_per_thread(*[int(v) for v in a.s6_qs.split(",")])
        b, L, d, n = a.batch, a.seq, a.channels, 16
        u = torch.randn(b, L, d, device=dev, dtype=bf, requires_grad=True)
        delta = (torch.rand(b, L, d, device=dev) * 0.1).requires_grad_(True)
        A_ = -torch.rand(d, n, device=dev).requires_grad_(True)
        Bm, Cm = (torch.randn(b, L, n, device=dev, requires_grad=True) for _ in range(2))
        D = torch.ones(d, device=dev, requires_grad=True)
        z = torch.randn(b, L, d, device=dev, dtype=bf, requires_grad=True)
        if a.op == "s6_fwd":
            fn = lambda: selective_scan(u.detach(), delta.detach(), A_.detach(), Bm.detach(), Cm.detach(), D.detach(), z.detach())
            bytes_ = b * L * d * (2 + 4 + 2 + 2 + 2.0)
        else:
            y = selective_scan(u, delta, A_, Bm, Cm, D, z)
            g = torch.randn_like(y)
            fn = lambda: torch.autograd.grad(y, (u, delta, A_, Bm, Cm, D, z), g, retain_graph=True)
            bytes_ = b * L * d * (2 + 4 + 2 + 2 + 2 + 2 + 4 + 2.0)
        flops = 9.0 * b * L * d * n
    elif a.op in ("gather_fwd", "gather_bwd"):
        from .gather_conv import gather_conv
        b, L, c, h, s = a.batch, a.seq, a.channels, a.heads, a.taps
        x = torch.randn(b, L, c, device=dev, dtype=bf, requires_grad=True)
        pos = (torch.rand(b, L, h, s, device=dev) * (L - 1)).requires_grad_(True)
        wgt = torch.rand(b, L, h, s, device=dev, requires_grad=True)
        if a.op == "gather_fwd":
            fn = lambda: gather_conv(x.detach(), pos.detach(), wgt.detach(), h)
        else:
            y = gather_conv(x, pos, wgt, h)
            g = torch.randn_like(y)
            fn = lambda: torch.autograd.grad(y, (x, pos, wgt), g, retain_graph=True)
        bytes_ = b * L * (2.0 * c * (1 + 2 * s) + 8.0 * h * s)  # every tap reads two rows of its head
    elif a.op in ("tele_fwd", "tele_bwd", "alc_fwd", "alc_bwd"):
        from . import fused_taps as T
        b, L, c, h, s = a.batch, a.seq, a.channels, a.heads, a.taps
        half, K = s // 2, 64
        x = torch.randn(b, L, c, device=dev, dtype=bf, requires_grad=True)
        kern = torch.randn(b, L, h, K, device=dev, requires_grad=True)
        if a.op.startswith("tele"):
            p1 = (torch.rand(b, L, h, device=dev) * 15 + 1).requires_grad_(True)          # stride per sample
            p2 = ((torch.rand(b, L, h, device=dev) * 2 - 1) * 16).requires_grad_(True)    # phase
            expo = (torch.rand(b, L, 1, device=dev) * 3.5 + 0.5).requires_grad_(True)
            call = lambda xx, *ps: T.telephone_gather(xx, *ps, h, half, half * 16.0)
            leaves = (x, p1, p2, kern, expo)
        else:
            p1 = (torch.rand(b, L, h, device=dev) * half + 0.5).requires_grad_(True)      # half window
            p2 = ((torch.rand(b, L, h, device=dev) * 2 - 1) * half).requires_grad_(True)  # centre offset
            call = lambda xx, *ps: T.adaptive_local_gather(xx, *ps, h, half)
            leaves = (x, p1, p2, kern)
        if a.op.endswith("fwd"):
            det = tuple(t.detach() for t in leaves)
            fn = lambda: call(*det)
        else:
            y = call(*leaves)
            g = torch.randn_like(y)
            fn = lambda: torch.autograd.grad(y, leaves, g, retain_graph=True)
        taps = 2 * half + 1
        bytes_ = b * L * (2.0 * c * (1 + 2 * taps) + 4.0 * h * (K + 3))  # every tap reads two bf16 rows of its head (mostly from L2)
    elif a.op == "rms_act":
        from .norm_act import rms_norm_act
        x = torch.randn(a.batch * a.seq, a.channels, device=dev, dtype=bf)
        w = torch.ones(a.channels, device=dev)
        fn = lambda: rms_norm_act(x, w, 1e-6, "silu", torch.float32)
        bytes_ = x.numel() * 6.0
    elif a.op == "rms_act_bwd":
        # backward of the bf16 RMSNorm with the gradient of a skip connection added in the same kernel
        from .runtime import ops
        x = torch.randn(a.batch * a.seq, a.channels, device=dev, dtype=bf)
        dy, dres, dx = torch.randn_like(x), torch.randn_like(x), torch.empty_like(x)
        w, rstd = torch.ones(a.channels, device=dev), torch.rsqrt(x.float().pow(2).mean(-1) + 1e-6)
        dw = torch.zeros(a.channels, device=dev)
        fn = lambda: ops().rms_act_bwd(x, w, rstd, dy, dres, None, dx, dw, 0)
        bytes_ = x.numel() * 8.0
    elif a.op == "newton_schulz":
        from .newton_schulz import newton_schulz_
        X = torch.randn(a.batch, a.m, a.n, device=dev, dtype=bf)
        X /= X.norm(dim=(1, 2), keepdim=True)
        work: dict = {}
        fn = lambda: newton_schulz_(X.clone(), work=work)
        small, big = min(a.m, a.n), max(a.m, a.n)
        flops = 5 * a.batch * (2.0 * small * small * big * 2 + 2.0 * small ** 3)
    elif a.op in ("jacobi", "jacobi_bwd"):
        # MIMO-Jacobi iteration (state 64, rank 4, 12 iterations) on [batch, seq]: fused kernel against the PyTorch loop
        from .jacobi_iter import jacobi_iterate, jacobi_iterate_torch
        b, L, R, n, iters_ = a.batch, a.seq, 4, 64, 12
        mk = lambda *s: torch.randn(*s, device=dev)
        args = [mk(b, L, n, R).permute(0, 3, 1, 2), mk(b, L, n, R).permute(0, 3, 1, 2), mk(b, L, n // 2), mk(b, L, R).permute(0, 2, 1),
                torch.sigmoid(mk(b, L, n)), torch.sigmoid(mk(b, L)), mk(n, 3) * 0.4, mk(n) * 0.1]
        train = a.op == "jacobi_bwd"
        if train:
            args = [t.requires_grad_(True) for t in args]

        def run(f):
            if not train:
                with torch.no_grad():
                    return f(*args, None, None, iters_)
            y = f(*args, None, None, iters_)
            y.backward(torch.ones_like(y))
            return y
        torch_ms = _time(lambda: run(jacobi_iterate_torch), max(a.iters // 4, 2), 1)
        fn = lambda: run(jacobi_iterate)
        state = b * R * L * n * 4.0
        # forward: B, C in, gated out (+ the n saved states when training); backward: the saved states, dgated, dB, dC
        bytes_ = state * (3 + (iters_ if train else 0)) + (state * (iters_ + 3) if train else 0)
        extra = {"torch_formulation_ms": round(torch_ms, 4)}
    else:  # ssd
        from .ssd_scan import ssd_chunk_scan
        b, L, h, p, n = a.batch, a.seq, a.heads, a.head_dim, 64
        x = torch.randn(b, L, h, p, device=dev, dtype=bf)
        Bm, Cm = (torch.randn(b, L, h, n, device=dev, dtype=bf) for _ in range(2))
        la = -torch.rand(b, L, h, device=dev) * 0.1
        gm = torch.rand(b, L, h, device=dev)
        import os

        from .ssd_scan import _ssd_chunk_scan_torch

        train = a.op == "ssd_bwd"
        if train:       # forward + backward: four launches of the kernel against autograd through the GEMM formulation
            for t in (x, Bm, Cm, la, gm):
                t.requires_grad_(True)

        def run(f):
            if not train:
                with torch.no_grad():
                    return f(x, Bm, Cm, la, gm)
            y = f(x, Bm, Cm, la, gm)
            y.backward(torch.ones_like(y))
            return y
        torch_ms = _time(lambda: run(_ssd_chunk_scan_torch), max(a.iters // 4, 2), 2)          # the batched-GEMM formulation, for the ratio
        fn = lambda: run(ssd_chunk_scan)
        flops = 2.0 * b * L * h * (128 * n + 128 * p + 2 * n * p)     # kernel: 128-step chunks
        bytes_ = (x.numel() * 2 + Bm.numel() * 2) * 2.0 + la.numel() * 12.0
        if train:
            flops, bytes_ = 4 * flops, 4 * bytes_
        extra = {"torch_formulation_ms": round(torch_ms, 4)}
    ms = _time(fn, a.iters, a.warmup)
    check_status()
    extra = locals().get("extra", {})
    pk = _peaks()
    out = {"op": a.op, "ms": round(ms, 4), "args": {k: v for k, v in vars(a).items() if k != "op"}, "peaks": pk["source"]}
    out.update(extra)
    if "torch_formulation_ms" in extra:
        out["speedup_vs_torch_formulation"] = round(extra["torch_formulation_ms"] / ms, 2)
    if flops:
        out["tflops"] = round(flops / ms / 1e9, 1)
        out["frac_of_bf16_peak"] = round(flops / ms / 1e9 / pk["bf16_tflops"], 3)
    if bytes_:
        out["gbs"] = round(bytes_ / ms / 1e6, 1)
        out["frac_of_hbm_peak"] = round(bytes_ / ms / 1e6 / pk["hbm_gbs"], 3)
    print(json.dumps(out))


if __name__ == "__main__":
    main()
