"""Peak-memory diagnostics of the gather operators (roles of the reference's ``scripts/diagnose_telephone.py`` and
``scripts/diagnose_gather_mem.py``): forward and forward+backward peak device memory of

* ``telephone``: the telephone attention layer, whole-sequence fused tap kernel against its chunked + checkpointed
  composition (the trade the reference tunes with ``checkpoint=True``);
* ``gather``: a sampled gather ``out[b, l] = sum_s w[b, l, h, s] x[b, idx[b, l, h, s]]`` done three ways: materialise
  every gathered row (``x[batch_idx, sample_idx]``), accumulate one tap at a time, and the fused gather kernel, which
  never stores a gathered row.

A case whose estimated materialised tensor exceeds ``--limit-gb`` is reported as skipped rather than run. On a host
without a GPU the table holds the estimates only.

    python -m ml_experiments_b200.cli.diagnose_memory --what gather --lengths 512,2048,8192
"""
from __future__ import annotations

import argparse
import json

import torch

from ..ops.gather_conv import gather_conv, gather_conv_ref


def peak_mb(fn, device) -> tuple[float, float]:
    """Runs ``fn() -> tensor``; returns (peak MB above the starting allocation after forward, after backward)."""
    if device.type != "cuda":
        out = fn()
        out.float().sum().backward()
        return 0.0, 0.0
    torch.cuda.synchronize(device)
    torch.cuda.empty_cache()
    base = torch.cuda.memory_allocated(device)
    torch.cuda.reset_peak_memory_stats(device)
    out = fn()
    torch.cuda.synchronize(device)
    fwd = torch.cuda.max_memory_allocated(device) - base
    out.float().sum().backward()
    torch.cuda.synchronize(device)
    bwd = torch.cuda.max_memory_allocated(device) - base
    return fwd / 2 ** 20, bwd / 2 ** 20


def gather_cases(B, L, C, H, S, device, dtype):
    g = torch.Generator(device=device).manual_seed(L)
    x = torch.randn(B, L, C, device=device, dtype=dtype, generator=g).requires_grad_()
    pos = torch.rand(B, L, H, S, device=device, generator=g) * (L - 1)
    wgt = torch.softmax(torch.randn(B, L, H, S, device=device, generator=g), -1)
    D = C // H
    idx = pos.round().long()

    def materialise():
        rows = x.view(B, L, H, D)[torch.arange(B, device=device).view(B, 1, 1, 1), idx, torch.arange(H, device=device).view(1, 1, H, 1)]
        return (rows * wgt.unsqueeze(-1).to(dtype)).sum(3).reshape(B, L, C)

    def per_tap():
        out = torch.zeros(B, L, H, D, device=device, dtype=dtype)
        xh = x.view(B, L, H, D)
        for s in range(S):
            rows = torch.gather(xh, 1, idx[..., s].unsqueeze(-1).expand(B, L, H, D))
            out = out + rows * wgt[..., s].unsqueeze(-1).to(dtype)
        return out.reshape(B, L, C)

    def fused():
        return (gather_conv if x.is_cuda else gather_conv_ref)(x, pos, wgt, H)

    return {"materialise": materialise, "per_tap": per_tap, "fused": fused}, x


def run_gather(a, device):
    rows = []
    dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
    esize = 2 if dtype == torch.bfloat16 else 4
    for L in a.lengths:
        est_gb = a.batch * L * a.samples * a.channels * esize / 2 ** 30
        row = {"L": L, "materialised_estimate_gb": round(est_gb, 3)}
        cases, x = gather_cases(a.batch, L, a.channels, a.heads, a.samples, device, dtype)
        for name, fn in cases.items():
            if name != "fused" and 3 * est_gb > a.limit_gb:               # forward + saved + gradient copies
                row[name] = "skipped"
                continue
            x.grad = None
            f, b = peak_mb(fn, device)
            row[name] = {"fwd_mb": round(f, 1), "bwd_mb": round(b, 1)}
        rows.append(row)
        print(json.dumps(row), flush=True)
        del cases, x
    return rows


def run_telephone(a, device):
    from ..models.ripple_ops import TelephoneAttentionND
    rows = []
    for L in a.lengths:
        row = {"L": L}
        for name, kw in (("fused_or_whole", dict(checkpoint=False, chunk_size=L)), ("chunked_checkpoint", dict(checkpoint=True, chunk_size=min(1024, L)))):
            torch.manual_seed(0)
            layer = TelephoneAttentionND(a.channels, ndim=1, num_heads=a.heads, **kw).to(device).train()
            layer.fused = name != "chunked_checkpoint"
            x = torch.randn(a.batch, L, a.channels, device=device, requires_grad=True)

            def fn():
                out = layer(x)
                return out[0] if isinstance(out, tuple) else out
            with torch.autocast(device.type, dtype=torch.bfloat16, enabled=device.type == "cuda"):
                f, b = peak_mb(fn, device)
            row[name] = {"fwd_mb": round(f, 1), "bwd_mb": round(b, 1)}
            del layer, x
        rows.append(row)
        print(json.dumps(row), flush=True)
    return rows


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--what", default="gather", choices=["gather", "telephone"])
    ap.add_argument("--lengths", type=lambda s: [int(v) for v in s.split(",")], default=[512, 1024, 2048, 4096, 8192, 16384])
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--channels", type=int, default=256)
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--samples", type=int, default=33)
    ap.add_argument("--limit-gb", type=float, default=16.0)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args(argv)
    device = torch.device(a.device)
    return run_gather(a, device) if a.what == "gather" else run_telephone(a, device)


if __name__ == "__main__":
    main()
