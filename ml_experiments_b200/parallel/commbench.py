"""Multi-rank benchmark of the fused peer-memory collectives against NCCL and against their rooflines.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 --master-port P -m ml_experiments_b200.parallel.commbench

Every number is timed with CUDA events on the launching stream after warm-up, bracketed by barrier + synchronize, and
reported as the maximum over ranks. Rank 0 prints one JSON line per measurement:

* ``allreduce``: the two-shot peer-memory mean all-reduce (scale and dtype handling fused) and ``dist.all_reduce`` on
  the same sizes. Each rank moves ``(W-1)/W * bytes`` in each direction, so the roofline time is that over the
  per-direction link bandwidth (``--link-gbs``, 770 GB/s measured peer copy by default).
* ``muon_step``: one fused Muon step (reduce-scatter + momentum + cast, Newton-Schulz on the owned slice, all-gather by
  peer stores + weight update) on the hidden matrices of a GPT of the given shape, with the equivalent built from NCCL
  ``reduce_scatter_tensor`` / ``all_gather_into_tensor`` around the same Newton-Schulz for comparison. Roofline = the
  slower of the Newton-Schulz FLOPs at the measured GEMM peak and the bytes crossing NVLink at link bandwidth
  (fp32 gradients in: ``(W-1)/W * 4`` bytes per element; bf16 updates out: ``(W-1)/W * 2`` bytes per element).
"""
from __future__ import annotations

import argparse
import json
import os
from pathlib import Path

import torch
import torch.distributed as dist

from ..ops.newton_schulz import newton_schulz_
from ..ops.runtime import check_status, ops, status
from ..optim.muon import NS5_COEFFS
from .ddp import CH_IN, CH_OUT
from .muon_dist import MuonShardEngine
from .symm import SymmWorld


def _timed(fn, iters, warmup, dev):
    for _ in range(warmup):
        fn()
    dist.barrier()
    torch.cuda.synchronize(dev)
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    dist.barrier()
    torch.cuda.synchronize(dev)
    t = torch.tensor([s.elapsed_time(e) / iters], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _gemm_peak_tflops():
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    return (json.loads(p.read_text())["bf16_tflops"], "measured") if p.exists() else (1590.0, "fallback")


def bench_allreduce(w: SymmWorld, sizes_mb, iters, warmup, link_gbs, emit, use_nvls=False):
    o, dev, W = ops(), w.device, w.world
    epoch = [0]
    for dtype, code in ((torch.bfloat16, 1), (torch.float32, 0)):
        esize = torch.tensor([], dtype=dtype).element_size()
        for mb in sizes_mb:
            vec = (8 if code else 4) * W
            n = (mb * (1 << 20) // esize) // vec * vec
            buf = w.alloc(n, dtype, zero=True)
            buf.local.normal_()
            ref = buf.local.clone()

            def fused():
                epoch[0] += 1
                o.comm_signal(w.flags.ptrs, w.rank, CH_IN, 10_000_000 + epoch[0], w.flags.local)
                o.allreduce_mean(buf.ptrs, w.rank, n, code, w.flags.local, w.flags.ptrs, CH_IN, 10_000_000 + epoch[0], status(dev))
                o.comm_wait(w.flags.local, W, CH_OUT, 10_000_000 + epoch[0], status(dev))

            def nccl():
                dist.all_reduce(ref, op=dist.ReduceOp.AVG)

            def nvls():
                epoch[0] += 1
                o.comm_signal(w.flags.ptrs, w.rank, CH_IN, 10_000_000 + epoch[0], w.flags.local)
                o.allreduce_mean_multimem(buf.mc_ptr, W, w.rank, n, code, w.flags.local, w.flags.ptrs, CH_IN, 10_000_000 + epoch[0], status(dev))
                o.comm_wait(w.flags.local, W, CH_OUT, 10_000_000 + epoch[0], status(dev))

            t_f, t_n = _timed(fused, iters, warmup, dev), _timed(nccl, iters, warmup, dev)
            t_m = _timed(nvls, iters, warmup, dev) if (use_nvls and buf.mc_ptr) else None
            check_status()

            def max_err(fn):  # every rank contributes rank + 1 + i / n: the mean is known in closed form
                ramp = torch.arange(n, device=dev, dtype=torch.float32) / n
                buf.local.copy_((ramp + w.rank + 1).to(dtype))
                dist.barrier()
                fn()
                torch.cuda.synchronize(dev)
                err = (buf.local.float() - (ramp + (W + 1) / 2)).abs().max()
                dist.all_reduce(err, op=dist.ReduceOp.MAX)
                dist.barrier()
                return round(float(err), 5)

            err_f = max_err(fused)
            err_m = max_err(nvls) if t_m is not None else None
            per_dir = (W - 1) / W * n * esize
            roof_ms = per_dir / (link_gbs * 1e6)
            emit(dict(bench="allreduce", dtype=str(dtype).split(".")[-1], mbytes=round(n * esize / 2 ** 20, 1), world=W, fused_ms=round(t_f, 4),
                      nccl_ms=round(t_n, 4), fused_busbw_gbs=round(2 * per_dir / t_f / 1e6, 1), nccl_busbw_gbs=round(2 * per_dir / t_n / 1e6, 1),
                      fused_max_err=err_f, multimem_max_err=err_m, multimem_ms=None if t_m is None else round(t_m, 4), multimem_frac_of_roofline=None if t_m is None else round(roof_ms / t_m, 3),
                      roofline_ms=round(roof_ms, 4), fused_frac_of_roofline=round(roof_ms / t_f, 3), link_gbs=link_gbs))


def hidden_matrices(layers: int, d: int, dev):
    """Muon's parameter set of a classic GPT block stack: qkv (3 x d x d), attention out (d x d), MLP in / out (4d x d, d x 4d)."""
    ps = []
    for _ in range(layers):
        ps += [torch.nn.Parameter(torch.randn(3, d, d, device=dev) * 0.02), torch.nn.Parameter(torch.randn(d, d, device=dev) * 0.02),
               torch.nn.Parameter(torch.randn(4 * d, d, device=dev) * 0.02), torch.nn.Parameter(torch.randn(d, 4 * d, device=dev) * 0.02)]
    return ps


def bench_muon(w: SymmWorld, layers, d, iters, warmup, link_gbs, emit):
    dev, W = w.device, w.world
    params = hidden_matrices(layers, d, dev)
    for p in params:
        p.grad = torch.randn_like(p)
    eng = MuonShardEngine(params, w)
    coeffs = [NS5_COEFFS[0]] * 5

    def fused():
        eng.publish_grads()
        eng.reduce_ns_push(0.95, True, coeffs)
        eng.apply(0.02)

    t_f = _timed(fused, iters, warmup, dev)
    check_status()
    # the same step from library collectives: reduce-scatter -> momentum -> Newton-Schulz -> all-gather -> update
    state = []
    for g in eng.groups:
        state.append(dict(g=g, gin=torch.randn(g["padded"], g["r"], g["c"], device=dev), gout=torch.empty(g["per"], g["r"], g["c"], device=dev),
                          mom=torch.zeros(g["per"], g["r"], g["c"], device=dev), ufull=torch.empty(g["padded"], g["r"], g["c"], device=dev, dtype=torch.bfloat16)))
    work: dict = {}

    def nccl():
        for s in state:
            dist.reduce_scatter_tensor(s["gout"], s["gin"], op=dist.ReduceOp.AVG)
            s["mom"].lerp_(s["gout"], 0.05)
            u = s["gout"].lerp(s["mom"], 0.95).to(torch.bfloat16)
            u = u / (u.float().norm(dim=(1, 2), keepdim=True) + 1e-7).to(torch.bfloat16)
            u = newton_schulz_(u, coeffs, work)
            dist.all_gather_into_tensor(s["ufull"], u.contiguous())
            s["g"]["p_stack"].add_(s["ufull"].float(), alpha=-0.02)

    t_n = _timed(nccl, iters, warmup, dev)
    elems = sum(g["padded"] * g["mat"] for g in eng.groups)
    flops = 0.0
    for g in eng.groups:
        small, big = min(g["r"], g["c"]), max(g["r"], g["c"])
        flops += g["per"] * 5 * (2.0 * small * small * big * 2 + 2.0 * small ** 3)
    peak, src = _gemm_peak_tflops()
    t_flops = flops / (peak * 1e9)
    # per rank and direction: it pulls (W-1)/W of its 1/W slice in fp32 ( = inbound) and pushes its slice to W-1 peers in bf16 (outbound)
    t_in = (W - 1) * (elems / W) * 4 / (link_gbs * 1e6) if W > 1 else 0.0
    t_out = (W - 1) * (elems / W) * 2 / (link_gbs * 1e6) if W > 1 else 0.0
    roof = max(t_flops, t_in, t_out)
    emit(dict(bench="muon_step", world=W, layers=layers, d_model=d, matrices_melems=round(elems / 1e6, 1), fused_ms=round(t_f, 4), nccl_ms=round(t_n, 4),
              ns_tflop=round(flops / 1e12, 3), roofline_ms=round(roof, 4), roofline_terms_ms=dict(ns_at_gemm_peak=round(t_flops, 4), nvlink_in=round(t_in, 4), nvlink_out=round(t_out, 4)),
              fused_frac_of_roofline=round(roof / t_f, 3), gemm_peak=src, link_gbs=link_gbs))


def bench_adam(w: SymmWorld, vocab: int, d: int, iters, warmup, link_gbs, emit):
    """Embedding / head tables of the GPT-2 124M trainer (4 bf16 tables, 1 fp32 head): the fused sharded Adam (one kernel per
    table: reduce-scatter + update + all-gather) against bucket all-reduce + replicated Adam kernel and against NCCL
    reduce-scatter + torch Adam on the slice + all-gather."""
    from ..optim.adam import FusedAdam
    from .adam_dist import ShardedAdam

    dev, W = w.device, w.world
    mk = lambda dt: torch.nn.Parameter((torch.randn(vocab, d, device=dev) * 0.02).to(dt))
    tables = [mk(torch.bfloat16) for _ in range(4)]
    head = mk(torch.float32)
    sharded = ShardedAdam([dict(params=[head], lr=0.008), dict(params=tables, lr=0.6)], w, betas=(0.8, 0.95), eps=1e-10)
    for p in [head] + tables:
        sharded.grad_views[id(p)].normal_(0, 1e-3)

    def fused():
        for p in [head] + tables:
            p.grad = sharded.grad_views[id(p)]
        sharded.step()

    t_f = _timed(fused, iters, warmup, dev)
    check_status()
    # replicated: bucket all-reduce (two-shot peer kernel) + the Adam kernel on every rank
    rep = [mk(torch.bfloat16) for _ in range(4)] + [mk(torch.float32)]
    b16 = w.alloc(sum(p.numel() for p in rep[:4]) // (8 * W) * (8 * W), torch.bfloat16)
    b32 = w.alloc(rep[4].numel() // (4 * W) * (4 * W), torch.float32)
    b16.local.normal_(0, 1e-3)
    b32.local.normal_(0, 1e-3)
    off = 0
    for p in rep[:4]:
        p.grad = b16.local[off:off + p.numel()].view(p.shape) if off + p.numel() <= b16.local.numel() else torch.zeros_like(p)
        off += p.numel()
    rep[4].grad = b32.local[: rep[4].numel()].view(rep[4].shape) if rep[4].numel() <= b32.local.numel() else torch.zeros_like(rep[4])
    opt = FusedAdam([dict(params=[rep[4]], lr=0.008), dict(params=rep[:4], lr=0.6)], betas=(0.8, 0.95), eps=1e-10)
    o = ops()
    ep = [0]

    def replicated():
        ep[0] += 1
        e = 20_000_000 + ep[0]
        for buf, code, ch in ((b16, 1, 2), (b32, 0, 4)):
            o.comm_signal(w.flags.ptrs, w.rank, ch, e, w.flags.local)
            o.allreduce_mean(buf.ptrs, w.rank, buf.local.numel(), code, w.flags.local, w.flags.ptrs, ch, e, status(dev))
            o.comm_wait(w.flags.local, W, ch + 1, e, status(dev))
        opt.step()

    t_r = _timed(replicated, iters, warmup, dev)
    check_status()
    # NCCL: reduce-scatter, torch Adam on the slice, all-gather
    ncc = []
    for p in rep:
        rows = p.shape[0] // W * W
        g = torch.randn(rows, d, device=dev, dtype=p.dtype) * 1e-3
        sl = torch.nn.Parameter(p.detach()[: rows // W].clone())
        ncc.append(dict(g=g, gs=torch.empty(rows // W, d, device=dev, dtype=p.dtype), sl=sl, full=torch.empty(rows, d, device=dev, dtype=p.dtype)))
    nopt = torch.optim.Adam([c["sl"] for c in ncc], lr=0.01, betas=(0.8, 0.95), eps=1e-10, fused=True)

    def nccl():
        for c in ncc:
            dist.reduce_scatter_tensor(c["gs"], c["g"], op=dist.ReduceOp.AVG)
            c["sl"].grad = c["gs"]
        nopt.step()
        for c in ncc:
            dist.all_gather_into_tensor(c["full"], c["sl"].detach())

    t_n = _timed(nccl, iters, warmup, dev)
    byts = sum(p.numel() * p.element_size() for p in [head] + tables)
    t_link = (W - 1) / W * byts / (link_gbs * 1e6) if W > 1 else 0.0       # per direction: gradients in, parameters out
    emit(dict(bench="sharded_adam", world=W, tables_mbytes=round(byts / 2 ** 20, 1), fused_ms=round(t_f, 4), allreduce_plus_replicated_ms=round(t_r, 4),
              nccl_ms=round(t_n, 4), roofline_ms=round(t_link, 4), fused_frac_of_roofline=round(t_link / t_f, 3) if W > 1 else None, link_gbs=link_gbs))


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes-mb", default="1,16,128,512")
    ap.add_argument("--layers", type=int, default=12)
    ap.add_argument("--d-model", type=int, default=768)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--link-gbs", type=float, default=770.0)
    ap.add_argument("--nvls", action="store_true", help="also time the NVSwitch-multicast (multimem) all-reduce")
    ap.add_argument("--skip", default="", help="comma list of benches to skip (allreduce, muon_step, sharded_adam)")
    a = ap.parse_args(argv)
    rank, world, local = (int(os.environ.get(k, d)) for k, d in (("RANK", 0), ("WORLD_SIZE", 1), ("LOCAL_RANK", 0)))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    w = SymmWorld.create(rank, world, dev)
    emit = lambda d: print(json.dumps(d), flush=True) if rank == 0 else None
    skip = set(a.skip.split(","))
    if "allreduce" not in skip:
        bench_allreduce(w, [int(s) for s in a.sizes_mb.split(",")], a.iters, a.warmup, a.link_gbs, emit, a.nvls)
    if "muon_step" not in skip:
        bench_muon(w, a.layers, a.d_model, a.iters, a.warmup, a.link_gbs, emit)
    if "sharded_adam" not in skip:
        bench_adam(w, 50304, a.d_model, a.iters, a.warmup, a.link_gbs, emit)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
