"""Headline benchmark: training throughput (tokens/s) of the GPT-2 124M Muon configuration.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # the unmodified reference model / optimizer classes, same protocol

Config: 12 layers, d_model 768, 6 heads x 128, vocab 50304 (fp8 lm_head), RoPE, ReLU², RMSNorm;
Muon on hidden matrices, Adam on embeddings / head / scalars; 48 x 1024 tokens per rank per step (weak scaling), token
ids uniform in [0, 50257) with a BOS token every 1024 positions (documents of 1024 tokens), random-init weights.

Protocol: W untimed warm-up steps, then exactly K optimizer steps (forward, backward, gradient synchronisation,
Muon + Adam updates) bracketed by barrier + synchronize and CUDA events; the reported time is the maximum over ranks.
Inputs of the device-timed loop are resident on the GPU and rotate over a pool larger than the step's working set is
not needed: one step streams > 20 GB of activations through HBM, far more than the 126 MB L2. A second loop measures the
same metric end to end through ``GPTTrainer.train_step`` with a host-to-device copy of every step's tokens from pinned
memory and a device-to-host read of the loss. SM clocks and throttle reasons are sampled with nvidia-smi during the
timed region.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

BASELINE_TOKENS_PER_S = 3.93e6   # 8xH100, step_avg 100.00 ms at 393 216 tokens/step (published reference number)
SEQ_LEN = 48 * 1024
WINDOW_BLOCKS = 14               # final sliding window of the run (1792 tokens): the most work per step


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.path = index, None, None

    def start(self):
        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=f,
                                         stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        try:
            for line in open(self.path):
                parts = [x.strip() for x in line.split(",")]
                if len(parts) < 8:
                    continue
                try:
                    sm.append(float(parts[0])); mx.append(float(parts[1])); power.append(float(parts[2]))
                except ValueError:
                    continue
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[4:8]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except OSError:
            pass
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm),
                       power_w_max=max(power) if power else None)
        return out


def run_ours(args, rank, local, world):
    import torch
    import torch.distributed as dist

    from ml_experiments_b200.models.gpt import GPTConfig
    from ml_experiments_b200.ops import runtime
    from ml_experiments_b200.trainers.gpt_trainer import GPTTrainer, Hyperparameters, synthetic_batch

    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    cfg = GPTConfig(max_seq_len=SEQ_LEN)
    trainer = GPTTrainer(cfg, Hyperparameters(seq_len=SEQ_LEN), device=dev, rank=rank, world_size=world, seed=0)
    # a small pool of distinct synthetic batches (per rank), on the host in pinned memory
    pool = [synthetic_batch(SEQ_LEN, seed=1000 * rank + i) for i in range(4)]
    dev_pool = [(x.to(dev), y.to(dev)) for x, y in pool]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(loop_fn, steps):
        barrier()
        sampler = ClockSampler(local)
        sampler.start()
        runtime.reset_launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        loop_fn(steps)
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        launches = runtime.launch_count()
        clocks = sampler.stop()
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()), launches, clocks

    def device_loop(steps):
        for i in range(steps):
            x, y = dev_pool[i % len(dev_pool)]
            trainer.train_step(x, y, window=WINDOW_BLOCKS)

    losses = []

    def e2e_loop(steps):
        for i in range(steps):
            x, y = pool[i % len(pool)]                      # pinned host tensors -> H2D inside train_step
            loss = trainer.train_step(x, y, window=WINDOW_BLOCKS)
            losses.append(float(loss.item()))               # D2H read of the step's result

    first_loss = float(trainer.train_step(*dev_pool[0], window=WINDOW_BLOCKS).item())   # loss at initialisation (= ln V)
    device_loop(args.warmup - 1)
    if args.breakdown:
        # not a timing run: per-kernel device time of three steps, as shares of one step
        from torch.profiler import ProfilerActivity, profile

        barrier()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            device_loop(3)
            torch.cuda.synchronize()
        if rank == 0:
            ev = [e for e in prof.key_averages() if e.device_time_total > 0]
            total = sum(e.device_time_total for e in ev)
            print(f"device time per step: {total / 3e3:.2f} ms over {sum(e.count for e in ev) // 3} launches")
            for e in sorted(ev, key=lambda e: -e.device_time_total)[: args.breakdown]:
                print(f"{100 * e.device_time_total / total:5.1f} %  {e.device_time_total / 3e3:8.3f} ms/step  {e.count // 3:4d} x {e.device_time_total / e.count:9.1f} us  {e.key[:110]}")
        return
    ms, launches, clocks = timed(device_loop, args.steps)
    e2e_loop(min(2, args.warmup))
    ms_e2e, _, _ = timed(e2e_loop, args.steps)
    runtime.check_status()
    tokens = SEQ_LEN * world * args.steps
    value = tokens / (ms / 1e3)
    e2e_value = tokens / (ms_e2e / 1e3)
    h2d = pool[0][0].numel() * pool[0][0].element_size() + pool[0][1].numel() * pool[0][1].element_size()
    if rank == 0:
        print(json.dumps({
            "metric": "tokens/s (device, max over ranks) GPT-2 124M Muon; ms/step",
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": value / BASELINE_TOKENS_PER_S, "dtype": "bf16 (fp8 lm_head)", "data": "synthetic",
            "impl": "ours",
            "config": {"model": "modded-nanogpt GPT-2 124M (12L, d768, 6x128, vocab 50304, fp8 lm_head, Muon+Adam)",
                       "global_batch": SEQ_LEN * world, "seq_len": 1024, "tokens_per_rank_per_step": SEQ_LEN,
                       "parallelism": f"dp{world}", "comm": trainer.comm_mode, "window_blocks": WINDOW_BLOCKS,
                       "l2": "inputs larger than L2: every step streams >20 GB of activations"},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
            "gpu_launches": launches,
            "first_loss": first_loss, "final_loss": losses[-1] if losses else None,
            "e2e_loss_min_max": [min(losses), max(losses)] if losses else None,
        }), flush=True)
    # a run whose loss never moved (or is not finite) did not train: fail loudly instead of reporting a throughput
    final = losses[-1] if losses else float("nan")
    trained = final == final and abs(final) != float("inf") and final != first_loss
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if not trained:
        if rank == 0:
            print(f"bench.py: loss did not move or is not finite ({first_loss} -> {final}); the timed steps are not valid training steps",
                  file=sys.stderr, flush=True)
        sys.exit(3)


def run_reference(args):
    """The reference's own classes and code path (see baseline/reference_arm.py); imports nothing of this package."""
    from baseline.reference_arm import run as run_ref

    run_ref(args, SEQ_LEN, WINDOW_BLOCKS, BASELINE_TOKENS_PER_S, ClockSampler)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--breakdown", type=int, default=0, metavar="ROWS",
                    help="instead of timing, profile 3 steps with torch.profiler and print the ROWS kernels with the most device time")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    world_env = int(os.environ.get("WORLD_SIZE", "1"))
    if args.gpus > 1 and world_env == 1:
        # convenience: re-launch under torchrun when called directly with --gpus N
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", os.environ.get("MASTER_PORT", "29511"), __file__,
               "--gpus", str(args.gpus), "--steps", str(args.steps), "--warmup", str(args.warmup), "--impl", args.impl]
        sys.exit(subprocess.call(cmd))
    if args.impl == "reference":
        try:
            run_reference(args)
        except Exception as e:  # the reference arm must never fail the driver: report the actual error
            import traceback

            traceback.print_exc()
            if int(os.environ.get("RANK", "0")) == 0:
                msg = " ".join(f"{type(e).__name__}: {e}".split())
                print(json.dumps({"impl": "reference", "unavailable": msg[:400]}), flush=True)
        return
    from ml_experiments_b200.trainers.gpt_trainer import init_distributed

    rank, local, world = init_distributed()
    run_ours(args, rank, local, world)


if __name__ == "__main__":
    main()
