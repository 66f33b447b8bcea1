"""GPT speedrun trainer (classic configuration): ``torchrun --standalone --nproc_per_node=N -m ml_experiments_b200.cli.train_gpt``.

Main-loop behaviour follows the reference script (records/track_1_short/2025-01-26_BatchSize/...txt:462-625 and
modded-nanogpt/train_gpt.py:1755-1910): torchrun environment, NCCL process group, parameters broadcast from rank 0, a
run log ``logs/{run_id}.txt`` that starts with this file's source and the ``nvidia-smi`` table, timing that excludes
validation, ``step:i/N val_loss:... train_time:...ms step_avg:...ms`` lines, validation every ``--val-loss-every``
steps averaged over ranks, peak memory at exit and an optional final checkpoint ``dict(step, code, model, optimizers)``.
``--synthetic`` trains on uniform random tokens (no data files needed); otherwise ``.bin`` shards are read.
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
import time
import uuid

import torch
import torch.distributed as dist

from ..data.nanogpt_loader import distributed_data_generator
from ..models.gpt import GPTConfig
from ..trainers.gpt_trainer import GPTTrainer, Hyperparameters, init_distributed, synthetic_batch, window_blocks


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--train-files", default="data/fineweb10B/fineweb_train_*.bin")
    ap.add_argument("--val-files", default="data/fineweb10B/fineweb_val_*.bin")
    ap.add_argument("--num-iterations", type=int, default=1770)
    ap.add_argument("--seq-len", type=int, default=48 * 1024)
    ap.add_argument("--val-tokens", type=int, default=10485760)
    ap.add_argument("--val-loss-every", type=int, default=125)
    ap.add_argument("--save-checkpoint", action="store_true")
    ap.add_argument("--resume", default=None, help="checkpoint written by --save-checkpoint (any world size)")
    ap.add_argument("--synthetic", action="store_true")
    ap.add_argument("--layers", type=int, default=12)
    a = ap.parse_args(argv)
    rank, local, world = init_distributed()
    master = rank == 0
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    run_id = uuid.uuid4()
    if world > 1:      # every rank writes its optimizer shard into the run's checkpoint folder: agree on the id
        import torch.distributed as dist

        box = [str(run_id)]
        dist.broadcast_object_list(box, src=0)
        run_id = box[0]
    logfile = None
    if master:
        os.makedirs("logs", exist_ok=True)
        logfile = f"logs/{run_id}.txt"
        print(logfile)

    def print0(s, console=False):
        if master:
            with open(logfile, "a") as f:
                if console:
                    print(s)
                print(s, file=f)

    print0(open(__file__).read())
    print0("=" * 100)
    print0(f"Running Python {sys.version}\nRunning PyTorch {torch.version.__version__} compiled for CUDA {torch.version.cuda}")
    try:
        print0(subprocess.run(["nvidia-smi"], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True).stdout)
    except OSError:
        pass
    print0("=" * 100)
    hp = Hyperparameters(num_iterations=a.num_iterations, seq_len=a.seq_len, val_tokens=a.val_tokens, val_loss_every=a.val_loss_every)
    cfg = GPTConfig(num_layers=a.layers, max_seq_len=a.seq_len, skip_attn_layers=(7,) if a.layers == 12 else ())
    tr = GPTTrainer(cfg, hp, device=dev, rank=rank, world_size=world)
    if a.resume:
        tr.load_checkpoint(a.resume)
        print0(f"resumed from {a.resume} at step {tr.step}", console=True)
    if a.synthetic:
        def batches(seed0):
            i = 0
            while True:
                x, y = synthetic_batch(a.seq_len, seed=seed0 + i)
                yield x, y
                i += 1
        train_iter, val_factory = batches(1000 * rank), lambda: batches(10 ** 6 + rank)
    else:
        gen = distributed_data_generator(a.train_files, a.seq_len * world, a.seq_len, align_to_bos=False, rank=rank,
                                         world_size=world, device=dev)
        train_iter = ((x, y) for x, y, _, _ in gen)
        val_factory = lambda: ((x, y) for x, y, _, _ in distributed_data_generator(
            a.val_files, a.seq_len * world, a.seq_len, align_to_bos=False, rank=rank, world_size=world, device=dev))
    training_time_ms = 0.0
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for step in range(tr.step, a.num_iterations + 1):
        last = step == a.num_iterations
        if step == 10:
            training_time_ms, t0 = 0.0, time.perf_counter()
        timed_steps = float("nan") if step <= 11 else (step - 10) + 1
        w = window_blocks(step, hp)
        if last or (a.val_loss_every > 0 and step % a.val_loss_every == 0):
            torch.cuda.synchronize()
            training_time_ms += 1000 * (time.perf_counter() - t0)
            vsteps = max(1, a.val_tokens // (a.seq_len * world))
            it = val_factory()
            vloss = torch.zeros((), device=dev)
            for _ in range(vsteps):
                x, y = next(it)
                vloss += tr.eval_loss(x, y, w)
            vloss /= vsteps
            print0(f"step:{step}/{a.num_iterations} val_loss:{vloss.item():.4f} train_time:{training_time_ms:.0f}ms "
                   f"step_avg:{training_time_ms / max(timed_steps - 1, 1):.2f}ms", console=True)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
        if last:
            if a.save_checkpoint:
                # rank 0: step / model / replicated optimizer state; every rank: its slice of the Muon momentum
                os.makedirs(f"logs/{run_id}", exist_ok=True)
                tr.save_checkpoint(f"logs/{run_id}/state_step{step:06d}.pt")
            break
        x, y = next(train_iter)
        tr.train_step(x, y, window=w)
        approx = training_time_ms + 1000 * (time.perf_counter() - t0)
        print0(f"step:{step + 1}/{a.num_iterations} train_time:{approx:.0f}ms step_avg:{approx / timed_steps:.2f}ms", console=True)
    print0(f"peak memory allocated: {torch.cuda.max_memory_allocated() // 1024 // 1024} MiB "
           f"reserved: {torch.cuda.max_memory_reserved() // 1024 // 1024} MiB", console=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
