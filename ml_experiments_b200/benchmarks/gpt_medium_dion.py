"""GPT-2 medium (24 layers, d_model 1024, 16 heads x 64, vocab 50304) with the Dion optimizer (rank d/4), bf16,
32 x 1024 tokens per rank per step.

    python -m ml_experiments_b200.benchmarks.gpt_medium_dion [--shape medium|medium_track] [--steps 5]
``--shape medium_track`` selects the reference's own medium-track shape (16 layers, 8 heads x 128).
"""
from __future__ import annotations

import argparse

import torch

from ..models.gpt import GPTConfig
from ..trainers.gpt_trainer import GPTTrainer, Hyperparameters, synthetic_batch
from .common import emit, init_dist, timed_steps


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", default="medium", choices=["medium", "medium_track"])
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--optimizer", default="dion", choices=["dion", "muon"])
    ap.add_argument("--ortho", default=None, choices=["ns", "cholqr", "qr"], help="Dion orthonormalisation (default: Newton-Schulz GEMMs on CUDA)")
    a = ap.parse_args()
    rank, world, local = init_dist()
    dev = torch.device("cuda", local)
    seq = 32 * 1024
    mk = GPTConfig.gpt2_medium if a.shape == "medium" else GPTConfig.medium_track
    cfg = mk(max_seq_len=seq, uniform_doc_len=1024)
    tr = GPTTrainer(cfg, Hyperparameters(seq_len=seq), device=dev, rank=rank, world_size=world, matrix_optimizer=a.optimizer)
    x, y = synthetic_batch(seq, seed=rank)
    x, y = x.to(dev), y.to(dev)
    if a.ortho and a.optimizer == "dion":
        tr.optimizer2.ortho = a.ortho
    losses = []
    ms = timed_steps(lambda: losses.append(tr.train_step(x, y, window=14)), a.steps, a.warmup, world, dev)
    from ..ops.runtime import check_status

    check_status()
    emit(rank, metric=f"tokens/s GPT-2 medium {a.optimizer}", value=seq * world / (ms / 1e3), unit="tokens/s", ms_per_step=ms,
         n_gpus=world, config=dict(shape=a.shape, layers=cfg.num_layers, heads=cfg.num_heads, head_dim=cfg.head_dim,
                                   tokens_per_rank=seq, optimizer=a.optimizer, comm=tr.comm_mode,
                                   ortho=getattr(tr.optimizer2, "ortho", None)), dtype="bf16 (fp8 lm_head)",
         data="synthetic", first_loss=float(losses[0]), final_loss=float(losses[-1]))


if __name__ == "__main__":
    main()
