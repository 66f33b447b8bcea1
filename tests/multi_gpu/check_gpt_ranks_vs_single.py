"""Run with ``python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 --master-port P
tests/multi_gpu/check_gpt_ranks_vs_single.py --mode fused|nccl``.

Every rank trains the small GPT for a few steps on its own sequence (gradients averaged over the ranks by the fused
peer-memory path or by NCCL); rank 0 then repeats the run in one process, feeding the ranks' sequences as micro-batches
whose gradients are accumulated and averaged, and compares losses and every parameter. Prints one JSON line and exits
non-zero on a mismatch.
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

STEPS = 4
T = 2048


def _cfg():
    from ml_experiments_b200.models.gpt import GPTConfig

    return GPTConfig(num_layers=4, num_heads=2, model_dim=256, head_dim=128, max_seq_len=4096, skip_attn_layers=(2,),
                     num_value_embeds=1)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", choices=["fused", "fused_allreduce", "nccl"], default="fused",
                    help="fused: peer-memory Muon + sharded Adam kernels; fused_allreduce: peer-memory Muon, bucket all-reduce + "
                         "replicated Adam; nccl: NCCL collectives")
    ap.add_argument("--full", action="store_true", help="the 124M model on 48 x 1024 tokens per rank (the benchmark's step) instead of the small one")
    ap.add_argument("--steps", type=int, default=STEPS)
    ap.add_argument("--pool", type=int, default=1, help="number of distinct sequences per rank, used in rotation (1: the same sequence every step)")
    ap.add_argument("--free-running", action="store_true", help="do not read the loss back between steps (the host runs ahead of the device)")
    a = ap.parse_args()
    global T
    steps, window = a.steps, 2
    if a.full:
        T, window = 48 * 1024, 14
    os.environ["B200_SHARDED_ADAM"] = "1" if a.mode == "fused" else "0"
    from ml_experiments_b200.ops.runtime import check_status
    from ml_experiments_b200.trainers.gpt_trainer import GPTTrainer, Hyperparameters, init_distributed, synthetic_batch

    rank, local, world = init_distributed()
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    batches = [[synthetic_batch(T, doc_len=1024 if a.full else 512, seed=50 + r + 1000 * i, pin=False) for i in range(a.pool)] for r in range(world)]
    batches = [[(x.to(dev), y.to(dev)) for x, y in b] for b in batches]
    cfg = (lambda: __import__("ml_experiments_b200.models.gpt", fromlist=["GPTConfig"]).GPTConfig(max_seq_len=T)) if a.full else _cfg
    # the model starts with a zero head and zero output projections: the first step moves only the head, the later ones
    # every parameter group
    tr = GPTTrainer(cfg(), Hyperparameters(seq_len=T), device=dev, rank=rank, world_size=world, seed=0,
                    grad_sync="nccl" if a.mode == "nccl" else "fused")
    assert tr.comm_mode == ("nccl" if a.mode == "nccl" else "fused-p2p"), tr.comm_mode
    assert tr.sharded_adam == (a.mode == "fused")
    mine = batches[rank]
    if a.free_running:
        losses = [float(l) for l in [tr.train_step(*mine[i % a.pool], window=window) for i in range(steps)]]
    else:
        losses = [float(tr.train_step(*mine[i % a.pool], window=window)) for i in range(steps)]
    check_status()
    mean_losses = torch.tensor(losses, device=dev, dtype=torch.float64)
    dist.all_reduce(mean_losses, op=dist.ReduceOp.AVG)
    params = {n: p.detach().float().clone() for n, p in tr.model.named_parameters()}
    # every rank must hold the same replica
    for n, p in params.items():
        q = p.clone()
        dist.broadcast(q, 0)
        assert torch.equal(p, q), f"rank {rank}: replica of {n} differs from rank 0"
    ok, worst = True, ("", 0.0)
    if rank == 0:
        single = GPTTrainer(cfg(), Hyperparameters(seq_len=T), device=dev, rank=0, world_size=1, seed=0)
        ref_losses = [float(single.train_step([b[i % a.pool][0] for b in batches], [b[i % a.pool][1] for b in batches], window=window))
                      for i in range(steps)]
        rels = []
        for n, p in single.model.named_parameters():
            d = (params[n] - p.detach().float()).norm().item()
            # relative to the distance the parameter moved (weights start at identical values): the two runs differ by
            # summation order of the gradient average (fp32 / bf16 buckets) amplified by bf16 Newton-Schulz
            moved = max((p.detach().float()).norm().item(), 1e-6)
            rel = d / moved
            rels.append((round(rel, 4), n))
            if rel > worst[1]:
                worst = (n, rel)
            # Muon matrices that start at zero (the output projections) have moved only a few orthogonalised steps: bf16
            # Newton-Schulz turns last-bit differences of the averaged gradient into a few percent of that small norm
            if rel > (8e-2 if p.ndim >= 2 and "embed" not in n and "lm_head" not in n else 3e-2):
                ok = False
        loss_gap = max(abs(u - v) for u, v in zip(mean_losses.tolist(), ref_losses))
        ok = ok and loss_gap < 5e-3 and ref_losses[-1] < ref_losses[0]        # measured gap: 1e-4
        print(json.dumps({"mode": a.mode, "world": world, "ok": ok, "losses": mean_losses.tolist(), "single_losses": ref_losses,
                          "worst_param": worst[0], "worst_rel": worst[1], "worst5": sorted(rels, reverse=True)[:5]}), flush=True)
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.broadcast(flag, 0)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
