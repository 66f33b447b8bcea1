"""Run with ``python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 --master-port P
tests/multi_gpu/check_checkpoint_resume.py --dir DIR``.

Distributed checkpoint / resume over the fused peer-memory path (sharded Muon momentum, sharded Adam moments): every
rank trains the small GPT for ``K + M`` steps; a second trainer trains ``K`` steps, saves (every rank writes its shard),
is thrown away, and a third trainer loads the files and trains the remaining ``M`` steps. Losses of the resumed run and
every parameter afterwards have to match the uninterrupted run (same kernels, same inputs: only the summation order of
atomics differs). Prints one JSON line on rank 0 and exits non-zero on a mismatch.
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

K, M = 3, 3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--dir", required=True)
    a = ap.parse_args()
    from ml_experiments_b200.models.gpt import GPTConfig
    from ml_experiments_b200.ops.runtime import check_status
    from ml_experiments_b200.trainers.gpt_trainer import GPTTrainer, Hyperparameters, init_distributed, synthetic_batch

    rank, local, world = init_distributed()
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    cfg = lambda: GPTConfig(num_layers=4, num_heads=2, model_dim=256, head_dim=128, max_seq_len=4096, skip_attn_layers=(2,), num_value_embeds=1)
    make = lambda: GPTTrainer(cfg(), Hyperparameters(seq_len=2048), device=dev, rank=rank, world_size=world, seed=0, grad_sync="fused")
    x, y = (t.to(dev) for t in synthetic_batch(2048, doc_len=512, seed=50 + rank, pin=False))
    steps = lambda tr, n: [float(tr.train_step(x, y, window=2)) for _ in range(n)]

    full = make()
    assert full.comm_mode == "fused-p2p" and full.sharded_adam
    want = steps(full, K + M)
    first = make()
    head = steps(first, K)
    path = os.path.join(a.dir, "ck.pt")
    first.save_checkpoint(path)
    dist.barrier()
    del first
    resumed = make()
    resumed.load_checkpoint(path)
    assert resumed.step == K
    tail = steps(resumed, M)
    check_status()
    got = head + tail
    gap = max(abs(u - v) for u, v in zip(got, want))
    worst = ("", 0.0)
    for (n, p), q in zip(resumed.model.named_parameters(), full.model.parameters()):
        rel = ((p.detach().float() - q.detach().float()).norm() / q.detach().float().norm().clamp_min(1e-6)).item()
        if rel > worst[1]:
            worst = (n, rel)
    # the two runs execute the same kernels on the same data; what differs is the order of fp32 atomics (embedding
    # scatter, split-K reductions) amplified by bf16 Newton-Schulz on the freshly initialised projections
    ok = gap < 5e-3 and worst[1] < 8e-2 and want[-1] < want[0]
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(json.dumps({"world": world, "ok": bool(flag.item()), "loss_gap": gap, "worst_param": worst[0], "worst_rel": worst[1],
                          "losses": got, "uninterrupted": want}), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
