"""Run with ``python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 --master-port P
tests/multi_gpu/check_failure_between_steps.py --out DIR``.

Every rank trains the small GPT over the fused peer-memory path. The last rank fails on the host before step
``FAIL_AT`` (an exception raised between two steps, after its device is idle), records the failure in the heartbeat store
and leaves. The other ranks learn of it at the heartbeat rendezvous BEFORE they launch the step's kernels (a kernel that
waits for the dead rank's flag would otherwise spin until its time limit), stop, and report which rank failed. No
collective is entered after the failure and nobody waits on the device for a rank that is gone.
"""
import argparse
import datetime
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

FAIL_AT = 3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", required=True)
    a = ap.parse_args()
    from ml_experiments_b200.models.gpt import GPTConfig
    from ml_experiments_b200.ops.runtime import check_status
    from ml_experiments_b200.runtime import FaultPlan, Heartbeat, InjectedFault, RankFailure
    from ml_experiments_b200.trainers.gpt_trainer import GPTTrainer, Hyperparameters, init_distributed, synthetic_batch

    rank, local, world = init_distributed()
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    store = dist.TCPStore("127.0.0.1", int(os.environ["MASTER_PORT"]) + 1, world, is_master=(rank == 0),
                          timeout=datetime.timedelta(seconds=30))
    hb = Heartbeat(store, rank, world, timeout=20.0)
    plan = FaultPlan(raise_at={world - 1: FAIL_AT})
    cfg = GPTConfig(num_layers=4, num_heads=2, model_dim=256, head_dim=128, max_seq_len=4096, skip_attn_layers=(2,), num_value_embeds=1)
    tr = GPTTrainer(cfg, Hyperparameters(seq_len=2048), device=dev, rank=rank, world_size=world, seed=0, grad_sync="fused")
    x, y = (t.to(dev) for t in synthetic_batch(2048, doc_len=512, seed=50 + rank, pin=False))
    outcome, losses = "done", []
    try:
        for step in range(6):
            torch.cuda.synchronize()                 # a rank only ever leaves with an idle device
            try:
                plan.before_step(rank, step)
            except InjectedFault as e:
                hb.mark_failed(str(e))
                raise
            hb.beat(step)
            hb.wait_all_at(step)                     # peers learn of a failure here, before any kernel of the step
            losses.append(float(tr.train_step(x, y, window=2)))
        check_status()
    except RankFailure as e:
        outcome = f"detected:{e.rank}"
    except InjectedFault:
        outcome = "injected"
    torch.cuda.synchronize()
    check_status()                                   # no wait ran out: nobody launched a step the failed rank never joined
    with open(os.path.join(a.out, f"out{rank}.txt"), "w") as f:
        f.write(f"{outcome} steps={len(losses)} first={losses[0]:.3f} last={losses[-1]:.3f}")
    if rank == 0:                                    # the store lives here: keep it up until the survivors have read it
        deadline = time.time() + 30
        while time.time() < deadline and not all(os.path.exists(os.path.join(a.out, f"out{r}.txt")) for r in range(world - 1)):
            time.sleep(0.05)
    os._exit(0)                                      # no collective on the way out: a rank is gone


if __name__ == "__main__":
    main()
