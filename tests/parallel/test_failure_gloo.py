"""Failure detection and recovery with CPU ranks (gloo) and faults injected on the host."""
import os
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ml_experiments_b200.runtime import DroppingStore, FaultPlan, Heartbeat, InjectedFault, RankFailure, StepWatchdog, run_with_recovery
from ml_experiments_b200.utils import checkpoint as C


def _free_port_pair() -> int:
    """A port p such that p and p + 1 are both free right now (rendezvous and heartbeat store)."""
    import socket
    for _ in range(50):
        with socket.socket() as a:
            a.bind(("127.0.0.1", 0))
            p = a.getsockname()[1]
            with socket.socket() as b:
                try:
                    b.bind(("127.0.0.1", p + 1))
                    return p
                except OSError:
                    continue
    raise RuntimeError("no free port pair")


def _worker(rank, world, port, tmp, plan_kind):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=__import__("datetime").timedelta(seconds=20))
    store = dist.TCPStore("127.0.0.1", port + 1, world, is_master=(rank == 0), timeout=__import__("datetime").timedelta(seconds=20))
    hb = Heartbeat(store, rank, world, timeout=6.0)   # well above a step (all-reduce + checkpoint write) on a loaded host
    plan = {"raise": FaultPlan(raise_at={1: 3}), "exit": FaultPlan(exit_at={1: 3})}[plan_kind]
    w = torch.zeros(4)
    outcome = "done"
    try:
        for step in range(6):
            try:
                plan.before_step(rank, step)
            except InjectedFault as e:
                hb.mark_failed(str(e))
                raise
            hb.beat(step)
            hb.wait_all_at(step)            # peers learn of a failure here, before any collective is entered
            g = torch.full((4,), float(rank + 1))
            dist.all_reduce(g)
            w += g
            if rank == 0:
                C.save_checkpoint({"step": step + 1, "w": w.clone()}, os.path.join(tmp, "ck.pt"))
    except RankFailure as e:
        outcome = f"detected:{e.rank}"
    except InjectedFault:
        outcome = "injected"
    with open(os.path.join(tmp, f"out{rank}.txt"), "w") as f:
        f.write(outcome)
    if rank == 0:
        # the store lives in this process: keep it up until the other survivors have read the failure from it
        deadline = time.time() + 30
        while time.time() < deadline and not all(os.path.exists(os.path.join(tmp, f"out{r}.txt")) for r in range(world) if r != 1):
            time.sleep(0.05)
    # no collective on the way out: the failed rank is gone
    os._exit(0)


@pytest.mark.parametrize("kind", ["raise", "exit"])
def test_peers_detect_failed_rank_before_next_collective(tmp_path, kind):
    port = _free_port_pair()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_worker, args=(r, 3, port, str(tmp_path), kind)) for r in range(3)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert not p.is_alive(), "a rank hung after a peer failed"
    outs = {r: (tmp_path / f"out{r}.txt").read_text() if (tmp_path / f"out{r}.txt").exists() else None for r in range(3)}
    assert outs[0] == "detected:1" and outs[2] == "detected:1"
    assert outs[1] == ("injected" if kind == "raise" else None)      # the exiting rank wrote nothing
    ck = C.load_checkpoint(tmp_path / "ck.pt")
    assert ck["step"] == 3 and torch.equal(ck["w"], torch.full((4,), 18.0))  # 3 completed steps of 1 + 2 + 3


def test_recovery_restarts_from_last_checkpoint(tmp_path):
    path = tmp_path / "ck.pt"
    C.save_checkpoint({"step": 0, "w": torch.zeros(2)}, path)
    failures = iter([4, None])

    def train(state):
        fail_at = next(failures)
        for step in range(state["step"], 8):
            if step == fail_at:
                raise RankFailure(1, "injected")
            state = {"step": step + 1, "w": state["w"] + 1}
            if (step + 1) % 2 == 0:
                C.save_checkpoint(state, path)
        return state

    restarts = []
    final = run_with_recovery(train, lambda: C.load_checkpoint(path), max_restarts=2, on_restart=lambda n, e: restarts.append((n, e.rank)))
    assert final["step"] == 8 and torch.equal(final["w"], torch.full((2,), 8.0)) and restarts == [(1, 1)]
    with pytest.raises(RankFailure):
        run_with_recovery(lambda s: (_ for _ in ()).throw(RankFailure(0, "always")), lambda: {}, max_restarts=1)


def test_heartbeat_timeout_dropped_messages_and_watchdog():
    store = dist.HashStore()
    a, b = Heartbeat(store, 0, 2, timeout=0.3), Heartbeat(DroppingStore(store, lambda k: "beat" in k), 1, 2, timeout=0.3)
    a.beat(0)
    b.beat(0)                      # dropped on the way: rank 1 looks silent
    a.check()                      # still within the start-up grace period
    time.sleep(0.4)
    with pytest.raises(RankFailure, match="no heartbeat"):
        a.check()
    c = Heartbeat(store, 1, 2, timeout=0.3)
    c.beat(5)
    a.check()
    time.sleep(0.4)
    with pytest.raises(RankFailure, match="step 5"):
        a.check()
    fired = []
    wd = StepWatchdog(0.2, on_timeout=fired.append, heartbeat=c)
    with wd.step():
        time.sleep(0.05)
    assert not wd.expired
    with wd.step():
        time.sleep(0.5)
    wd.close()
    assert wd.expired and fired == [0.2]
    with pytest.raises(RankFailure, match="reported failure"):
        a.check()
