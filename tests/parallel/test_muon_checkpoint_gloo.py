"""Distributed Muon on CPU ranks (gloo): the sharded momentum survives a checkpoint, a killed run that resumes from
it ends with the parameters of the uninterrupted run, and a checkpoint written by 2 ranks loads into 1 rank."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

SHAPES = [(3, 16, 16), (16, 16), (32, 16), (16, 32)]      # 4 matrices of 16x16 (stack padded for 3 ranks), 1 + 1 others
STEPS, CUT = 4, 2


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _grads(step, world):
    g = torch.Generator().manual_seed(100 + step)
    return [torch.randn(world, *s, generator=g) for s in SHAPES]


def _params():
    torch.manual_seed(4)
    return [torch.nn.Parameter(torch.randn(*s) * 0.2) for s in SHAPES]


def _make_opt(ps, rank, world):
    from ml_experiments_b200.parallel.muon_dist import DistMuon, GradSync

    comm = GradSync(torch.nn.ParameterList(ps), ps, rank, world)
    return DistMuon(ps, comm, lr=0.05, momentum=0.9)


def _run(ps, opt, rank, world, steps, grad_world):
    for step in steps:
        for p, g in zip(ps, _grads(step, grad_world)):
            # with fewer ranks than the run that produced the data, feed the mean (what the averaging would give)
            p.grad = g[rank].clone() if world == grad_world else g.mean(0)
        opt.step()


def _worker(rank, world, port, tmp, mode):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from ml_experiments_b200.utils.checkpoint import load_sharded, save_sharded

        ps = _params()
        opt = _make_opt(ps, rank, world)
        ck = os.path.join(tmp, "ck.pt")
        if mode == "full":
            _run(ps, opt, rank, world, range(STEPS), 2)
        elif mode == "first_half":          # the run that is "killed" after CUT steps: it only leaves its checkpoint behind
            _run(ps, opt, rank, world, range(CUT), 2)
            save_sharded({"params": [p.detach().clone() for p in ps]}, opt.sharded_state(), ck, rank, world, opt.sharded_rows())
            return
        elif mode == "resume":
            rep, shard = load_sharded(ck, rank, world)
            with torch.no_grad():
                for p, q in zip(ps, rep["params"]):
                    p.copy_(q)
            opt.load_sharded_state(shard)
            _run(ps, opt, rank, world, range(CUT, STEPS), 2)
        if rank == 0:
            torch.save([p.detach().clone() for p in ps], os.path.join(tmp, f"{mode}_{world}.pt"))
    finally:
        dist.destroy_process_group()


def test_killed_run_resumes_to_the_same_parameters(tmp_path):
    tmp = str(tmp_path)
    mp.spawn(_worker, args=(2, _free_port(), tmp, "full"), nprocs=2, join=True)
    mp.spawn(_worker, args=(2, _free_port(), tmp, "first_half"), nprocs=2, join=True)
    assert os.path.exists(os.path.join(tmp, "ck.pt.rank1"))          # every rank wrote its momentum slice
    mp.spawn(_worker, args=(2, _free_port(), tmp, "resume"), nprocs=2, join=True)
    full, res = torch.load(os.path.join(tmp, "full_2.pt")), torch.load(os.path.join(tmp, "resume_2.pt"))
    for a, b in zip(full, res):
        assert torch.allclose(a, b, atol=1e-6), (a - b).abs().max()
    # without the momentum the resumed run would differ by about lr * (orthogonal update) ~ 5e-2 per element
    # the same checkpoint into ONE rank (re-partitioned, padding dropped): same parameters up to bf16 Newton-Schulz order
    mp.spawn(_worker, args=(1, _free_port(), tmp, "resume"), nprocs=1, join=True)
    one = torch.load(os.path.join(tmp, "resume_1.pt"))
    for a, b in zip(full, one):
        assert torch.allclose(a, b, atol=2e-3), (a - b).abs().max()
