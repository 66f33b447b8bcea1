"""NorMuon / Adam update rules and the combined optimizer (CPU, single process) + a 2-rank gloo equivalence check."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ml_experiments_b200.optim.normuon import (DistAdam, NorMuon, NorMuonAndAdam, adam_cautious_, cautious_update_,
                                               normuon_variance_reduction, polar_express)


def test_polar_express_orthogonalises():
    torch.manual_seed(0)
    for shape in ((64, 64), (32, 96), (96, 32), (3, 48, 48)):
        X = polar_express(torch.randn(*shape)).float()
        s = torch.linalg.svdvals(X)
        assert s.max() < 1.35 and s.flatten().quantile(0.1) > 0.6, (shape, s.min().item(), s.max().item())


def test_variance_reduction_keeps_norm():
    torch.manual_seed(1)
    v = torch.randn(2, 16, 48)
    buf = torch.zeros(2, 16, 1)
    out = normuon_variance_reduction(v.clone(), buf, 0.95, -1)
    assert torch.allclose(out.norm(dim=(-2, -1)), v.norm(dim=(-2, -1)), rtol=1e-4)
    assert (buf > 0).all()


def test_mantissa_update_is_fp32_exact():
    torch.manual_seed(2)
    ref = torch.randn(64, 64)
    p = ref.bfloat16()
    exact_bits = ref.view(torch.int32)
    mant = (exact_bits & 0xFFFF).clone()
    p = ((exact_bits >> 16).to(torch.int16)).view(torch.bfloat16).clone()
    for _ in range(50):
        upd = torch.randn(64, 64) * 1e-3
        cautious_update_(p, mant, upd, lr=0.1, wd_lr=0.001)
        ref = ref - ref * ((upd * ref) >= 0) * 0.001 - upd * 0.1
    recon = ((p.view(torch.int16).to(torch.int32) << 16) | (mant & 0xFFFF)).view(torch.float32)
    assert torch.allclose(recon, ref, atol=1e-6)


def test_adam_cautious_matches_formula():
    p, g = torch.tensor([1.0, -2.0, 0.5]), torch.tensor([0.1, 0.2, -0.3])
    m, v = torch.zeros(3), torch.zeros(3)
    adam_cautious_(p, g, m, v, 0.9, 0.99, 1e-10, 0.01, 0.001)
    upd = (0.1 * g) / ((0.01 * g * g).sqrt() + 1e-10) * 0.01
    p0 = torch.tensor([1.0, -2.0, 0.5])
    want = p0 - (upd + p0 * ((upd * p0) > 0) * 0.001)
    assert torch.allclose(p, want, atol=1e-7)


def _make():
    torch.manual_seed(3)
    params = {"attn": torch.nn.Parameter(torch.randn(4, 32, 32) * 0.1), "mlp": torch.nn.Parameter(torch.randn(4, 64, 32) * 0.1),
              "embed": torch.nn.Parameter(torch.randn(64, 32) * 0.1), "scalars": torch.nn.Parameter(torch.ones(8))}
    table = {"attn": dict(optim="normuon", comms="sharded"), "mlp": dict(optim="normuon", comms="sharded", per_matrix_lr_mul=[1, 2, 1, 2]),
             "embed": dict(optim="adam", comms="sharded", adam_betas=(0.5, 0.95)), "scalars": dict(optim="adam", comms="replicated", lr_mul=5.0, wd_mul=0.0)}
    return params, table


def test_combined_optimizer_single_process():
    params, table = _make()
    opt = NorMuonAndAdam(params.items(), table, scatter_order=["scalars", "embed", "attn", "mlp"], work_order=["scalars", "attn", "mlp", "embed"])
    before = {k: v.detach().clone() for k, v in params.items()}
    for step in range(3):
        for p in params.values():
            p.grad = torch.randn_like(p)
        opt.step(do_adam=(step % 2 == 1))
    assert not torch.equal(params["attn"], before["attn"]) and not torch.equal(params["mlp"], before["mlp"])
    assert not torch.equal(params["embed"], before["embed"])
    sd = opt.state_dict()
    assert set(sd) >= {"param_states", "param_cfgs"} and "momentum_buffer" in sd["param_states"]["attn"]
    opt.reset()
    assert float(opt.param_states["attn"]["momentum_buffer"].abs().sum()) == 0.0
    opt.load_state_dict(sd)
    assert float(opt.param_states["attn"]["momentum_buffer"].abs().sum()) > 0.0


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        params, table = _make()
        opt = NorMuonAndAdam(params.items(), table)
        g = torch.Generator().manual_seed(10)
        for _ in range(2):
            full = {k: torch.randn(world, *p.shape, generator=g) for k, p in params.items()}
            for k, p in params.items():
                p.grad = full[k][rank].clone()
            opt.step()
        if rank == 0:
            torch.save({k: p.detach().clone() for k, p in params.items()}, out)
        lin = torch.nn.Linear(2048, 4, bias=False)
        torch.manual_seed(0)
        a = DistAdam(lin.parameters(), lr=1e-2)
        lin(torch.randn(3, 2048, generator=torch.Generator().manual_seed(rank))).sum().backward()
        a.step()
        mats = [torch.nn.Parameter(torch.ones(16, 16) * 0.1) for _ in range(3)]
        nm = NorMuon(mats, lr=0.01)
        for m_ in mats:
            m_.grad = torch.randn(16, 16, generator=torch.Generator().manual_seed(rank))
        nm.step()
        flat = torch.cat([lin.weight.detach().reshape(-1)] + [m_.detach().reshape(-1) for m_ in mats])
        gathered = [torch.zeros_like(flat) for _ in range(world)]
        dist.all_gather(gathered, flat)
        assert torch.allclose(gathered[0], gathered[1], atol=1e-6)
    finally:
        dist.destroy_process_group()


def test_sharded_equals_single_process_on_mean_gradient(tmp_path):
    world = 2
    out = str(tmp_path / "p.pt")
    mp.spawn(_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    got = torch.load(out)
    params, table = _make()
    opt = NorMuonAndAdam(params.items(), table, world_size=1, rank=0)
    g = torch.Generator().manual_seed(10)
    for _ in range(2):
        full = {k: torch.randn(world, *p.shape, generator=g) for k, p in params.items()}
        for k, p in params.items():
            p.grad = full[k].mean(0)
        opt.step()
    for k in params:
        assert torch.allclose(got[k], params[k].detach(), atol=2e-3), (k, (got[k] - params[k]).abs().max())
