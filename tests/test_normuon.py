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


def _reference_adam_step(p, g, m, v, beta1, beta2, eps, step_size, eff_wd):
    """The reference's compiled Adam update (modded-nanogpt/train_gpt.py:683-691), restated line by line."""
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    update = m.div(v.sqrt().add_(eps)).mul_(step_size)
    mask = (update * p) > 0
    update.addcmul_(p, mask, value=eff_wd)
    p.add_(other=update, alpha=-1.0)


def test_adam_weight_decay_follows_lr_squared_schedule():
    """eff_wd = (lr * lr_mul)**2 * weight_decay * wd_mul in the combined optimizer (modded-nanogpt/train_gpt.py:658-672)
    and lr * wd * wd_mul * lr with lr = group lr * param.lr_mul in DistAdam (train_gpt_medium.py:805-826)."""
    torch.manual_seed(5)
    lr, wd, lr_mul, wd_mul, betas = 0.008, 0.005, 5.0, 3.0, (0.65, 0.95)
    p0 = torch.randn(64, 8)
    grads = [torch.randn(64, 8) for _ in range(3)]
    # combined optimizer
    p = torch.nn.Parameter(p0.clone())
    opt = NorMuonAndAdam([("x", p)], {"x": dict(optim="adam", comms="none", adam_betas=betas, lr_mul=lr_mul, wd_mul=wd_mul)},
                         adam_defaults=None, world_size=1, rank=0)
    ref, m, v = p0.clone(), torch.zeros_like(p0), torch.zeros_like(p0)
    for t, g in enumerate(grads, 1):
        p.grad = g.clone()
        opt.step()
        l = lr * lr_mul
        _reference_adam_step(ref, g, m, v, betas[0], betas[1], 1e-10, l * ((1 - betas[1] ** t) ** 0.5 / (1 - betas[0] ** t)),
                             l * l * wd * wd_mul)
    assert torch.allclose(p.detach(), ref, atol=1e-6), (p.detach() - ref).abs().max()
    # DistAdam honours p.lr_mul / p.wd_mul
    q = torch.nn.Parameter(p0.clone())
    q.lr_mul, q.wd_mul = lr_mul, wd_mul
    da = DistAdam([q], lr=lr, betas=betas, eps=1e-10, weight_decay=wd)
    ref, m, v = p0.clone(), torch.zeros_like(p0), torch.zeros_like(p0)
    for t, g in enumerate(grads, 1):
        q.grad = g.clone()
        da.step()
        l = lr * lr_mul
        _reference_adam_step(ref, g, m, v, betas[0], betas[1], 1e-10, l * ((1 - betas[1] ** t) ** 0.5 / (1 - betas[0] ** t)),
                             l * wd * wd_mul * l)
    assert torch.allclose(q.detach(), ref, atol=1e-6), (q.detach() - ref).abs().max()


def test_normuon_decay_is_scaled_by_the_effective_lr():
    """p -= p * mask * (wd_mul * wd * lr) * lr_eff + v * lr_eff (modded-nanogpt/train_gpt.py:708-760)."""
    torch.manual_seed(6)
    p0 = torch.randn(2, 16, 16) * 0.3
    p = torch.nn.Parameter(p0.clone())
    opt = NorMuonAndAdam([("w", p)], {"w": dict(optim="normuon", comms="none", lr=0.02, weight_decay=1.5, lr_mul=2.0, wd_mul=0.5)},
                         world_size=1, rank=0)
    g = torch.randn_like(p0)
    p.grad = g.clone()
    opt.step()
    mom = torch.zeros_like(g).lerp_(g, 1 - 0.95)
    u = g.lerp(mom, 0.95)
    v = normuon_variance_reduction(polar_express(u), torch.zeros(2, 16, 1), 0.95, -1).float()
    lr_eff = 0.02 * 2.0
    want = p0 - p0 * ((v * p0) >= 0) * (0.5 * 1.5 * 0.02) * lr_eff - v * lr_eff
    assert torch.allclose(p.detach(), want, atol=1e-6), (p.detach() - want).abs().max()


def test_bank_reshape_hint_and_per_matrix_rates():
    """A bank parameter carries its optimizer view as a tuple attribute named ``reshape`` (the reference's convention,
    modded-nanogpt/train_gpt.py:1125); per-matrix multipliers index the leading axis of THAT view: with [1, 2] per layer
    the second matrix of every layer (the output projection) moves twice as far."""
    torch.manual_seed(7)
    p = torch.nn.Parameter(torch.zeros(3, 2, 16, 8))
    p.reshape = (6, 16, 8)
    opt = NorMuonAndAdam([("mlp", p)], {"mlp": dict(optim="normuon", comms="none", lr=0.02, weight_decay=0.0, per_matrix_lr_mul=[1.0, 2.0] * 3)},
                         world_size=1, rank=0)
    assert opt.cfgs["mlp"].reshape == (6, 16, 8)
    p.grad = torch.randn(3, 2, 16, 8)
    opt.step()
    moved = p.detach().view(6, -1).norm(dim=1)
    ratio = moved[1::2] / moved[0::2]
    assert torch.allclose(ratio, torch.full((3,), 2.0), rtol=0.15), ratio
