"""Fused peer-memory collectives, exercised on one GPU with virtual ranks.

Every rank's producer phase is launched before any consumer phase, so no kernel waits for a later launch."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu
W = 4


def test_allreduce_mean_virtual_ranks():
    from ml_experiments_b200.ops.runtime import check_status, ops, status
    from ml_experiments_b200.parallel.symm import VirtualWorld

    vw = VirtualWorld(W)
    o = ops()
    for dtype, code, n in ((torch.float32, 0, 4 * W * 1000 + 4 * W), (torch.bfloat16, 1, 8 * W * 777)):
        bufs = vw.alloc(n, dtype)
        torch.manual_seed(0)
        for b in bufs:
            b.local.copy_(torch.randn(n, device="cuda").to(dtype))
        ref = torch.stack([b.local.float() for b in bufs]).mean(0)
        ch = 2 if code else 4
        for r, w in enumerate(vw.worlds):
            o.comm_signal(w.flags.ptrs, r, ch, 1, w.flags.local)
        for r, w in enumerate(vw.worlds):
            o.allreduce_mean(bufs[r].ptrs, r, n, code, w.flags.local, w.flags.ptrs, ch, 1, status())
        for r, w in enumerate(vw.worlds):
            o.comm_wait(w.flags.local, W, ch + 1, 1, status())
        check_status()
        tol = 1e-6 if code == 0 else 1e-2
        for b in bufs:
            assert torch.allclose(b.local.float(), ref, atol=tol, rtol=tol)


def test_wait_times_out_cleanly():
    """A wait on a flag that nobody sets really runs out (limit shortened to 1 ms), reports code 5 through the status
    word, and the context stays usable. Nothing is poisoned beforehand: the expiry branch itself is what runs."""
    from ml_experiments_b200.ops.runtime import check_status, ops, set_peer_wait_limit_ms, status
    from ml_experiments_b200.parallel.symm import VirtualWorld

    vw = VirtualWorld(2)
    st = status()
    check_status()
    set_peer_wait_limit_ms(1.0)
    try:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        ops().comm_wait(vw.worlds[0].flags.local, 2, 6, 123, st)
        e1.record()
        torch.cuda.synchronize()
        assert 0.5 < e0.elapsed_time(e1) < 500.0          # it waited about a millisecond, not 0 and not 5 s
        with pytest.raises(RuntimeError, match="peer flag"):
            check_status()
        check_status()  # cleared by the failed check
        # a second wait after the failure was cleared times out again on its own (no sticky state)
        ops().comm_wait(vw.worlds[0].flags.local, 2, 6, 124, st)
        with pytest.raises(RuntimeError, match="peer flag"):
            check_status()
    finally:
        set_peer_wait_limit_ms(None)
    assert torch.ones(4, device="cuda").sum().item() == 4


def test_poisoned_status_makes_waits_return_at_once():
    from ml_experiments_b200.ops.runtime import check_status, ops, status
    from ml_experiments_b200.parallel.symm import VirtualWorld

    vw = VirtualWorld(2)
    st = status()
    st[0] = 9
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    ops().comm_wait(vw.worlds[0].flags.local, 2, 6, 123, st)
    e1.record()
    torch.cuda.synchronize()
    assert e0.elapsed_time(e1) < 100.0
    with pytest.raises(RuntimeError):
        check_status()
    check_status()


def test_fused_muon_matches_single_process():
    from ml_experiments_b200.ops.newton_schulz import NS5_COEFFS
    from ml_experiments_b200.ops.runtime import check_status
    from ml_experiments_b200.optim import Muon
    from ml_experiments_b200.parallel.muon_dist import MuonShardEngine
    from ml_experiments_b200.parallel.symm import VirtualWorld

    torch.manual_seed(0)
    shapes = [(3, 256, 256), (256, 256), (256, 256), (1024, 256), (256, 1024), (256, 1024)]
    base = [torch.randn(s, device="cuda") * 0.02 for s in shapes]
    vw = VirtualWorld(W)
    rank_params = [[b.clone().requires_grad_(True) for b in base] for _ in range(W)]
    engines = [MuonShardEngine(rank_params[r], vw.worlds[r], alloc=vw.allocator(r)) for r in range(W)]
    ref_params = [b.clone().requires_grad_(True) for b in base]
    ref = Muon(ref_params, lr=0.05, momentum=0.95)
    for step in range(2):
        grads = [[torch.randn(s, device="cuda") for s in shapes] for _ in range(W)]
        for r in range(W):
            for p, g in zip(rank_params[r], grads[r]):
                p.grad = g
        for p, *gs in zip(ref_params, *grads):
            p.grad = torch.stack(gs).mean(0)
        ref.step()
        for e in engines:
            e.publish_grads()
        for e in engines:
            e.reduce_ns_push(0.95, True, [NS5_COEFFS[0]] * 5)
        for e in engines:
            e.apply(0.05)
        check_status()
    from ml_experiments_b200.utils.shadow import shadow_of

    for r in range(W):
        for p, q in zip(rank_params[r], ref_params):
            assert (p.detach() - q.detach()).abs().max().item() < 2e-2
            assert torch.equal(shadow_of(p, torch.bfloat16), p.detach().bfloat16())
    for p0, p1 in zip(rank_params[0], rank_params[W - 1]):
        assert torch.equal(p0.detach(), p1.detach())  # replicas stay bit-identical


def test_sharded_adam_virtual_ranks_match_torch_adam():
    """Fused reduce-scatter + Adam + all-gather on 4 virtual ranks against ``torch.optim.Adam`` on the mean gradient."""
    from ml_experiments_b200.ops.runtime import check_status
    from ml_experiments_b200.parallel.adam_dist import ShardedAdam
    from ml_experiments_b200.parallel.symm import VirtualWorld

    vw = VirtualWorld(W)
    torch.manual_seed(0)
    shapes = [((300, 64), torch.bfloat16, 0), ((257, 40), torch.float32, 1), ((7,), torch.float32, 2), ((5,), torch.float32, 2)]
    base = [torch.randn(*s, device="cuda").to(dt) for s, dt, _ in shapes]
    lrs = [0.3, 0.01, 0.04]
    ranks = []
    for r in range(W):
        ps = [b.clone().requires_grad_(True) for b in base]
        groups = [dict(params=[p for p, (_, _, g) in zip(ps, shapes) if g == gi], lr=lrs[gi]) for gi in range(3)]
        opt = ShardedAdam(groups, vw.worlds[r], betas=(0.8, 0.95), eps=1e-10, alloc=vw.allocator(r), pack_below=1024)
        ranks.append((ps, opt))
    ref = [b.clone().float().requires_grad_(True) for b in base]
    ref_opt = torch.optim.Adam([dict(params=[p for p, (_, _, g) in zip(ref, shapes) if g == gi], lr=lrs[gi]) for gi in range(3)],
                               betas=(0.8, 0.95), eps=1e-10)
    nseg = len(ranks[0][1].segments)
    assert nseg == 3      # the two small fp32 vectors share a segment
    for step in range(3):
        grads = [[torch.randn_like(b.float()).to(b.dtype) for b in base] for _ in range(W)]
        for r, (ps, opt) in enumerate(ranks):
            for p, g in zip(ps, grads[r]):
                # half of the gradients are written straight into their bucket views, the others are staged by the optimizer
                view = opt.grad_views[id(p)]
                if p.ndim == 2:
                    view.copy_(g)
                    p.grad = view
                else:
                    p.grad = g.clone()
        for i in range(nseg):             # every rank announces before any rank's kernel waits
            for _, opt in ranks:
                opt.publish(i)
            for _, opt in ranks:
                opt.reduce(i)
        for _, opt in ranks:
            opt.finish()
        check_status()
        for p, gs in zip(ref, zip(*grads)):
            p.grad = torch.stack([g.float() for g in gs]).mean(0)
        ref_opt.step()
        for r, (ps, _) in enumerate(ranks):
            for p, q, (_, dt, _) in zip(ps, ref, shapes):
                assert p.grad is None
                if dt == torch.float32:
                    assert torch.allclose(p.detach(), q.detach(), atol=2e-6, rtol=1e-5), (r, step)
                else:   # bf16 master parameters: the kernel rounds the parameter each step, the oracle does not
                    assert torch.allclose(p.detach().float(), q.detach(), atol=0.03, rtol=0.02), (r, step, (p.detach().float() - q.detach()).abs().max())
    # replicas are bit-identical across ranks and the moments exist only for the owned slice
    for ps, opt in ranks[1:]:
        for p, p0 in zip(ps, ranks[0][0]):
            assert torch.equal(p.detach(), p0.detach())
    seg = ranks[0][1].segments[0]
    assert seg.m.numel() == seg.numel // W
