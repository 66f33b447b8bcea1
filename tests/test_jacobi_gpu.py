"""Fused MIMO-Jacobi iteration kernel (forward and backward) against the plain PyTorch loop in fp32."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(b, R, L, N, seed, strided):
    g = torch.Generator(device="cuda").manual_seed(seed)
    rn = lambda *s: torch.randn(*s, device="cuda", generator=g)
    if strided:  # the layout the module produces: a [b, L, N, R] projection viewed as [b, R, L, N]
        Bm, Cm = rn(b, L, N, R).permute(0, 3, 1, 2), rn(b, L, N, R).permute(0, 3, 1, 2)
        xr = rn(b, L, R).permute(0, 2, 1)
    else:
        Bm, Cm, xr = rn(b, R, L, N), rn(b, R, L, N), rn(b, R, L)
    theta = rn(b, L, N // 2)
    alpha, gamma = torch.sigmoid(rn(b, L, N)), torch.sigmoid(rn(b, L))
    conv_w, conv_b = rn(N, 3) * 0.4, rn(N) * 0.1
    return [Bm, Cm, theta, xr, alpha, gamma, conv_w, conv_b]


@pytest.mark.parametrize("N,R,L,n_iters,mix,strided", [
    (64, 4, 300, 12, False, True),       # the module's defaults; three windows of the forward, eight of the backward
    (64, 2, 97, 5, True, False),         # sum / difference mixes, ragged length
    (16, 3, 700, 3, True, True),
    (32, 1, 64, 1, False, False),        # a single iteration: no halo
    (128, 2, 150, 12, True, True),
])
def test_forward_and_backward_match_torch(N, R, L, n_iters, mix, strided):
    from ml_experiments_b200.ops.jacobi_iter import jacobi_iterate, jacobi_iterate_torch, kernel_supported

    assert kernel_supported(N, n_iters)
    b = 2
    base = _inputs(b, R, L, N, seed=N + L, strided=strided)
    lams = [torch.tensor(0.5, device="cuda"), torch.tensor(0.3, device="cuda")] if mix else [None, None]
    outs = []
    for fn in (jacobi_iterate_torch, jacobi_iterate):
        # strided views must stay views: the leaves are their storage-order parents
        args, leaves = list(base), []
        for i, t in enumerate(base):
            if strided and i in (0, 1):
                leaf = t.permute(0, 2, 3, 1).contiguous().detach().requires_grad_(True)
                args[i] = leaf.permute(0, 3, 1, 2)
            elif strided and i == 3:
                leaf = t.permute(0, 2, 1).contiguous().detach().requires_grad_(True)
                args[i] = leaf.permute(0, 2, 1)
            else:
                leaf = t.detach().clone().requires_grad_(True)
                args[i] = leaf
            leaves.append(leaf)
        ls = [None if l is None else l.detach().clone().requires_grad_(True) for l in lams]
        y = fn(*args, ls[0], ls[1], n_iters)
        w = torch.randn(y.shape, device="cuda", generator=torch.Generator(device="cuda").manual_seed(7))
        (y * w).sum().backward()
        outs.append((y.detach(), [l.grad for l in leaves] + [l.grad for l in ls if l is not None]))
    (y0, g0), (y1, g1) = outs
    rel = lambda a, b_: ((a - b_).norm() / b_.norm().clamp_min(1e-12)).item()
    assert rel(y1, y0) < 2e-4, rel(y1, y0)
    names = ["B", "C", "theta", "x_r", "alpha", "gamma", "taps", "bias", "lam_inject", "lam_readout"]
    for name, a, b_ in zip(names, g1, g0):
        if b_ is None:      # an input the loop never touched (gamma with a single iteration)
            assert a is None or float(a.abs().max()) == 0.0, name
            continue
        assert a.shape == b_.shape and rel(a, b_) < 2e-3, (name, rel(a, b_))


def test_module_uses_the_kernel_and_matches_its_own_loop(monkeypatch):
    from ml_experiments_b200.models.jacobi import MIMOJacobiSSM

    torch.manual_seed(0)
    m = MIMOJacobiSSM(128, state_dim=64, mimo_rank=4, n_iters=12, diff_inject=True, diff_readout=True, bc_norm=True).cuda()
    x = torch.randn(2, 513, 128, device="cuda")
    y = m(x)
    y.square().mean().backward()
    g_kernel = [p.grad.clone() for p in m.parameters()]
    m.zero_grad()
    monkeypatch.setenv("B200_JACOBI_KERNEL", "0")
    y_ref = m(x)
    y_ref.square().mean().backward()
    assert ((y - y_ref).norm() / y_ref.norm()).item() < 1e-3
    for (name, p), g in zip(m.named_parameters(), g_kernel):
        assert ((g - p.grad).norm() / p.grad.norm().clamp_min(1e-12)).item() < 5e-3, name
