"""CPU checks of the host-side logic around two scan kernels: the PyTorch restatement of the MIMO-Jacobi iteration (the
GPU kernel's oracle) against the module's own loop, and the SSD backward's orchestration (three more scans with
exchanged operand roles, chunk-boundary states for the decay gradient) with the kernels emulated in fp64."""
import types

import pytest
import torch


@pytest.mark.parametrize("kw", [dict(), dict(diff_inject=True, diff_readout=True, bc_norm=True), dict(relu2=True)])
def test_jacobi_restatement_equals_the_module_loop(kw):
    from ml_experiments_b200.models.jacobi import MIMOJacobiSSM
    from ml_experiments_b200.ops.jacobi_iter import jacobi_iterate, kernel_supported

    torch.manual_seed(0)
    m = MIMOJacobiSSM(32, state_dim=16, mimo_rank=2, n_iters=5, **kw)
    x = torch.randn(2, 24, 32)
    want = m(x)                                                   # CPU: the module's own per-iteration loop
    Bm, Cm, theta, xr, alpha, gamma = m._project(x)
    g = jacobi_iterate(Bm, Cm, theta.squeeze(1), xr.squeeze(-1), alpha.squeeze(1), gamma.squeeze(1).squeeze(-1), m.diffuse.weight,
                       m.diffuse.bias, m.inject_lambda if m.diff_inject else None, m.readout_lambda if m.diff_readout else None, 5)
    assert torch.allclose(m.act(m.out_proj(g)), want, atol=1e-6)
    assert kernel_supported(64, 12) and kernel_supported(128, 12) and not kernel_supported(48, 12) and not kernel_supported(128, 40)


def _scan_emulation(x, B, C, la, go, gd, states=False, Q=4):
    """The kernel's contract in fp64: ``y_i = gd_i (C_i.B_i) x_i + C_i . S_{i-1} e^{la_i}``, ``S_i = e^{la_i} S_{i-1} + go_i B_i x_i^T``;
    with ``states`` the state after every ``Q`` steps as well."""
    b, L, H, P = x.shape
    rep = H // B.shape[2]
    Bh, Ch = B.double().repeat_interleave(rep, 2), C.double().repeat_interleave(rep, 2)
    st = torch.zeros(b, H, B.shape[-1], P, dtype=torch.float64)
    ys, sts = [], []
    for t in range(L):
        st = torch.exp(la[:, t].double())[:, :, None, None] * st
        ys.append(gd[:, t, :, None].double() * (Ch[:, t] * Bh[:, t]).sum(-1, keepdim=True) * x[:, t].double()
                  + torch.einsum("bhn,bhnp->bhp", Ch[:, t], st))
        st = st + go[:, t, :, None, None].double() * Bh[:, t, :, :, None] * x[:, t, :, None, :].double()
        if (t + 1) % Q == 0:
            sts.append(st.clone())
    y = torch.stack(ys, 1)
    return (y, torch.stack(sts, 2)) if states else y


def test_ssd_backward_orchestration_with_emulated_kernels(monkeypatch):
    from ml_experiments_b200.ops import runtime, ssd_scan as S

    def post(x, dy, y, dx_rev, dB_rev, dC_h, B, C, go, gd, dx, dB, dC, d_goff, d_gdiag, inner):
        b, L, H, P = x.shape
        Hb, N = B.shape[2], B.shape[3]
        rep = H // Hb
        Bh, Ch = B.repeat_interleave(rep, 2), C.repeat_interleave(rep, 2)
        cb, dyx = (Ch * Bh).sum(-1), (dy * x).sum(-1)
        dxo, dBo = dx_rev.flip(1), dB_rev.flip(1)
        dx.copy_(go.unsqueeze(-1) * dxo + (gd * cb).unsqueeze(-1) * dy)
        dB.copy_((go.unsqueeze(-1) * dBo + (gd * dyx).unsqueeze(-1) * Ch).view(b, L, Hb, rep, N).sum(3))
        dC.copy_(dC_h.view(b, L, Hb, rep, N).sum(3))
        d_goff.copy_((x * dxo).sum(-1))
        d_gdiag.copy_(cb * dyx)
        inner.copy_((dy * y).sum(-1) - gd * cb * dyx - go * (x * dxo).sum(-1))

    fake = types.SimpleNamespace(ssd_flip_time=lambda t: t.flip(1).contiguous(), ssd_bwd_post=post)
    monkeypatch.setattr(runtime, "ops", lambda: fake)
    monkeypatch.setattr(runtime, "add_launches", lambda n: None)
    monkeypatch.setattr(S, "_Q", 4)
    monkeypatch.setattr(S, "_launch", lambda *a, states=False: _scan_emulation(*a, states=states, Q=4))
    # the autograd function casts its operands to bf16 / fp32 for the kernel; keep fp64 for this check
    monkeypatch.setattr(torch.Tensor, "float", lambda self: self.double())
    real_to = torch.Tensor.to
    monkeypatch.setattr(torch.Tensor, "to", lambda self, *a, **k: self if (a and a[0] == torch.bfloat16) else real_to(self, *a, **k))

    torch.manual_seed(0)
    b, L, H, Hb, N, P = 2, 12, 4, 2, 6, 5
    mk = lambda *s: torch.randn(*s, dtype=torch.float64)
    ins = [mk(b, L, H, P), mk(b, L, Hb, N), mk(b, L, Hb, N), -torch.rand(b, L, H, dtype=torch.float64) * 0.5,
           torch.rand(b, L, H, dtype=torch.float64), torch.rand(b, L, H, dtype=torch.float64)]
    ref_in = [t.clone().requires_grad_(True) for t in ins]
    y_ref = _scan_emulation(*ref_in)
    w = mk(*y_ref.shape)
    want = torch.autograd.grad((y_ref * w).sum(), ref_in)
    got_in = [t.clone().requires_grad_(True) for t in ins]
    y = S._SsdKernelGradFn.apply(*got_in)
    got = torch.autograd.grad((y * w).sum(), got_in)
    assert torch.allclose(y, y_ref, atol=1e-12)
    for name, a, r in zip(("x", "B", "C", "log_alpha", "g_off", "g_diag"), got, want):
        assert torch.allclose(a, r, atol=1e-10), (name, float((a - r).abs().max()))
