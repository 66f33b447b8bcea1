"""Fused tap kernels (telephone attention, adaptive local convolution) against the unfused PyTorch restatement."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp(min=1e-12)).item()


@pytest.mark.parametrize("B,L,H,D,K,half", [(2, 300, 4, 64, 64, 8), (1, 1000, 2, 16, 16, 21), (2, 130, 3, 128, 8, 3), (1, 257, 8, 8, 33, 5)])
def test_telephone_fused(B, L, H, D, K, half):
    from ml_experiments_b200.ops import fused_taps as T

    g = torch.Generator().manual_seed(B * L + K)
    dev = "cuda"
    x = torch.randn(B, L, H * D, generator=g).bfloat16().float().to(dev)
    freq = (torch.rand(B, L, H, generator=g) * 15 + 1).to(dev)
    phase = ((torch.rand(B, L, H, generator=g) * 2 - 1) * 16).to(dev)
    kern = torch.randn(B, L, H, K, generator=g).to(dev)
    expo = (torch.rand(B, L, 1, generator=g) * 3.5 + 0.5).to(dev)
    leaves = [t.clone().requires_grad_(True) for t in (x, freq, phase, kern, expo)]
    ref_leaves = [t.clone().requires_grad_(True) for t in (x, freq, phase, kern, expo)]
    max_rec = half * 16.0
    out = T.telephone_gather(*leaves, H, half, max_rec)
    ref = T.telephone_gather_ref(*ref_leaves, H, half, max_rec)
    assert _rel(out, ref) < 1e-2
    dout = torch.randn(B, L, H * D, generator=g).bfloat16().float().to(dev)
    out.backward(dout)
    ref.backward(dout)
    for name, a, b in zip(("dx", "dfreq", "dphase", "dkern", "dexpo"), leaves, ref_leaves):
        assert _rel(a.grad, b.grad) < 2e-2, (name, _rel(a.grad, b.grad))


@pytest.mark.parametrize("B,L,H,D,K,half", [(2, 300, 4, 64, 64, 29), (1, 1000, 2, 16, 16, 9), (2, 130, 3, 128, 8, 3), (1, 257, 8, 8, 64, 12)])
def test_adaptive_local_fused(B, L, H, D, K, half):
    from ml_experiments_b200.ops import fused_taps as T

    g = torch.Generator().manual_seed(B * L + K + 1)
    dev = "cuda"
    x = torch.randn(B, L, H * D, generator=g).bfloat16().float().to(dev)
    half_w = (torch.rand(B, L, H, generator=g) * half + 0.5).to(dev)
    half_w[:, ::7] = 0.5                      # narrow windows: the tap sum stays below the normalisation threshold
    center = ((torch.rand(B, L, H, generator=g) * 2 - 1) * 12).to(dev)
    kern = torch.randn(B, L, H, K, generator=g).to(dev)
    leaves = [t.clone().requires_grad_(True) for t in (x, half_w, center, kern)]
    ref_leaves = [t.clone().requires_grad_(True) for t in (x, half_w, center, kern)]
    out = T.adaptive_local_gather(*leaves, H, half)
    ref = T.alc_gather_ref(*ref_leaves, H, half)
    assert _rel(out, ref) < 1e-2
    dout = torch.randn(B, L, H * D, generator=g).bfloat16().float().to(dev)
    out.backward(dout)
    ref.backward(dout)
    for name, a, b in zip(("dx", "dhalf_w", "dcenter", "dkern"), leaves, ref_leaves):
        assert _rel(a.grad, b.grad) < 2e-2, (name, _rel(a.grad, b.grad))


@pytest.mark.parametrize("C", [1, 4, 8, 64, 256, 300, 512, 768, 1024])
@pytest.mark.parametrize("act", ["none", "silu", "sigmoid", "tanh"])
@pytest.mark.parametrize("dtypes", [(torch.bfloat16, torch.float32), (torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16)])
def test_rms_norm_act(C, act, dtypes):
    from ml_experiments_b200.ops.norm_act import rms_norm_act, rms_norm_act_ref

    din, dout = dtypes
    g = torch.Generator().manual_seed(C)
    x = torch.randn(3, 37, C, generator=g).to("cuda", din)
    w = (torch.rand(C, generator=g) + 0.5).to("cuda")
    xa, wa = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    xb, wb = x.float().clone().requires_grad_(True), w.clone().requires_grad_(True)
    ya = rms_norm_act(xa, wa, 1e-6, act, dout)
    yb = rms_norm_act_ref(xb, wb, 1e-6, act, torch.float32)
    assert ya.dtype == dout and _rel(ya, yb) < (1e-2 if dout == torch.bfloat16 else 1e-5)
    gy = torch.randn(3, 37, C, generator=g).to("cuda")
    ya.backward(gy.to(dout))
    yb.backward(gy.to(dout).float())
    tol = 2e-2 if torch.bfloat16 in dtypes else 1e-4
    assert _rel(xa.grad, xb.grad) < tol and _rel(wa.grad, wb.grad) < tol


@pytest.mark.parametrize("C,dtype,lead", [(768, torch.bfloat16, 12), (1024, torch.bfloat16, 0), (512, torch.bfloat16, 9), (300, torch.bfloat16, 12),
                                          (256, torch.float32, 5)])
def test_rms_norm_act_skip_adds_the_skip_gradient_in_the_backward_kernel(C, dtype, lead):
    """``h, skip[, first] = rms_norm_act_skip(x, w)``; ``out = skip + f(h) + g(first)``: dx = norm backward of (dh with
    d first added into its leading columns) + the skip's gradient, from one kernel (16-byte path for bf16 rows of 256 k
    columns, several rows per warp; the general path otherwise)."""
    from ml_experiments_b200.ops.norm_act import rms_norm_act_ref, rms_norm_act_skip

    g = torch.Generator().manual_seed(C)
    x = torch.randn(6000, C, generator=g).to("cuda", dtype)
    w = (torch.rand(C, generator=g) + 0.5).to("cuda")
    xa, wa = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    xb, wb = x.float().clone().requires_grad_(True), w.clone().requires_grad_(True)
    outs = rms_norm_act_skip(xa, wa, 1e-6, "silu", lead_cols=lead)
    h, skip = outs[0], outs[1]
    loss = (skip.float() * 0.5 + torch.sin(h.float())).sum()
    if lead:
        assert outs[2].shape == (6000, lead) and torch.equal(outs[2], h[:, :lead])
        loss = loss + (outs[2].float() * 3.0).pow(2).sum()
    loss.backward()
    hb = rms_norm_act_ref(xb, wb, 1e-6, "silu", torch.float32)
    hq = hb.detach().to(dtype).float() + (hb - hb.detach())          # the slice's consumer sees the rounded output
    loss_b = (xb * 0.5 + torch.sin(hb)).sum() + ((hq[:, :lead] * 3.0).pow(2).sum() if lead else 0.0)
    loss_b.backward()
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-4
    assert _rel(h, hb) < (1e-2 if dtype == torch.bfloat16 else 1e-5)
    assert _rel(xa.grad, xb.grad) < tol and _rel(wa.grad, wb.grad) < tol
