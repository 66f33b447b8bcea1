"""Gather-convolution kernels against the plain-torch restatement (values and all three gradients)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("B,L,H,D,S", [(2, 300, 4, 64, 17), (1, 129, 2, 32, 9), (2, 64, 1, 128, 5)])
def test_gather_conv(B, L, H, D, S):
    from ml_experiments_b200.ops.gather_conv import gather_conv, gather_conv_ref

    torch.manual_seed(0)
    x = torch.randn(B, L, H * D, device="cuda").bfloat16().float().requires_grad_(True)
    pos = (torch.rand(B, L, H, S, device="cuda") * (L + 20) - 10).requires_grad_(True)  # some taps out of range
    wgt = torch.randn(B, L, H, S, device="cuda")
    wgt[..., 0] = 0.0
    wgt.requires_grad_(True)
    g = torch.randn(B, L, H * D, device="cuda").bfloat16().float()
    ref = gather_conv_ref(x, pos, wgt, H)
    ref.backward(g)
    want = [t.grad.clone() for t in (x, pos, wgt)]
    for t in (x, pos, wgt):
        t.grad = None
    out = gather_conv(x, pos, wgt, H)
    assert ((out - ref).abs().max() / ref.abs().max()).item() < 2e-2
    out.backward(g)
    for name, t, w in zip(("dx", "dpos", "dwgt"), (x, pos, wgt), want):
        rel = ((t.grad - w).norm() / (w.norm() + 1e-9)).item()
        assert rel < 2e-2, (name, rel)


def test_gather_conv_chunk_of_queries():
    from ml_experiments_b200.ops.gather_conv import gather_conv, gather_conv_ref

    torch.manual_seed(1)
    B, L, Lq, H, D, S = 2, 200, 48, 2, 64, 7
    x = torch.randn(B, L, H * D, device="cuda").bfloat16().float()
    pos = torch.rand(B, Lq, H, S, device="cuda") * L
    wgt = torch.randn(B, Lq, H, S, device="cuda")
    out, ref = gather_conv(x, pos, wgt, H), gather_conv_ref(x, pos, wgt, H)
    assert out.shape == (B, Lq, H * D) and ((out - ref).abs().max() / ref.abs().max()).item() < 2e-2


@pytest.mark.gpu
@pytest.mark.parametrize("L,size", [(1000, 177), (177, 1000), (64, 64), (5, 300)])
def test_linear_resample_matches_interpolate(L, size):
    from ml_experiments_b200.ops.gather_conv import linear_resample

    x = torch.randn(2, L, 96, device="cuda").bfloat16().float()
    a, b = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
    ya = linear_resample(a, size)
    yb = torch.nn.functional.interpolate(b.transpose(1, 2), size=size, mode="linear", align_corners=False).transpose(1, 2)
    assert torch.allclose(ya, yb, atol=2e-2, rtol=2e-2)
    g = torch.randn_like(yb).bfloat16().float()
    ya.backward(g)
    yb.backward(g)
    assert ((a.grad - b.grad).norm() / b.grad.norm()).item() < 1e-2
