"""UnifiedModel family on the GPU: the CUDA gather / S6 kernels and the SSD scan against the CPU fp32 path."""
import copy

import pytest
import torch

from ml_experiments_b200.models import unified as U
from ml_experiments_b200.ops.ssd_scan import ssd_chunk_scan, ssd_scan_ref

pytestmark = pytest.mark.gpu


def _fill(module):
    with torch.no_grad():
        for p in module.parameters():
            if p.abs().sum() == 0:
                p.normal_(0, 0.05)


def test_deform_conv_cuda_gather_matches_cpu():
    torch.manual_seed(0)
    conv = U.DeformConv1d(64, kernel_size=5, groups=4).eval()
    _fill(conv)
    x = torch.randn(2, 300, 64)
    want = conv(x)
    got = copy.deepcopy(conv).cuda()(x.cuda()).cpu()
    assert torch.allclose(got, want, atol=3e-2, rtol=3e-2), (got - want).abs().max()


def test_deform_conv2d_cuda_gather_matches_cpu():
    torch.manual_seed(0)
    conv = U.DeformConv2d(32, kernel_size=3, groups=2).eval()
    _fill(conv)
    x = torch.randn(2, 12, 10, 32)
    want = conv(x)
    got = copy.deepcopy(conv).cuda()(x.cuda()).cpu()
    assert torch.allclose(got, want, atol=3e-2, rtol=3e-2), (got - want).abs().max()


def test_s6_mixer_cuda_kernel_matches_cpu():
    torch.manual_seed(0)
    m = U.SSMMixer(64, state_size=16, conv_groups=4, dropout=0.0).eval()
    _fill(m)
    x = torch.randn(2, 200, 64)
    want = m(x)
    got = copy.deepcopy(m).cuda()(x.cuda()).cpu()
    assert torch.allclose(got, want, atol=5e-2, rtol=5e-2), (got - want).abs().max()


def test_ssd_scan_cuda_matches_sequential():
    torch.manual_seed(0)
    b, L, H, P, N = 2, 777, 3, 16, 32
    x = torch.randn(b, L, H, P, device="cuda")
    B, C = torch.randn(b, L, H, N, device="cuda"), torch.randn(b, L, H, N, device="cuda")
    la = -torch.rand(b, L, H, device="cuda") * 0.2
    g, be = torch.rand(b, L, H, device="cuda"), torch.rand(b, L, H, device="cuda")
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        y = ssd_chunk_scan(x, B, C, la, g, be)
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    yr, _ = ssd_scan_ref(x.cpu(), B.cpu(), C.cpu(), la.cpu(), g.cpu(), be.cpu())
    assert torch.allclose(y.cpu(), yr, atol=2e-3, rtol=2e-3), (y.cpu() - yr).abs().max()


@pytest.mark.parametrize("kw", [dict(), dict(adaptive_conv=True, n_adaptive_branches=2)])
def test_unified_model_trains_on_gpu(kw):
    torch.manual_seed(0)
    cfg = U.ModelConfig(n_layers=2, layer=U.LayerConfig(embed_width=64, dropout=0.0, attn_heads=2, ssm_n_heads=2, ssm_state_size=16,
                                                        attn_window_size=128, conv_groups=4, **kw), head=U.HeadConfig("classifier", 2))
    m = U.Model(cfg)
    x = torch.randint(0, 256, (4, 256))
    mask = torch.arange(256)[None] >= torch.tensor([256, 200, 64, 256])[:, None]
    cpu_logits, _ = m.eval()(x, mask)
    g = copy.deepcopy(m).cuda()
    logits, aux = g(x.cuda(), mask.cuda())
    assert torch.allclose(logits.cpu(), cpu_logits, atol=5e-2, rtol=5e-2), (logits.cpu() - cpu_logits).abs().max()
    (logits.sum() + sum(aux.values())).backward()
    assert all(p.grad is None or torch.isfinite(p.grad).all() for p in g.parameters())


def test_model2d_runs_on_gpu():
    torch.manual_seed(0)
    cfg = U.ModelConfig2d(n_layers=1, layer=U.LayerConfig2d(embed_width=32, dropout=0.0, ssm_kernel_sizes=(3,), attn_window_size=8),
                          head=U.HeadConfig2d(n_classes=10))
    m = U.Model2d(cfg).eval()
    x = torch.randn(2, 3, 16, 16)
    want = m(x)[0]
    g = copy.deepcopy(m).cuda()
    out, aux = g(x.cuda())
    assert torch.allclose(out.cpu(), want, atol=5e-2, rtol=5e-2), (out.cpu() - want).abs().max()
    out.sum().backward()
