"""Ripple family on CPU: shapes, gradients, reference-compatible parameter names; GPU variant uses the gather kernels."""
import pytest
import torch

from ml_experiments_b200.models.ripple import RippleAttention, RippleClassifier


def test_classifier_2d_and_lm_shapes():
    torch.manual_seed(0)
    m = RippleClassifier(width=32, n_layers=2, n_classes=2, seq_len=256, num_heads=4, max_kernel_size=16, embed_2d=(16, 16),
                         max_seq_len=256)
    out = m(torch.rand(3, 16, 16))
    assert out.shape == (3, 2)
    out.sum().backward()
    assert all(p.grad is not None for n, p in m.named_parameters() if "lambda" not in n)
    lm = RippleClassifier(width=32, n_layers=1, n_classes=50, seq_len=64, num_heads=2, vocab_size=50, order="attn,conv",
                          max_seq_len=64)
    assert lm(torch.randint(0, 50, (2, 64))).shape == (2, 64, 50)
    names = set(m.state_dict())
    for k in ("layers.0.attn.telephone.wave_proj.weight", "layers.0.attn.conv.kernel_gamma", "layers.0.attn.lowrank.lambda_q1",
              "layers.0.attn.norms.tele.weight", "layers.1.mlp.2.bias", "embed.pixel_embed.weight", "head.weight"):
        assert k in names, k


def test_attention_orders():
    x = torch.randn(2, 100, 32)
    for order in ("tele", "conv", "lowrank", "attn", "jacobi", "tele,conv,lowrank,attn"):
        y, _ = RippleAttention(32, num_heads=2, order=order, max_seq_len=128)(x)
        assert y.shape == x.shape and torch.isfinite(y).all(), order


@pytest.mark.gpu
def test_gpu_matches_cpu_path():
    torch.manual_seed(1)
    m = RippleClassifier(width=64, n_layers=1, n_classes=3, seq_len=300, num_heads=2, max_kernel_size=16, max_seq_len=512).eval()
    x = torch.rand(2, 300)
    ref = m(x)
    out = m.cuda()(x.cuda()).cpu()
    assert (out - ref).abs().max().item() < 5e-2 * ref.abs().max().item() + 1e-3
