"""2-D UnifiedModel family against the reference modules (same state dict -> same outputs), on CPU."""
import os
import sys

import pytest
import torch

REF_SRC = os.environ.get("ML_EXPERIMENTS_REFERENCE_SRC") or os.path.abspath(
    os.path.join(os.path.dirname(__file__), "..", "..", "..", "reference", "src"))
try:
    sys.path.insert(0, REF_SRC)
    from heuristic_secrets.models import backbone2d as RB
    from heuristic_secrets.models import composed2d as RC
    HAVE_REF = True
except Exception:
    HAVE_REF = False
finally:
    if REF_SRC in sys.path:
        sys.path.remove(REF_SRC)

from ml_experiments_b200.models.unified import two_d as U

needs_ref = pytest.mark.skipif(not HAVE_REF, reason="reference sources not available")


def _fill_zero_init(module):
    with torch.no_grad():
        for p in module.parameters():
            if p.abs().sum() == 0:
                p.normal_(0, 0.05)


@needs_ref
@pytest.mark.parametrize("kw", [
    dict(attn_window_size=6, ssm_kernel_sizes=(3, 5), ssm_n_heads=2),
    dict(adaptive_conv=True, n_adaptive_branches=2, adaptive_kernel_size=5, attn_window_size=6, ssm_n_heads=2),
    dict(adaptive_conv=True, n_adaptive_branches=2, adaptive_kernel_size=3, use_attention=False, ssm_n_heads=2),
    dict(use_attention=False, ssm_kernel_sizes=(3,)),
])
def test_model2d_matches_reference(kw):
    torch.manual_seed(0)
    rc = RC.ModelConfig2d(n_layers=2, layer=RC.LayerConfig2d(embed_width=32, dropout=0.0, **kw), head=RC.HeadConfig2d(n_classes=5))
    mc = U.ModelConfig2d.from_dict(rc.to_dict())
    assert mc.to_dict() == rc.to_dict()
    ref, mine = RC.Model2d(rc).eval(), U.Model2d(mc).eval()
    _fill_zero_init(ref)
    r = mine.load_state_dict(ref.state_dict(), strict=False)
    assert not r.missing_keys and not r.unexpected_keys, r
    x = torch.randn(2, 3, 9, 11)
    mask = torch.zeros(2, 9, 11, dtype=torch.bool)
    mask[1, 6:] = True
    mask[1, :, 8:] = True
    with torch.no_grad():
        a, aux_a = ref(x, mask)
        b, aux_b = mine(x, mask)
    assert torch.allclose(a, b, atol=2e-5), (a - b).abs().max()
    for k in aux_a:
        assert torch.allclose(aux_a[k], aux_b[k], atol=1e-5), k
    assert mine.predict(x).shape == (2,)


@needs_ref
@pytest.mark.parametrize("heads", [1, 4])
def test_four_way_scan_matches_reference(heads):
    torch.manual_seed(1)
    ref = RB.SSMBlock3_2d(32, state_size=8, n_heads=heads, dropout=0.0, use_conv=True).eval()
    mine = U.SSMBlock3_2d(32, state_size=8, n_heads=heads, dropout=0.0, use_conv=True).eval()
    with torch.no_grad():
        ref.A_log.normal_()
        ref.b_bias.normal_()
    mine.load_state_dict(ref.state_dict())
    x = torch.randn(2, 5, 7, 32)
    with torch.no_grad():
        assert torch.allclose(ref(x)[0], mine(x)[0], atol=2e-5)


def test_deform_conv2d_and_embeddings_run_and_differentiate():
    torch.manual_seed(2)
    conv = U.DeformConv2d(16, kernel_size=3, groups=2)
    _fill_zero_init(conv)
    x = torch.randn(2, 6, 5, 16, requires_grad=True)
    conv(x).sum().backward()
    assert torch.isfinite(x.grad).all()
    emb = U.PixelEmbedding2dLearned(3, 16, max_height=8, max_width=8, dropout=0.0)
    assert emb(torch.randn(2, 3, 6, 5)).shape == (2, 6, 5, 16)
    pe = U.get_2d_sinusoidal_pos_embed(16, 4, 5, torch.device("cpu"), torch.float32)
    assert pe.shape == (4, 5, 16)
