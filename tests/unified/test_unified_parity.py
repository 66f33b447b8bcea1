"""UnifiedModel family against the reference modules (same state dict -> same outputs), on CPU."""
import os
import sys

import pytest
import torch

REF_SRC = os.environ.get("ML_EXPERIMENTS_REFERENCE_SRC") or os.path.abspath(
    os.path.join(os.path.dirname(__file__), "..", "..", "..", "reference", "src"))
try:
    sys.path.insert(0, REF_SRC)
    from heuristic_secrets.models import backbone as RB
    from heuristic_secrets.models import composed as RC
    HAVE_REF = True
except Exception:  # the reference tree is not present on every machine
    HAVE_REF = False
finally:
    if REF_SRC in sys.path:
        sys.path.remove(REF_SRC)

from ml_experiments_b200.models import unified as U

needs_ref = pytest.mark.skipif(not HAVE_REF, reason="reference sources not available")


def _fill_zero_init(module):
    with torch.no_grad():
        for p in module.parameters():
            if p.abs().sum() == 0:
                p.normal_(0, 0.05)


def _load(mine, ref):
    r = mine.load_state_dict(ref.state_dict(), strict=False)
    assert not r.missing_keys and not r.unexpected_keys, r


@needs_ref
@pytest.mark.parametrize("layer_kw,n_classes", [
    (dict(attn_window_size=24), 2),
    (dict(adaptive_conv=True, attn_window_size=24), 2),
    (dict(adaptive_conv=True, use_attention=False, depthwise_conv=True), 2),
    (dict(ssm_kernel_sizes=(0,)), 5),
    (dict(ssm_kernel_sizes=(7,), use_attention=False, conv_groups=1), 2),
])
def test_model_matches_reference(layer_kw, n_classes):
    torch.manual_seed(0)
    rc = RC.ModelConfig(n_layers=2, layer=RC.LayerConfig(embed_width=32, dropout=0.0, **layer_kw),
                        head=RC.HeadConfig("classifier", n_classes))
    mc = U.ModelConfig.from_dict(rc.to_dict())
    assert mc.to_dict() == rc.to_dict()
    ref, mine = RC.Model(rc).eval(), U.Model(mc).eval()
    _fill_zero_init(ref)
    _load(mine, ref)
    L = 40
    x = torch.randint(0, 256, (3, L))
    mask = torch.arange(L)[None] >= torch.tensor([L, L - 7, 5])[:, None]
    pre = torch.randn(3)
    with torch.no_grad():
        a, aux_a = ref(x, mask, pre)
        b, aux_b = mine(x, mask, pre)
    assert torch.allclose(a, b, atol=2e-5), (a - b).abs().max()
    assert aux_a.keys() == aux_b.keys()
    for k in aux_a:
        assert torch.allclose(aux_a[k], aux_b[k], atol=1e-5), k


def test_s6_mixer_is_the_selective_recurrence():
    """The reference's ``SSMMixer`` cannot run (its ``dt * B`` broadcast has mismatched axes, backbone.py:1220-1222),
    so the oracle is the recurrence written out: ``h = exp(A dt) h + dt B x``, ``y = C . h + D x``, gated by ``silu(z)``."""
    torch.manual_seed(1)
    m = U.SSMMixer(16, state_size=4, conv_groups=1, dropout=0.0).eval()
    _fill_zero_init(m)
    x = torch.randn(2, 13, 16)
    mask = torch.arange(13)[None] >= torch.tensor([13, 6])[:, None]
    with torch.no_grad():
        got = m(x, mask)
        xb, z = m.in_proj(x).chunk(2, -1)
        xb = xb.masked_fill(mask.unsqueeze(-1), 0.0)
        xc = torch.nn.functional.silu(m.se(m.conv_norm(m.conv(xb)), mask)).masked_fill(mask.unsqueeze(-1), 0.0)
        dt, Bp, Cp = m.x_proj(xc).split([m.dt_rank, 4, 4], -1)
        dt = torch.nn.functional.softplus(m.dt_proj(dt))
        A = -torch.exp(m.A_log)
        h = torch.zeros(2, 32, 4)
        ys = []
        for t in range(13):
            h = torch.exp(A * dt[:, t, :, None]) * h + dt[:, t, :, None] * Bp[:, t, None, :] * xc[:, t, :, None]
            ys.append((h * Cp[:, t, None, :]).sum(-1))
        y = (torch.stack(ys, 1) + xc * m.D) * torch.nn.functional.silu(z)
        want = m.out_proj(y)
    assert torch.allclose(got, want, atol=1e-5)


@needs_ref
def test_local_attention_matches_reference():
    torch.manual_seed(1)
    mask = torch.arange(20)[None] >= torch.tensor([20, 11])[:, None]
    q, k, v = torch.randn(3, 2, 2, 20, 8).unbind(0)
    assert torch.allclose(RB.chunked_local_attention(q, k, v, 6, mask), U.chunked_local_attention(q, k, v, 6, mask), atol=1e-6)
    assert torch.allclose(RB.chunked_local_attention(q, k, v, 5), U.chunked_local_attention(q, k, v, 5), atol=1e-6)


def test_grouped_deform_conv_is_a_weighted_bilinear_read():
    """Groups > 1 (which the reference's gather cannot reshape) against a direct loop."""
    torch.manual_seed(2)
    conv = U.DeformConv1d(16, kernel_size=3, groups=4).eval()
    _fill_zero_init(conv)
    x = torch.randn(2, 9, 16)
    out = conv(x)
    xp = conv.input_proj(x)
    ctx = conv._context(x)
    off = conv.offset_net(ctx).view(2, 9, 4, 3) * conv.offset_scale
    w = torch.softmax(conv.mask_net(ctx).view(2, 9, 4, 3), -1)
    want = torch.zeros(2, 9, 4, 4)
    for n in range(2):
        for l in range(9):
            for g in range(4):
                for k in range(3):
                    p = l + (k - 1) + off[n, l, g, k].item()
                    if p < 0 or p > 8:
                        continue
                    lo = int(p)
                    hi = min(lo + 1, 8)
                    fr = p - lo
                    want[n, l, g] += w[n, l, g, k] * ((1 - fr) * xp[n, lo, 4 * g:4 * g + 4] + fr * xp[n, hi, 4 * g:4 * g + 4])
    assert torch.allclose(out, conv.output_proj(want.view(2, 9, 16)), atol=1e-5)


def test_mask_head_is_per_position_and_trains():
    torch.manual_seed(3)
    cfg = U.ModelConfig(n_layers=1, layer=U.LayerConfig(embed_width=16, dropout=0.0, adaptive_conv=True, n_adaptive_branches=2,
                                                        attn_heads=2, ssm_n_heads=2, ssm_state_size=8), head=U.HeadConfig("mask"))
    m = U.Model(cfg)
    x = torch.randint(0, 256, (2, 21))
    logits, aux = m(x)
    assert logits.shape == (2, 21) and "layer0_offset_reg" in aux
    (logits.sum() + sum(aux.values())).backward()
    assert all(p.grad is None or torch.isfinite(p.grad).all() for p in m.parameters())
    assert m.predict(x).shape == (2, 21)
