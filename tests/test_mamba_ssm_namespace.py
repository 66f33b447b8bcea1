"""``zoology.mixers.mamba_ssm`` under the reference's module names: layouts and semantics of the adapter functions."""
import importlib

import pytest
import torch
import torch.nn.functional as F

PKG = "ml_experiments_b200.zoology.mixers.mamba_ssm"


def test_modules_of_the_reference_tree_import():
    for m in ("", ".selective_scan_interface", ".ops.selective_scan_interface", ".ops.triton.ssd_combined", ".ops.triton.layernorm_gated",
              ".ops.triton.layer_norm", ".ops.triton.layernorm", ".ops.triton.selective_state_update", ".ops.triton.k_activations",
              ".ops.triton.softplus", ".triton.layernorm", ".triton.selective_state_update"):
        importlib.import_module(PKG + m)


def _naive_s6(u, delta, A, B, C, D, z, bias):
    """Channel-first step-by-step recurrence written from the definition."""
    d = F.softplus(delta + bias[None, :, None])
    h = torch.zeros(u.shape[0], u.shape[1], A.shape[1], dtype=u.dtype)
    ys = []
    for t in range(u.shape[2]):
        h = torch.exp(d[:, :, t, None] * A) * h + (d[:, :, t] * u[:, :, t]).unsqueeze(-1) * B[:, None, :, t]
        ys.append((h * C[:, None, :, t]).sum(-1))
    y = torch.stack(ys, -1) + u * D[None, :, None]
    return y * F.silu(z), h


def test_selective_scan_fn_channel_first_layout_and_last_state():
    from ml_experiments_b200.zoology.mixers.mamba_ssm.ops.selective_scan_interface import selective_scan_fn, selective_scan_ref

    torch.manual_seed(0)
    b, d, L, n = 2, 6, 19, 4
    u, delta, z = torch.randn(b, d, L), torch.randn(b, d, L), torch.randn(b, d, L)
    A, B, C, D, bias = -torch.rand(d, n), torch.randn(b, n, L), torch.randn(b, n, L), torch.randn(d), torch.randn(d) * 0.1
    want, h_want = _naive_s6(u, delta, A, B, C, D, z, bias)
    for fn in (selective_scan_fn, selective_scan_ref):
        y, last = fn(u, delta, A, B, C, D, z, bias, True, return_last_state=True)
        assert y.shape == (b, d, L) and torch.allclose(y, want, atol=1e-5) and torch.allclose(last, h_want, atol=1e-5)
    y4 = selective_scan_fn(u, delta, A, B.unsqueeze(1), C.unsqueeze(1), D, z, bias, True)       # one group, 4-D B / C
    assert torch.allclose(y4, want, atol=1e-5)


def test_mamba_inner_fn_is_the_mixer_forward():
    """Against this package's S6 mixer module with the same parameters (the mixer runs conv -> x_proj -> dt_proj -> scan ->
    gate -> out_proj on channel-last tensors)."""
    from ml_experiments_b200.models.s6 import S6Config, S6Mixer
    from ml_experiments_b200.zoology.mixers.mamba_ssm.ops.selective_scan_interface import mamba_inner_fn, mamba_inner_ref

    torch.manual_seed(1)
    m = S6Mixer(S6Config(d_model=16, n_layers=1, d_state=4)).eval()
    x = torch.randn(2, 11, 16)
    xz = F.linear(x, m.in_proj.weight).transpose(1, 2)                                        # [b, 2 dim, L]
    args = (xz, m.conv1d.weight, m.conv1d.bias, m.x_proj.weight, m.dt_proj.weight, m.out_proj.weight, None, -torch.exp(m.A_log.float()))
    kw = dict(D=m.D, delta_bias=m.dt_proj.bias, delta_softplus=True)
    with torch.no_grad():
        want = m(x)
        assert torch.allclose(mamba_inner_fn(*args, **kw), want, atol=1e-5)
        assert torch.allclose(mamba_inner_ref(*args, **kw), want, atol=1e-5)


def test_ssd_functions_agree_with_the_stepwise_oracle():
    from ml_experiments_b200.zoology.mixers.mamba_ssm.ops.triton import ssd_combined as S

    torch.manual_seed(2)
    b, l, h, p, g, n = 2, 48, 4, 8, 2, 8
    x, z = torch.randn(b, l, h, p), torch.randn(b, l, h, p)
    dt, A = torch.randn(b, l, h) * 0.5, -torch.rand(h) - 0.2
    B, C, D, dt_bias = torch.randn(b, l, g, n), torch.randn(b, l, g, n), torch.randn(h), torch.randn(h) * 0.1
    want = S.ssd_selective_scan(x, dt, A, B, C, D=D, z=z, dt_bias=dt_bias, dt_softplus=True)
    for got in (S.mamba_chunk_scan_combined(x, dt, A, B, C, 16, D=D, z=z, dt_bias=dt_bias, dt_softplus=True),
                S.mamba_chunk_scan(x, dt, A, B, C, 16, D=D, z=z, dt_bias=dt_bias, dt_softplus=True),
                S.ssd_chunk_scan_combined_ref(x, dt, A, B, C, 16, D=D, z=z, dt_bias=dt_bias, dt_softplus=True)):
        assert torch.allclose(got, want, atol=2e-4, rtol=1e-3)


@pytest.mark.parametrize("norm", [False, True])
def test_split_conv_scan_block_matches_its_reference_form(norm):
    from ml_experiments_b200.zoology.mixers.mamba_ssm.ops.triton import ssd_combined as S

    torch.manual_seed(3)
    b, l, h, p, g, n, out = 2, 32, 2, 8, 1, 4, 12
    dim = h * p
    zxbcdt = torch.randn(b, l, 2 * dim + 2 * g * n + h) * 0.5
    cw, cb = torch.randn(dim + 2 * g * n, 4) * 0.3, torch.randn(dim + 2 * g * n) * 0.1
    A, D, dt_bias = -torch.rand(h) - 0.2, torch.randn(h), torch.randn(h) * 0.1
    kw = dict(headdim=p, ngroups=g, outproj_weight=torch.randn(out, dim) * 0.2, rmsnorm_weight=torch.rand(dim) + 0.5 if norm else None,
              norm_before_gate=False)
    got = S.mamba_split_conv1d_scan_combined(zxbcdt, cw, cb, dt_bias, A, D, 16, **kw)
    want = S.mamba_split_conv1d_scan_ref(zxbcdt, cw, cb, dt_bias, A, D, 16, **kw)
    assert got.shape == (b, l, out) and torch.allclose(got, want, atol=3e-4, rtol=1e-3)


def test_gated_norms():
    from ml_experiments_b200.zoology.mixers.mamba_ssm.ops.triton.layernorm_gated import RMSNorm, layernorm_fn, rms_norm_ref, rmsnorm_fn

    torch.manual_seed(4)
    x, z, w = torch.randn(3, 5, 16), torch.randn(3, 5, 16), torch.rand(16) + 0.5
    a = rmsnorm_fn(x, w, None, z=z, eps=1e-5, group_size=8, norm_before_gate=False)
    xg = (x * F.silu(z)).view(3, 5, 2, 8)
    assert torch.allclose(a, (xg * torch.rsqrt(xg.pow(2).mean(-1, keepdim=True) + 1e-5)).view(3, 5, 16) * w, atol=1e-6)
    assert torch.allclose(rms_norm_ref(x, w, None), rmsnorm_fn(x, w, None))
    assert torch.allclose(layernorm_fn(x, w, None, eps=1e-5), F.layer_norm(x, (16,), w, None, 1e-5), atol=1e-6)
    assert RMSNorm(16)(x, z).shape == x.shape
