"""``heuristic_secrets.models`` under the reference's module names: every module of the reference's package exists, carries
the reference's public names, and the adapter functions with the Triton entry-point names compute what the reference's
PyTorch fallbacks of the same operators compute."""
import importlib
import os
import re

import pytest
import torch

from ml_experiments_b200.benchmarks.common import reference_root

_ROOT = reference_root()          # a plain copy of the reference's packages next to the repository, when there is one
REF = os.path.join(_ROOT, "heuristic_secrets", "models") if _ROOT else ""
PKG = "ml_experiments_b200.heuristic_secrets.models"
# classes of the reference that nothing can construct any more (they read fields its ModelConfig no longer has)
DEAD = {"BinaryModel", "MaskModel"}


@pytest.mark.skipif(not os.path.isdir(REF), reason="reference tree not present")
def test_every_reference_module_and_public_name_exists():
    for f in sorted(os.listdir(REF)):
        if not f.endswith(".py"):
            continue
        mod = importlib.import_module(PKG if f == "__init__.py" else f"{PKG}.{f[:-3]}")
        src = open(os.path.join(REF, f)).read()
        if f == "__init__.py":
            names = re.findall(r'^\s+"(\w+)",', src, re.M)
        else:
            names = [n for n in re.findall(r"^(?:class|def) (\w+)", src, re.M) if not n.startswith("_")]
        missing = [n for n in dict.fromkeys(names) if not hasattr(mod, n) and n not in DEAD]
        assert not missing, (f, missing)


def _ref(name):
    import importlib.util
    spec = importlib.util.spec_from_file_location(f"_ref_{name}", os.path.join(REF, f"{name}.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.mark.skipif(not os.path.isdir(REF), reason="reference tree not present")
def test_scatter_and_window_adapters_match_the_reference_fallbacks():
    from ml_experiments_b200.heuristic_secrets.models import triton_scatter as T

    ref = _ref("triton_scatter")
    torch.manual_seed(0)
    a, b = T.TritonLocalWindowAttn(32, 9, 4), ref.TritonLocalWindowAttn(32, 9, 4)
    with torch.no_grad():
        a.window_proj.weight.normal_(0, 0.3)
    b.load_state_dict(a.state_dict())
    x = torch.randn(2, 21, 32)
    assert torch.allclose(a(x), b(x), atol=1e-5)

    c, d = T.TritonScatterConv(32, 8, 4), ref.TritonScatterConv(32, 8, 4)
    wave = torch.randn(2, 21, 3, 4)
    q = torch.randn(2, 21, 4, 16)
    freq = (torch.sigmoid(wave[:, :, 0]) * 15 + 1).mean(2)
    phase = (torch.tanh(wave[:, :, 1]) * 16).mean(2)
    decay = (torch.sigmoid(wave[:, :, 2]) * 9.5 + 0.5).mean(2)
    want = d._pytorch_fallback(x, q, freq, phase, decay)
    ex = lambda t: t.unsqueeze(-1).expand(-1, -1, 4).contiguous()
    got = T.triton_scatter_attention(x, q, ex(freq), ex(phase), ex(decay), d.key_weight, d.stride_grid, d.scale)
    assert torch.allclose(got, want, atol=1e-5)

    s1, s2 = T.TritonSSMStep(32, 16, 2), ref.TritonSSMStep(32, 16, 2)
    s2.load_state_dict(s1.state_dict())
    H1, o1 = s1(x, s1.init_state(x) + 0.3, 2)
    H2, o2 = s2(x, s2.init_state(x) + 0.3, 2)
    assert torch.allclose(H1, H2, atol=1e-6) and torch.allclose(o1, o2, atol=1e-6)


def test_telephone_adapter_chunk_equals_slice_of_the_whole():
    from ml_experiments_b200.heuristic_secrets.models.triton_telephone import triton_telephone_attn

    torch.manual_seed(1)
    B, L, C, H, K = 2, 40, 16, 2, 8
    x = torch.randn(B, L, C)
    freq, phase = torch.rand(B, L, H) * 3 + 1, torch.randn(B, L, H)
    kern, expo = torch.randn(B, L, H, K), torch.rand(B, L, 1) + 0.5
    whole = triton_telephone_attn(x, freq, phase, kern, expo, 4, 32.0)
    part = triton_telephone_attn(x, freq[:, 8:24], phase[:, 8:24], kern[:, 8:24], expo[:, 8:24], 4, 32.0, chunk_start=8)
    assert part.shape == (B, 16, C) and torch.allclose(part, whole[:, 8:24], atol=1e-6)


def test_gates_and_small_modules():
    from ml_experiments_b200.heuristic_secrets.models.composed import AttentionGate, SSMGate3, check_nan
    from ml_experiments_b200.heuristic_secrets.models.ripple_attention import ReLUSquared
    from ml_experiments_b200.heuristic_secrets.models.scatter_attention import RippleClassifier, SEBlock1d

    h = torch.randn(2, 12, 16)
    f, b = AttentionGate(16, 1, 2, 2, 0.0, 3, 4)(h, None)
    assert f.shape == (2, 4) and b.shape == (2, 7)
    f, b = SSMGate3(16, 1, 8, 2, 2, 0.0, 3, 4)(h, None)
    assert f.shape == (2, 4) and b.shape == (2, 7)
    assert torch.equal(ReLUSquared()(torch.tensor([-1.0, 2.0])), torch.tensor([0.0, 4.0]))
    assert SEBlock1d(16)(h).shape == h.shape
    check_nan(h, "h")
    assert RippleClassifier(16, 3, n_layers=1, kernel_size=5, num_channels=2, state_dim=8, mimo_rank=2)(torch.randn(2, 12)).shape == (2, 3)
