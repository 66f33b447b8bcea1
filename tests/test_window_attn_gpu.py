"""Local window attention CUDA kernels against the unfold restatement in fp32 (forward and all gradients)."""
import pytest
import torch

from ml_experiments_b200.ops.window_attn import window_attention, window_attention_ref

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("B,L,H,D,K", [(2, 300, 4, 64, 17), (1, 130, 2, 32, 8), (2, 77, 3, 16, 64)])
def test_window_attention(B, L, H, D, K):
    torch.manual_seed(0)
    dev = "cuda"
    q, k, v = (torch.randn(B, L, H, D, device=dev).bfloat16().float().requires_grad_(True) for _ in range(3))
    bias = (torch.randn(B, L, H, K, device=dev) * 2).requires_grad_(True)
    g = torch.randn(B, L, H, D, device=dev).bfloat16().float()
    scale = D ** -0.5
    ref = window_attention_ref(q, k, v, bias, scale)
    ref.backward(g)
    want = [t.grad.clone() for t in (q, k, v, bias)]
    for t in (q, k, v, bias):
        t.grad = None
    out = window_attention(q, k, v, bias, scale)
    assert ((out - ref).abs().max() / ref.abs().max()).item() < 2e-2
    out.backward(g)
    for name, t, w in zip("q k v bias".split(), (q, k, v, bias), want):
        rel = ((t.grad - w).norm() / (w.norm() + 1e-9)).item()
        assert rel < 2e-2, (name, rel)


def _fill(module):
    with torch.no_grad():
        for name, p in module.named_parameters():
            if p.abs().sum() == 0 and "wave_proj" not in name:
                p.normal_(0, 0.05)


@pytest.mark.parametrize("make,shape", [
    (lambda S: S.AdaptiveConvND(128, 1, 9, 4), (2, 300, 128)),
    (lambda S: S.AdaptiveConvND(64, 2, 9, 4), (2, 12, 10, 64)),
    (lambda S: S.LocalAttentionND(128, 17, 1, 4), (2, 300, 128)),
    (lambda S: S.HierarchicalLocalBlockND(128, 17, 1, 4), (2, 256, 128)),
    (lambda S: S.SGSBBlockND(64, 9, 1, 4), (2, 200, 64)),
])
def test_scatter_family_cuda_paths_match_cpu(make, shape):
    """The gather-convolution and window-attention kernels inside the modules against the PyTorch paths on the CPU."""
    import copy

    from ml_experiments_b200.models import scatter as S

    torch.manual_seed(0)
    m = make(S).eval()
    _fill(m)
    x = torch.randn(*shape)
    want = m(x)
    want = want[0] if isinstance(want, tuple) else want
    g = copy.deepcopy(m).cuda()
    xg = x.cuda().requires_grad_(True)
    got = g(xg)
    got = got[0] if isinstance(got, tuple) else got
    assert ((got.cpu() - want).abs().max() / want.abs().max()).item() < 4e-2
    got.sum().backward()
    assert torch.isfinite(xg.grad).all()
