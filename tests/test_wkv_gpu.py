"""WKV-4 / WKV-5 CUDA kernels against the sequential fp32 restatements (forward and all gradients)."""
import pytest
import torch

from ml_experiments_b200.ops.wkv import wkv4, wkv4_ref, wkv5, wkv5_ref

pytestmark = pytest.mark.gpu


def _compare(names, leaves, run_ref, run_cuda, g, tol):
    ref = run_ref()
    ref.backward(g)
    want = [t.grad.clone() for t in leaves]
    for t in leaves:
        t.grad = None
    out = run_cuda()
    assert ((out.float() - ref).abs().max() / ref.abs().max()).item() < tol
    out.backward(g.to(out.dtype))
    for name, t, w in zip(names, leaves, want):
        rel = ((t.grad.float() - w).norm() / (w.norm() + 1e-9)).item()
        assert rel < tol, (name, rel)


def test_wkv4():
    torch.manual_seed(0)
    B, T, C = 3, 70, 96
    dev = "cuda"
    decay = (torch.randn(C, device=dev) - 1).requires_grad_(True)
    u = torch.randn(C, device=dev).requires_grad_(True)
    k = torch.randn(B, T, C, device=dev).requires_grad_(True)
    v = torch.randn(B, T, C, device=dev).requires_grad_(True)
    g = torch.randn(B, T, C, device=dev)
    _compare("decay u k v".split(), (decay, u, k, v), lambda: wkv4_ref(decay, u, k, v), lambda: wkv4(decay, u, k, v), g, 1e-3)


@pytest.mark.parametrize("N", [32, 64])
def test_wkv5(N):
    torch.manual_seed(0)
    B, T, H = 2, 50, 3
    dev = "cuda"
    decay = (torch.rand(H, N, device=dev) * 5 - 6).requires_grad_(True)
    u = (torch.randn(H, N, device=dev) * 0.5).requires_grad_(True)
    r, k, v = ((torch.randn(B, T, H * N, device=dev) * 0.5).requires_grad_(True) for _ in range(3))
    g = torch.randn(B, T, H * N, device=dev)
    _compare("r k v decay u".split(), (r, k, v, decay, u), lambda: wkv5_ref(r, k, v, decay, u), lambda: wkv5(r, k, v, decay, u), g, 2e-3)
