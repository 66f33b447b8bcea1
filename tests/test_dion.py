"""Dion against a float64 numpy restatement of the published algorithm (single process, CPU)."""
import numpy as np
import torch

from ml_experiments_b200.optim.dion import Dion, orthonormalize


def _dion_np(W, grads, Q, lr, mu):
    M = np.zeros_like(W)
    for G in grads:
        B = M + G
        P = B @ Q
        P, _ = np.linalg.qr(P)
        R = B.T @ P
        M = B - (1 - mu) * P @ R.T
        Q = R / np.maximum(np.linalg.norm(R, axis=0, keepdims=True), 1e-8)
        W = W - lr * np.sqrt(W.shape[0] / W.shape[1]) * P @ Q.T
    return W


def test_orthonormalize():
    P = torch.randn(3, 40, 8)
    for method in ("cholqr", "qr"):
        Qm = orthonormalize(P, method)
        eye = torch.eye(8).expand(3, 8, 8)
        assert torch.allclose(Qm.transpose(1, 2) @ Qm, eye, atol=1e-3)


def test_dion_matches_restatement():
    torch.manual_seed(0)
    W0 = torch.randn(48, 32, dtype=torch.float32)
    p = W0.clone().requires_grad_(True)
    opt = Dion([p], lr=0.05, mu=0.9, rank_fraction=0.25, ortho="qr")
    grads = [torch.randn(48, 32) for _ in range(4)]
    for g in grads:
        p.grad = g.clone()
        opt.step()
    Q0 = None
    # rebuild the optimizer's initial basis deterministically
    gen = torch.Generator().manual_seed(0)
    Q0 = torch.linalg.qr(torch.randn(1, 32, 8, generator=gen)).Q[0].double().numpy()
    want = _dion_np(W0.double().numpy(), [g.double().numpy() for g in grads], Q0, 0.05, 0.9)
    # QR sign conventions cancel in P Qᵀ; compare the parameters
    assert np.allclose(p.detach().double().numpy(), want, atol=2e-4), np.abs(p.detach().double().numpy() - want).max()


def test_dion_reduces_loss():
    torch.manual_seed(1)
    A, Y = torch.randn(256, 64), torch.randn(256, 32)
    W = torch.zeros(32, 64, requires_grad=True)
    opt = Dion([W], lr=0.05, mu=0.9)
    losses = []
    for _ in range(100):
        loss = ((A @ W.T - Y) ** 2).mean()
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(loss.item())
    assert losses[-1] < 0.9 * losses[0]


def test_newton_schulz_orthonormalisation_trains_too():
    """``ortho="ns"`` (the CUDA default: GEMMs only, no factorisation): columns near-orthonormal, loss still falls."""
    P = torch.randn(2, 64, 16)
    Qm = orthonormalize(P, "ns")
    s = torch.linalg.svdvals(Qm)
    assert s.max() < 1.3 and s.min() > 0.6
    torch.manual_seed(1)
    A, Y = torch.randn(256, 64), torch.randn(256, 32)
    W = torch.zeros(32, 64, requires_grad=True)
    opt = Dion([W], lr=0.05, mu=0.9, ortho="ns")
    losses = []
    for _ in range(100):
        loss = ((A @ W.T - Y) ** 2).mean()
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(loss.item())
    assert losses[-1] < 0.9 * losses[0]
