"""MRA block-sparse primitives and attention."""
import math

import pytest
import torch

from ml_experiments_b200.ops import mra as M


def _setup(B=2, L=128, D=16, n=5, device="cpu", seed=0):
    g = torch.Generator().manual_seed(seed)
    Q, K, V = (torch.randn(B, L, D, generator=g).to(device) for _ in range(3))
    nb = L // 32
    idx = torch.stack([torch.randperm(nb * nb, generator=g)[:n] for _ in range(B)]).to(device)
    return Q, K, V, idx


def test_block_primitives_match_dense_algebra():
    Q, K, V, idx = _setup()
    B, L, D = Q.shape
    nb = L // 32
    S = M.sddmm_ref(Q, K, idx)
    dense = Q @ K.transpose(-1, -2)
    for b in range(B):
        for n, flat in enumerate(idx[b].tolist()):
            qb, kb = divmod(flat, nb)
            assert torch.allclose(S[b, n], dense[b, qb * 32:(qb + 1) * 32, kb * 32:(kb + 1) * 32], atol=1e-5)
    # spmm = block-masked dense product
    P = torch.rand(B, idx.shape[1], 32, 32)
    Pd = torch.zeros(B, L, L)
    for b in range(B):
        for n, flat in enumerate(idx[b].tolist()):
            qb, kb = divmod(flat, nb)
            Pd[b, qb * 32:(qb + 1) * 32, kb * 32:(kb + 1) * 32] = P[b, n]
    assert torch.allclose(M.spmm_ref(P, idx, V, L, L), Pd @ V, atol=1e-4)
    assert torch.allclose(M.spmm_ref(P, idx, V, L, L, transposed=True), Pd.transpose(-1, -2) @ V, atol=1e-4)
    rm = M.rowmax_ref(P, idx, L, L)
    want = torch.where(Pd.sum(-1) > 0, Pd.amax(-1), torch.full_like(Pd[..., 0], float("-inf")))
    assert torch.allclose(rm, want)
    assert torch.allclose(M.sparse_row_sum(P, idx, L, L), Pd.sum(-1), atol=1e-4)


def test_attention_with_every_block_selected_is_softmax_attention():
    torch.manual_seed(0)
    Q, K, V = (torch.randn(2, 2, 96, 16) for _ in range(3))
    out = M.mra2_attention(Q, K, V, num_blocks=9, approx_mode="sparse")
    want = torch.softmax(Q @ K.transpose(-1, -2) / 4.0, dim=-1) @ V
    assert torch.allclose(out, want, atol=1e-4)
    causal = M.mra2_attention(Q, K, V, num_blocks=9, approx_mode="sparse", causal=True)
    want_c = torch.nn.functional.scaled_dot_product_attention(Q, K, V, is_causal=True)
    assert torch.allclose(causal, want_c, atol=1e-4)
    full = M.mra2_attention(Q, K, V, num_blocks=4, approx_mode="full", initial_prior_diagonal_n_blocks=1)
    assert full.shape == Q.shape and torch.isfinite(full).all()


def test_mixer_is_causal_and_trains():
    from ml_experiments_b200.zoology.mixers.mra import MRAAttention
    torch.manual_seed(0)
    m = MRAAttention(32, max_position_embeddings=96, num_heads=2, num_block_per_row=2)
    x = torch.randn(2, 80, 32, requires_grad=True)
    y = m(x)
    x2 = x.detach().clone()
    x2[:, 64:] += 1.0
    assert torch.allclose(y[:, :64], m(x2)[:, :64], atol=1e-4)
    y.sum().backward()
    assert torch.isfinite(x.grad).all()


@pytest.mark.gpu
def test_cuda_kernels_match_reference_forward_and_backward():
    Q, K, V, idx = _setup(B=3, L=256, D=64, n=20, device="cuda")
    Qr, Kr, Vr = (t.clone().requires_grad_(True) for t in (Q, K, V))
    Q, K, V = (t.requires_grad_(True) for t in (Q, K, V))
    S = M.SampledDenseMM.apply(Q, K, idx)
    Sr = M.sddmm_ref(Qr, Kr, idx)
    assert torch.allclose(S, Sr, atol=1e-3)
    assert torch.allclose(M.sparse_row_max(S, idx, 256, 256), M.rowmax_ref(Sr.detach(), idx, 256, 256))
    P, Pr = torch.exp(S * 0.05), torch.exp(Sr * 0.05)
    out, outr = M.SparseDenseMM.apply(P, idx, V, 256), M.spmm_ref(Pr, idx, Vr, 256, 256)
    assert torch.allclose(out, outr, atol=1e-3, rtol=1e-4)
    g = torch.randn_like(out)
    out.backward(g)
    outr.backward(g)
    for a, b in ((Q, Qr), (K, Kr), (V, Vr)):
        assert ((a.grad - b.grad).norm() / b.grad.norm()).item() < 1e-4
