"""tcgen05 flash attention (forward and backward) against a dense fp32 oracle."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(t, h, d, doc_len, seed=0):
    torch.manual_seed(seed)
    qkv = torch.randn(t, 3, h, d, device="cuda", dtype=torch.bfloat16)
    q, k, v = qkv[:, 0], qkv[:, 1], qkv[:, 2]  # strided views, heads contiguous
    from ml_experiments_b200.ops.attention import doc_bounds_from_starts

    is_start = torch.zeros(t, dtype=torch.bool, device="cuda")
    is_start[::doc_len] = True
    ds, de = doc_bounds_from_starts(is_start)
    return q, k, v, ds, de


@pytest.mark.parametrize("t,doc_len,window", [(256, 256, 0), (1024, 1024, 0), (1024, 384, 0), (2048, 1000, 3), (1536, 1536, 2)])
@pytest.mark.parametrize("d", [128, 64])
def test_attention_forward(t, doc_len, window, d):
    from ml_experiments_b200.ops import attention as A

    q, k, v, ds, de = _setup(t, 3, d, doc_len)
    o, lse = A.flash_attention_forward(q, k, v, ds, de, 0.12, window)
    ref = A.attention_reference(q, k, v, ds, 0.12, window)
    err = (o.float() - ref).abs().max().item()
    assert err < 2e-2, err


@pytest.mark.parametrize("t,doc_len,window", [(256, 256, 0), (1024, 1024, 0), (1024, 384, 0), (2048, 1000, 3)])
@pytest.mark.parametrize("d", [128, 64])
def test_attention_backward(t, doc_len, window, d):
    from ml_experiments_b200.ops import attention as A

    q, k, v, ds, de = _setup(t, 2, d, doc_len, seed=1)
    d_o = torch.randn(t, 2, d, device="cuda", dtype=torch.bfloat16)
    qf, kf, vf = (x.float().detach().requires_grad_(True) for x in (q, k, v))
    ref = A.attention_reference(qf, kf, vf, ds, 0.12, window)
    ref.backward(d_o.float())
    o, lse = A.flash_attention_forward(q, k, v, ds, de, 0.12, window)
    dq, dk, dv = A.flash_attention_backward(q, k, v, o, d_o, lse, ds, de, 0.12, window)
    for name, got, want in (("dq", dq, qf.grad), ("dk", dk, kf.grad), ("dv", dv, vf.grad)):
        rel = ((got.float() - want).norm() / want.norm()).item()
        assert rel < 2e-2, (name, rel)


def test_doc_bounds():
    from ml_experiments_b200.ops.attention import doc_bounds_from_starts

    s = torch.tensor([1, 0, 0, 1, 0, 1, 0, 0], dtype=torch.bool)
    ds, de = doc_bounds_from_starts(s)
    assert ds.tolist() == [0, 0, 0, 3, 3, 5, 5, 5]
    assert de.tolist() == [3, 3, 3, 5, 5, 8, 8, 8]


def test_doc_bounds_kernel_matches_the_scan_formulation():
    from ml_experiments_b200.ops.attention import doc_bounds_from_starts, doc_bounds_from_tokens

    g = torch.Generator(device="cuda").manual_seed(3)
    for t, p in ((1, 0.5), (77, 0.1), (1024, 0.01), (49152, 0.001), (5000, 0.0)):
        tok = torch.randint(0, 50, (t,), device="cuda", generator=g)
        tok = torch.where(torch.rand(t, device="cuda", generator=g) < p, torch.full_like(tok, 99), tok)
        s0, e0 = doc_bounds_from_starts(tok == 99)
        s1, e1 = doc_bounds_from_tokens(tok, 99)
        assert torch.equal(s0, s1) and torch.equal(e0, e1), t


@pytest.mark.parametrize("d,dv", [(32, 64), (16, 32), (64, 128)])
def test_differential_flash_attention_matches_two_sdpa_calls(d, dv):
    import torch.nn.functional as F

    from ml_experiments_b200.ops.attention import differential_flash_attention

    torch.manual_seed(d)
    B, L, H = 2, 200, 3
    mk = lambda w: torch.randn(B, L, H, w, device="cuda").bfloat16().float().requires_grad_(True)
    q1, k1, q2, k2, v = mk(d), mk(d), mk(d), mk(d), mk(dv)
    o1, o2 = differential_flash_attention(q1, k1, q2, k2, v)
    t = lambda x: x.transpose(1, 2)
    r1 = t(F.scaled_dot_product_attention(t(q1), t(k1), t(v), is_causal=True))
    r2 = t(F.scaled_dot_product_attention(t(q2), t(k2), t(v), is_causal=True))
    assert o1.shape == r1.shape and (o1.float() - r1).abs().max() < 3e-2 and (o2.float() - r2).abs().max() < 3e-2
    w1, w2 = torch.randn_like(r1), torch.randn_like(r2)
    (o1.float() * w1).sum().add((o2.float() * w2).sum()).backward()
    got = [x.grad.clone() for x in (q1, k1, q2, k2, v)]
    for x in (q1, k1, q2, k2, v):
        x.grad = None
    ((r1 * w1).sum() + (r2 * w2).sum()).backward()
    for name, g, x in zip("q1 k1 q2 k2 v".split(), got, (q1, k1, q2, k2, v)):
        rel = ((g - x.grad).norm() / x.grad.norm()).item()
        assert rel < 3e-2, (name, rel)


def test_causal_self_attention_module_uses_the_flash_path_in_eval():
    from ml_experiments_b200.models.ripple_ops import CausalSelfAttention

    torch.manual_seed(0)
    m = CausalSelfAttention(256, num_heads=4, differential=True).cuda().eval()
    x = torch.randn(2, 160, 256, device="cuda")
    y, _ = m(x)
    ref, _ = m.cpu()(x.cpu())
    assert (y.cpu() - ref).abs().max() < 5e-2 * ref.abs().max() + 1e-2
