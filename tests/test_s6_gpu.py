"""S6 selective-scan kernels against the sequential fp32 oracle, and the S6 LM end to end."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture
def default_scan_shape():
    yield
    from ml_experiments_b200.ops.selective_scan import set_states_per_thread
    set_states_per_thread()


@pytest.mark.parametrize("qs", [(4, 4), (2, 4), (4, 2), (2, 2)])
@pytest.mark.parametrize("bsz,L,din", [(2, 200, 128), (1, 64, 72), (3, 333, 192)])
def test_scan_forward_backward(bsz, L, din, qs, default_scan_shape):
    from ml_experiments_b200.ops.selective_scan import selective_scan, selective_scan_ref, set_states_per_thread

    set_states_per_thread(*qs)
    torch.manual_seed(0)
    n = 16
    dev = "cuda"
    u = torch.randn(bsz, L, din, device=dev).bfloat16().float().requires_grad_(True)
    delta = (torch.rand(bsz, L, din, device=dev) * 0.2 + 0.01).requires_grad_(True)
    A = (-torch.rand(din, n, device=dev) * 4 - 0.2).requires_grad_(True)
    B = torch.randn(bsz, L, n, device=dev).requires_grad_(True)
    C = torch.randn(bsz, L, n, device=dev).requires_grad_(True)
    D = torch.randn(din, device=dev).requires_grad_(True)
    z = torch.randn(bsz, L, din, device=dev).bfloat16().float().requires_grad_(True)
    g = torch.randn(bsz, L, din, device=dev)
    ref = selective_scan_ref(u, delta, A, B, C, D, z)
    ref.backward(g)
    want = [t.grad.clone() for t in (u, delta, A, B, C, D, z)]
    for t in (u, delta, A, B, C, D, z):
        t.grad = None
    out = selective_scan(u, delta, A, B, C, D, z)
    assert ((out - ref).abs().max() / ref.abs().max()).item() < 2e-2
    out.backward(g)
    for name, t, w in zip("u delta A B C D z".split(), (u, delta, A, B, C, D, z), want):
        rel = ((t.grad - w).norm() / (w.norm() + 1e-9)).item()
        assert rel < 3e-2, (name, rel)


@pytest.mark.parametrize("delta_dtype", [torch.float32, torch.bfloat16])
def test_scan_fused_softplus_bias_gate(delta_dtype):
    """Raw step + bias + softplus and the silu(z) gate run inside the kernels; gradients reach the raw step and the bias."""
    from ml_experiments_b200.ops.selective_scan import selective_scan, selective_scan_ref

    torch.manual_seed(1)
    bsz, L, din, n, dev = 2, 150, 100, 16, "cuda"
    u = torch.randn(bsz, L, din, device=dev).bfloat16().float().requires_grad_(True)
    raw = (torch.randn(bsz, L, din, device=dev) - 3).to(delta_dtype).float().requires_grad_(True)
    bias = torch.randn(din, device=dev).requires_grad_(True)
    A = (-torch.rand(din, n, device=dev) * 4 - 0.2).requires_grad_(True)
    B = torch.randn(bsz, L, n, device=dev).requires_grad_(True)
    C = torch.randn(bsz, L, n, device=dev).requires_grad_(True)
    z = torch.randn(bsz, L, din, device=dev).bfloat16().float().requires_grad_(True)
    g = torch.randn(bsz, L, din, device=dev)
    leaves = (u, raw, bias, A, B, C, z)
    ref = selective_scan_ref(u, raw, A, B, C, None, z, delta_bias=bias, delta_softplus=True)
    ref.backward(g)
    want = [t.grad.clone() for t in leaves]
    for t in leaves:
        t.grad = None
    raw_in = raw.to(delta_dtype)
    raw_in.retain_grad()
    out = selective_scan(u, raw_in, A, B, C, None, z, delta_bias=bias, delta_softplus=True)
    assert ((out - ref).abs().max() / ref.abs().max()).item() < 2e-2
    out.backward(g)
    tol = 3e-2 if delta_dtype == torch.float32 else 5e-2
    for name, t, w in zip("u raw bias A B C z".split(), leaves, want):
        rel = ((t.grad.float() - w).norm() / (w.norm() + 1e-9)).item()
        assert rel < tol, (name, rel)


def test_s6_lm_trains():
    from ml_experiments_b200.models.s6 import S6Config, S6LM

    torch.manual_seed(0)
    m = S6LM(S6Config(d_model=128, n_layers=2, vocab_size=256)).cuda().bfloat16()
    ids = torch.randint(0, 256, (2, 256), device="cuda")
    ids[:, 1::2] = ids[:, 0::2]  # every second byte repeats the previous one: learnable
    opt = torch.optim.AdamW(m.parameters(), lr=3e-3)
    first = None
    for _ in range(30):
        loss = m(ids[:, :-1], ids[:, 1:])
        opt.zero_grad()
        loss.backward()
        opt.step()
        first = first if first is not None else loss.item()
    assert loss.item() < 0.8 * first


def test_causal_conv1d_silu():
    from ml_experiments_b200.ops.causal_conv import causal_conv1d_silu, causal_conv1d_silu_ref

    torch.manual_seed(1)
    B, L, C = 2, 150, 264
    wide = torch.randn(B, L, 2 * C, device="cuda").bfloat16()
    x = wide[..., :C].detach().requires_grad_(True)           # channel slice of a wider tensor
    w = (torch.randn(C, 1, 4, device="cuda") * 0.5).requires_grad_(True)
    b = torch.randn(C, device="cuda").requires_grad_(True)
    g = torch.randn(B, L, C, device="cuda").bfloat16()
    xr = x.detach().float().requires_grad_(True)
    wr, br = w.detach().clone().requires_grad_(True), b.detach().clone().requires_grad_(True)
    ref = causal_conv1d_silu_ref(xr, wr, br)
    ref.backward(g.float())
    y = causal_conv1d_silu(x, w, b)
    assert ((y.float() - ref).abs().max() / ref.abs().max()).item() < 2e-2
    y.backward(g)
    for name, got, want in (("dx", x.grad, xr.grad), ("dw", w.grad, wr.grad), ("db", b.grad, br.grad)):
        rel = ((got.float() - want).norm() / want.norm()).item()
        assert rel < 2e-2, (name, rel)
