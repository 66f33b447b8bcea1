"""CPU behaviour of the fused autograd nodes: without a GPU every node must reduce to the plain PyTorch expression it
stands for, value and gradient (the models call them unconditionally)."""
import torch


def _grads(loss, *leaves):
    return torch.autograd.grad(loss, leaves)


def test_linear_pair_and_tee_fall_back_to_plain_linear():
    from ml_experiments_b200.ops.linear import linear_pair, linear_tee

    torch.manual_seed(0)
    x = torch.randn(3, 5, 16, dtype=torch.float64, requires_grad=True)
    w = torch.randn(24, 16, dtype=torch.float64, requires_grad=True)
    a, b = linear_pair(x, w, 8)
    ref = x @ w.T
    assert torch.allclose(a, ref[..., :8]) and torch.allclose(b, ref[..., 8:])
    g1 = _grads(a.sin().sum() + b.cos().sum(), x, w)
    g2 = _grads(ref[..., :8].sin().sum() + ref[..., 8:].cos().sum(), x, w)
    assert all(torch.allclose(p, q) for p, q in zip(g1, g2))

    y, x2 = linear_tee(x, w)
    g1 = _grads(y.sin().sum() + x2.pow(3).sum(), x, w)
    g2 = _grads((x @ w.T).sin().sum() + x.pow(3).sum(), x, w)
    assert torch.allclose(y, ref) and all(torch.allclose(p, q) for p, q in zip(g1, g2))


def test_linear_and_mlp_residual_fall_back():
    from ml_experiments_b200.ops.linear import linear, mlp_relu2

    torch.manual_seed(1)
    x = torch.randn(2, 7, 8, requires_grad=True)
    r = torch.randn(2, 7, 8, requires_grad=True)
    w = torch.randn(8, 8, requires_grad=True)
    wf, wp = torch.randn(32, 8, requires_grad=True), torch.randn(32, 8, requires_grad=True)
    assert torch.allclose(linear(x, w, residual=r), r + x @ w.T, atol=1e-6)
    assert torch.allclose(mlp_relu2(x, wf, wp, r), r + torch.relu(x @ wf.T).square() @ wp, atol=1e-5)


def test_rms_norm_act_skip_falls_back_with_and_without_lead_columns():
    from ml_experiments_b200.ops.norm_act import rms_norm_act_ref, rms_norm_act_skip

    torch.manual_seed(2)
    x = torch.randn(6, 10, requires_grad=True)
    w = torch.rand(10) + 0.5
    h, skip = rms_norm_act_skip(x, w, 1e-6, "silu")
    assert skip is x and torch.allclose(h, rms_norm_act_ref(x, w, 1e-6, "silu"))
    h, skip, lead = rms_norm_act_skip(x, w, 1e-6, "none", lead_cols=3)
    assert lead.shape == (6, 3) and torch.equal(lead, h[:, :3])
    g1, = _grads(h.sin().sum() + skip.sum() + lead.pow(2).sum(), x)
    hr = rms_norm_act_ref(x, w, 1e-6, "none")
    g2, = _grads(hr.sin().sum() + x.sum() + hr[:, :3].pow(2).sum(), x)
    assert torch.allclose(g1, g2, atol=1e-6)


def test_head_and_medium_blocks_use_the_skip_nodes_without_changing_the_function():
    """``norm_skip`` + residual arguments against the textbook pre-norm block on CPU (HEAD block, MLP branch only)."""
    import torch.nn.functional as F

    from ml_experiments_b200.models.gpt_head import MLP, norm, norm_skip

    torch.manual_seed(3)
    x = torch.randn(1, 9, 16, requires_grad=True)
    fc, pj = torch.randn(64, 16) * 0.1, torch.randn(64, 16) * 0.1
    h, skip = norm_skip(x)
    out = MLP()(h, fc, pj, residual=skip)
    ref = x + torch.relu(F.rms_norm(x, (16,)) @ fc.T).square() @ pj
    assert torch.allclose(out, ref, atol=1e-5) and torch.allclose(norm(x), F.rms_norm(x, (16,)))
    h, skip, gate = norm_skip(x, 12)
    assert gate.shape == (1, 9, 12) and torch.equal(gate, h[..., :12])
