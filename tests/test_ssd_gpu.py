"""tcgen05 SSD scan kernel against the sequential fp32 recurrence (and the batched-GEMM formulation)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(b, L, H, Hb, N, P, beta, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    r = lambda *s: torch.randn(*s, device="cuda", generator=g)
    x = r(b, L, H, P).bfloat16()
    B = (r(b, L, Hb, N) * N ** -0.5).bfloat16()
    C = (r(b, L, Hb, N) * N ** -0.5).bfloat16()
    dt = torch.nn.functional.softplus(r(b, L, H) - 2.0)
    log_alpha = -dt * torch.rand(H, device="cuda", generator=g).mul(4).add(0.5)
    gamma = dt * 0.7
    bt = dt * 0.3 * torch.exp(log_alpha) if beta else None
    return x, B, C, log_alpha, gamma, bt


@pytest.mark.parametrize("N,P", [(64, 64), (128, 64), (64, 128), (128, 128)])
@pytest.mark.parametrize("beta,init,Hb", [(False, False, 3), (True, True, 3), (True, False, 1)])
def test_kernel_matches_sequential_recurrence(N, P, beta, init, Hb):
    from ml_experiments_b200.ops.runtime import check_status
    from ml_experiments_b200.ops.ssd_scan import kernel_supported, ssd_forward_kernel, ssd_scan_ref

    b, L, H = 2, 384, 3
    x, B, C, la, g, bt = _inputs(b, L, H, Hb, N, P, beta)
    s0 = torch.randn(b, H, N, P, device="cuda") * 0.5 if init else None
    assert kernel_supported(x, B, C)
    y, st = ssd_forward_kernel(x, B, C, la, g, bt, s0, return_state=True)
    check_status()
    y_ref, st_ref = ssd_scan_ref(x.float(), B.float(), C.float(), la, g, bt, s0)
    scale = y_ref.abs().max().item()
    # operands and the intra-chunk weights are rounded to bf16 before the tensor-core products (fp32 accumulation): 2^-8
    # relative per factor, a few of them per term
    assert (y.float() - y_ref).abs().max().item() < 2e-2 * scale, ((y.float() - y_ref).abs().max().item(), scale)
    assert (st - st_ref).abs().max().item() < 2e-2 * st_ref.abs().max().item()


def test_autograd_path_and_fallback_agree():
    """``ssd_chunk_scan`` takes the kernel in the forward and differentiates the batched-GEMM form in the backward."""
    from ml_experiments_b200.ops.ssd_scan import _ssd_chunk_scan_torch, ssd_chunk_scan

    x, B, C, la, g, bt = _inputs(2, 256, 2, 2, 64, 64, True, seed=3)
    leaves = [t.clone().requires_grad_(True) for t in (x, B, C, la, g, bt)]
    y = ssd_chunk_scan(*leaves)
    w = torch.randn_like(y.float())
    (y.float() * w).sum().backward()
    ref_leaves = [t.clone().requires_grad_(True) for t in (x, B, C, la, g, bt)]
    y2 = _ssd_chunk_scan_torch(*ref_leaves)
    (y2.float() * w).sum().backward()
    assert (y.float() - y2.float()).abs().max() < 3e-2 * y2.float().abs().max()
    for a, r in zip(leaves, ref_leaves):
        assert a.grad is not None and torch.allclose(a.grad.float(), r.grad.float(), rtol=1e-3, atol=1e-5)


def test_fp32_inputs_take_the_kernel_only_under_bf16_autocast():
    from ml_experiments_b200.ops.ssd_scan import _ssd_chunk_scan_torch, kernel_supported, ssd_chunk_scan

    x, B, C, la, g, bt = _inputs(1, 256, 2, 2, 64, 64, True, seed=5)
    x, B, C = x.float(), B.float(), C.float()
    assert not kernel_supported(x, B, C)
    ref = _ssd_chunk_scan_torch(x, B, C, la, g, bt)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        assert kernel_supported(x, B, C)
        y = ssd_chunk_scan(x, B, C, la, g, bt)
    assert y.dtype == x.dtype
    assert (y - ref).abs().max() < 3e-2 * ref.abs().max()
