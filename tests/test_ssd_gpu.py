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


@pytest.mark.parametrize("N,P,H,Hb,beta,L", [(64, 64, 2, 2, True, 384), (128, 64, 4, 2, True, 384), (64, 128, 3, 1, False, 384),
                                              (128, 128, 2, 2, True, 256), (64, 64, 2, 1, True, 2048)])
def test_backward_on_the_kernel_matches_fp32_autograd(N, P, H, Hb, beta, L):
    """Forward and backward of ``ssd_chunk_scan`` are launches of the tcgen05 kernel (the backward: three scans with
    exchanged operand roles + elementwise sums). Oracle: autograd through the batched-GEMM formulation in fp32 on the
    same bf16-rounded inputs. The kernel rounds its operands (dy among them) and the intra-chunk weights to bf16.
    The decay gradient is a difference of row and column sums of two such scans, taken inside a 128-step chunk (the
    part of later chunks comes from the fp32 boundary states): its rounding noise is larger than that of the other
    gradients but does not grow with the sequence length, which the L = 2048 case pins."""
    from ml_experiments_b200.ops.runtime import check_status
    from ml_experiments_b200.ops.ssd_scan import _ssd_chunk_scan_torch, ssd_chunk_scan

    ins = _inputs(2 if L <= 384 else 1, L, H, Hb, N, P, beta, seed=3)
    leaves = [None if t is None else t.clone().requires_grad_(True) for t in ins]
    y = ssd_chunk_scan(*leaves)
    assert y.grad_fn is not None and "SsdKernelGradFn" in type(y.grad_fn).__name__
    w = torch.randn_like(y.float()).bfloat16().float()
    (y.float() * w).sum().backward()
    check_status()
    ref_leaves = [None if t is None else t.float().clone().requires_grad_(True) for t in ins]
    grouped = list(ref_leaves)      # the GEMM formulation broadcasts one B / C group at most: spell the groups out
    if 1 < Hb < H:
        grouped[1], grouped[2] = (t.repeat_interleave(H // Hb, dim=2) for t in ref_leaves[1:3])
    y2 = _ssd_chunk_scan_torch(*grouped)
    (y2 * w).sum().backward()
    rel = lambda a, r: ((a.float() - r.float()).norm() / r.float().norm().clamp_min(1e-12)).item()
    assert rel(y, y2) < 2e-2
    for name, a, r in zip(("x", "B", "C", "log_alpha", "gamma", "beta"), leaves, ref_leaves):
        if a is None:
            continue
        tol = 6e-2 if name == "log_alpha" else 3e-2
        assert a.grad is not None and a.grad.shape == r.grad.shape and rel(a.grad, r.grad) < tol, (name, rel(a.grad, r.grad))


def test_calls_with_states_differentiate_the_gemm_formulation():
    """An initial or returned state keeps the earlier route: kernel forward, batched-GEMM backward."""
    from ml_experiments_b200.ops.ssd_scan import _ssd_chunk_scan_torch, ssd_chunk_scan

    x, B, C, la, g, bt = _inputs(2, 256, 2, 2, 64, 64, True, seed=3)
    s0 = torch.randn(2, 2, 64, 64, device="cuda") * 0.3
    leaves = [t.clone().requires_grad_(True) for t in (x, B, C, la, g, bt)]
    y, st = ssd_chunk_scan(*leaves, init_state=s0, return_state=True)
    w = torch.randn_like(y.float())
    ((y.float() * w).sum() + st.sum()).backward()
    ref_leaves = [t.clone().requires_grad_(True) for t in (x, B, C, la, g, bt)]
    y2, st2 = _ssd_chunk_scan_torch(*ref_leaves, init_state=s0, return_state=True)
    ((y2.float() * w).sum() + st2.sum()).backward()
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
