"""NorMuon update kernels (variance reduction + cautious update with the mantissa extension) against the plain torch
restatement of the same formulas."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape,red_dim", [((3, 64, 96), -2), ((3, 96, 64), -1), ((2, 128, 128), -1), ((1, 40, 72), -2)])
@pytest.mark.parametrize("p_dtype,v_dtype", [(torch.float32, torch.bfloat16), (torch.bfloat16, torch.bfloat16), (torch.float32, torch.float32)])
def test_normuon_step_matches_torch(shape, red_dim, p_dtype, v_dtype):
    from ml_experiments_b200.optim.normuon import cautious_update_, normuon_step_, normuon_variance_reduction

    torch.manual_seed(0)
    v = (torch.randn(*shape, device="cuda") * 0.05).to(v_dtype)
    p0 = (torch.randn(*shape, device="cuda") * 0.3).to(p_dtype)
    sshape = list(shape)
    sshape[red_dim] = 1
    second0 = torch.rand(*sshape, device="cuda") * 1e-3
    lr, wd = 0.03, 0.002
    for per_matrix in (False, True):
        lrs = [lr * (1 + i) for i in range(shape[0])] if per_matrix else lr
        wds = [wd * (1 + i) for i in range(shape[0])] if per_matrix else wd
        # kernel path
        p, second = p0.clone(), second0.clone()
        mant = torch.zeros(shape, dtype=torch.int16, device="cuda") if p_dtype == torch.bfloat16 else None
        normuon_step_(p, mant, v, second, 0.95, red_dim, lrs, wds)
        # torch path
        q, second_ref = p0.clone(), second0.clone()
        mant_ref = torch.zeros(shape, dtype=torch.int32, device="cuda") if p_dtype == torch.bfloat16 else None
        vr = normuon_variance_reduction(v.clone(), second_ref, 0.95, red_dim)
        if per_matrix:
            for i in range(shape[0]):
                cautious_update_(q[i], None if mant_ref is None else mant_ref[i], vr[i], lrs[i], wds[i])
        else:
            cautious_update_(q, mant_ref, vr, lr, wd)
        assert torch.allclose(second, second_ref, rtol=1e-5, atol=1e-9)
        if p_dtype == torch.bfloat16:
            wide = lambda t, m: ((t.view(torch.int16).to(torch.int32) << 16) | (m.to(torch.int32) & 0xFFFF)).view(torch.float32)
            # the oracle rounds the rescaled update to v's dtype before the step; the kernel keeps it in fp32
            assert torch.allclose(wide(p, mant), wide(q, mant_ref), atol=lr * 0.05 * 2e-2 * 4, rtol=0)
        else:
            assert torch.allclose(p, q, atol=lr * 0.05 * 2e-2 * 4 if v_dtype == torch.bfloat16 else 2e-6, rtol=0)


def test_combined_optimizer_runs_on_the_kernels():
    """NorMuonAndAdam on CUDA parameters (bf16 matrices with mantissa state) follows the CPU run of the same steps."""
    from ml_experiments_b200.optim.normuon import NorMuonAndAdam

    def make(dev):
        torch.manual_seed(3)
        params = {"attn": torch.nn.Parameter((torch.randn(4, 64, 64) * 0.1).to(torch.bfloat16).to(dev)),
                  "mlp": torch.nn.Parameter((torch.randn(4, 128, 64) * 0.1).to(dev)),
                  "embed": torch.nn.Parameter((torch.randn(64, 32) * 0.1).to(dev))}
        table = {"attn": dict(optim="normuon"), "mlp": dict(optim="normuon", per_matrix_lr_mul=[1, 2, 1, 2]),
                 "embed": dict(optim="adam", adam_betas=(0.5, 0.95))}
        return params, NorMuonAndAdam(params.items(), table, world_size=1, rank=0)

    (pc, oc), (pg, og) = make("cpu"), make("cuda")
    assert og.param_states["attn"]["mantissa"].dtype == torch.int16
    g = torch.Generator().manual_seed(11)
    for _ in range(3):
        for k in pc:
            gr = torch.randn(pc[k].shape, generator=g)
            pc[k].grad, pg[k].grad = gr.to(pc[k].dtype), gr.to(pg[k].dtype).cuda()
        oc.step()
        og.step()
    for k in pc:
        # bf16 Newton-Schulz on different back ends (tcgen05 vs CPU matmul) differs in the last bits; three steps of
        # lr 0.023 * O(0.1) updates stay within a few 1e-3
        assert torch.allclose(pg[k].detach().float().cpu(), pc[k].detach().float(), atol=5e-3), (k, (pg[k].detach().float().cpu() - pc[k].detach().float()).abs().max())


@pytest.mark.parametrize("p_dtype,g_dtype", [(torch.bfloat16, torch.bfloat16), (torch.float32, torch.bfloat16), (torch.float32, torch.float32)])
def test_adam_cautious_kernel_matches_the_operator_chain(p_dtype, g_dtype):
    from ml_experiments_b200.optim.normuon import adam_cautious_

    torch.manual_seed(4)
    n = (1000, 96)
    p0 = (torch.randn(*n, device="cuda") * 0.3).to(p_dtype)
    m0, v0 = torch.randn(*n, device="cuda") * 1e-3, torch.rand(*n, device="cuda") * 1e-5
    for _ in range(2):
        g = (torch.randn(*n, device="cuda") * 1e-2).to(g_dtype)
        p, m, v = p0.clone(), m0.clone(), v0.clone()
        adam_cautious_(p, g, m, v, 0.75, 0.95, 1e-10, 3e-3, 2e-4)                      # kernel
        q, mr, vr = p0.float().cpu(), m0.cpu(), v0.cpu()
        adam_cautious_(q, g.float().cpu(), mr, vr, 0.75, 0.95, 1e-10, 3e-3, 2e-4)      # operator chain (CPU, fp32)
        assert torch.allclose(m.cpu(), mr, rtol=1e-5, atol=1e-9) and torch.allclose(v.cpu(), vr, rtol=1e-5, atol=1e-12)
        want = q.to(p_dtype).float()
        assert torch.allclose(p.float().cpu(), want, rtol=1e-2 if p_dtype == torch.bfloat16 else 1e-5, atol=1e-6)
        p0, m0, v0 = p, m, v
