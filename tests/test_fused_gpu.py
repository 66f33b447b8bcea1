"""Fused row kernels against fp32 torch restatements."""
import pytest
import torch

pytestmark = pytest.mark.gpu
EPS = torch.finfo(torch.bfloat16).eps


def _close(a, b, tol):
    err = (a.float() - b.float()).abs().max().item()
    scale = b.float().abs().max().item() + 1e-6
    assert err <= tol * scale, (err, scale)


@pytest.mark.parametrize("c", [768, 1024, 256, 2048])
def test_rmsnorm_and_backward(c):
    from ml_experiments_b200.ops import fused as Fz

    torch.manual_seed(0)
    x = torch.randn(1000, c, device="cuda").bfloat16()
    _close(Fz.rmsnorm(x), Fz.rmsnorm_ref(x), 1e-2)
    dy = torch.randn_like(x)
    dres = torch.randn_like(x)
    xf = x.float().requires_grad_(True)
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + EPS)
    y.backward(dy.float())
    _close(Fz.norm_bwd_add(dy, x, dres), dres.float() + xf.grad, 1.5e-2)
    _close(Fz.norm_bwd_add(dy, x, None), xf.grad, 1.5e-2)


def test_mix_norm_and_backward():
    from ml_experiments_b200.ops import fused as Fz
    from ml_experiments_b200.ops.runtime import ops

    torch.manual_seed(1)
    r, c = 777, 768
    x, x0, skip, dmix = (torch.randn(r, c, device="cuda").bfloat16() for _ in range(4))
    lam = torch.tensor([0.9, 0.3], device="cuda")
    w = torch.tensor([0.7], device="cuda")
    x_mix, xn = Fz.mix_norm(x, x0, lam, skip, w)
    ref_mix = 0.9 * (x.float() + 0.7 * skip.float()) + 0.3 * x0.float()
    _close(x_mix, ref_mix, 1e-2)
    _close(xn, Fz.rmsnorm_ref(x_mix), 1e-2)
    dx = torch.empty_like(x); dskip = torch.empty_like(x)
    dx0 = torch.zeros(r, c, device="cuda"); dlam = torch.zeros(2, device="cuda"); dw = torch.zeros(1, device="cuda")
    ops().mix_bwd(dmix, x, x0, skip, lam, w, dx, dskip, dx0, dlam, dw)
    g = dmix.float()
    _close(dx, 0.9 * g, 1e-2)
    _close(dskip, 0.9 * 0.7 * g, 1e-2)
    _close(dx0, 0.3 * g, 1e-3)
    ref_dlam = torch.stack([(g * (x.float() + 0.7 * skip.float())).sum(), (g * x0.float()).sum()])
    assert torch.allclose(dlam, ref_dlam, rtol=2e-3, atol=1.0)
    assert torch.allclose(dw, (0.9 * g * skip.float()).sum().view(1), rtol=2e-3, atol=1.0)


@pytest.mark.parametrize("d", [128, 64])
def test_qkv_post(d):
    from ml_experiments_b200.ops import fused as Fz
    from ml_experiments_b200.ops.runtime import ops

    torch.manual_seed(2)
    t, h = 300, 3
    qkv = torch.randn(t, 3, h, d, device="cuda").bfloat16()
    ve = torch.randn(t, h * d, device="cuda").bfloat16()
    lam = torch.tensor([0.6, 0.4], device="cuda")
    cos, sin = Fz.rotary_tables(d, 512, "cuda")
    out = torch.empty_like(qkv)
    ops().qkv_post_fwd(qkv, ve, lam, cos, sin, out, h, d, EPS)

    def ref_fwd(qkv_f, ve_f, lam_f):
        q, k, v = qkv_f[:, 0], qkv_f[:, 1], qkv_f[:, 2]
        nrm = lambda z: z * torch.rsqrt(z.pow(2).mean(-1, keepdim=True) + EPS)
        rope = lambda z: torch.cat((z[..., : d // 2] * cos[:t, None] + z[..., d // 2:] * sin[:t, None],
                                    -z[..., : d // 2] * sin[:t, None] + z[..., d // 2:] * cos[:t, None]), -1)
        return torch.stack([rope(nrm(q)), rope(nrm(k)), lam_f[0] * v + lam_f[1] * ve_f.view(t, h, d)], 1)

    qf = qkv.float().requires_grad_(True); vf = ve.float().requires_grad_(True); lf = lam.clone().requires_grad_(True)
    ref = ref_fwd(qf, vf, lf)
    _close(out, ref, 2e-2)
    g = torch.randn(t, 3, h, d, device="cuda")
    ref.backward(g)
    dq = g[:, 0].contiguous(); dk = g[:, 1].contiguous().bfloat16(); dv = g[:, 2].contiguous().bfloat16()
    dqkv = torch.empty_like(qkv); dve = torch.empty_like(ve); dlam = torch.zeros(2, device="cuda")
    ops().qkv_post_bwd(dq, dk, dv, qkv, ve, lam, cos, sin, dqkv, dve, dlam, h, d, EPS)
    _close(dqkv, qf.grad, 2e-2)
    _close(dve, vf.grad, 2e-2)
    assert torch.allclose(dlam, lf.grad, rtol=1e-2, atol=0.5)


def test_embed_gather_scatter():
    from ml_experiments_b200.ops import fused as Fz
    from ml_experiments_b200.ops.runtime import ops

    torch.manual_seed(3)
    table = torch.randn(1000, 768, device="cuda").bfloat16()
    idx = torch.randint(0, 1000, (4096,), device="cuda", dtype=torch.int32)
    assert torch.equal(Fz.embed_gather(idx, table), table[idx.long()])
    _close(Fz.embed_gather(idx, table, normalize=True), Fz.rmsnorm_ref(table[idx.long()]), 1e-2)
    src = torch.randn(4096, 768, device="cuda").bfloat16()
    gt = torch.zeros(1000, 768, device="cuda")
    ops().embed_scatter_add(idx, src, gt)
    ref = torch.zeros(1000, 768, device="cuda").index_add_(0, idx.long(), src.float())
    assert torch.allclose(gt, ref, rtol=1e-4, atol=1e-3)


def test_cast_fp8():
    from ml_experiments_b200.ops import fused as Fz

    x = torch.randn(1000, 777, device="cuda").bfloat16()
    for dt in (torch.float8_e4m3fn, torch.float8_e5m2):
        got = Fz.cast_fp8(x, 2.0, dt)
        ref = (x.float() * 2.0).to(dt)
        assert torch.equal(got.float(), ref.float())


@pytest.mark.parametrize("cache", [False, True])               # exp(z) of the row recomputed / cached in shared memory
@pytest.mark.parametrize("t,v", [(300, 50304), (64, 65536)])
def test_softcap_ce(t, v, cache):
    from ml_experiments_b200.ops import fused as Fz
    from ml_experiments_b200.ops.runtime import ops

    ops().softcap_ce_set_cache(cache, torch.empty(0, device="cuda"))
    torch.manual_seed(4)
    logits = (torch.randn(t, v, device="cuda") * 3).bfloat16()
    tg = torch.randint(0, v - 47, (t,), device="cuda")
    lf = logits.float().requires_grad_(True)
    ref = Fz.softcap_ce_ref(lf, tg)
    ref.mean().backward()
    g16 = torch.empty_like(logits)
    rows = Fz.softcap_ce(logits, tg, g16, grad_scale=1.0 / t * 1024)
    assert torch.allclose(rows, ref.detach(), rtol=2e-3, atol=2e-3)
    rel = ((g16.float() / 1024 - lf.grad).norm() / lf.grad.norm()).item()
    assert rel < 1e-2, rel
    g8 = torch.empty(t, v, device="cuda", dtype=torch.float8_e5m2)
    Fz.softcap_ce(logits, tg, g8, grad_scale=1.0 / t * 2.0 ** 19)
    rel8 = ((g8.float() / 2.0 ** 19 - lf.grad).norm() / lf.grad.norm()).item()
    ops().softcap_ce_set_cache(True, torch.empty(0, device="cuda"))
    assert rel8 < 0.15, rel8


def test_optimizer_pieces():
    from ml_experiments_b200.ops.runtime import ops

    torch.manual_seed(5)
    n = 768 * 3072
    p = torch.randn(n, device="cuda"); g = torch.randn(n, device="cuda") * 1e-2
    m = torch.zeros(n, device="cuda"); v = torch.zeros(n, device="cuda")
    p_ref = p.clone().requires_grad_(True)
    opt = torch.optim.Adam([p_ref], lr=0.01, betas=(0.8, 0.95), eps=1e-10)
    for step in range(1, 4):
        p_ref.grad = g.clone()
        opt.step()
        ops().adam_step(p, g, m, v, 0.01, 0.8, 0.95, 1e-10, 0.0, 1 - 0.8 ** step, 1 - 0.95 ** step, 1.0)
    assert torch.allclose(p, p_ref.detach(), rtol=1e-4, atol=1e-5)
    buf = torch.zeros(n, device="cuda"); out = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    ss = torch.zeros(1, device="cuda")
    ops().muon_momentum(g, buf, out, ss, 0.95, True, 1.0)
    b_ref = 0.05 * g
    u_ref = 0.05 * g + 0.95 * b_ref
    assert torch.allclose(buf, b_ref, rtol=1e-5, atol=1e-8)
    assert torch.allclose(out.float(), u_ref, rtol=1e-2, atol=1e-6)
    assert torch.allclose(ss, out.float().pow(2).sum().view(1), rtol=1e-3)
    ops().scale_by_inv_norm(out, ss, 1e-7)
    assert abs(out.float().norm().item() - 1.0) < 1e-2
    pb = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    p2 = p.clone()
    ops().axpy_bf16_to_f32(p2, out, pb, -0.5)
    assert torch.allclose(p2, p - 0.5 * out.float(), rtol=1e-5, atol=1e-6)
    assert torch.equal(pb, p2.bfloat16())


@pytest.mark.parametrize("n,off", [(4096 + 3, 0), (1001, 1), (8, 0), (3, 0)])
@pytest.mark.parametrize("p_dtype,g_dtype", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16), (torch.bfloat16, torch.float32)])
def test_adam_step_vector_and_scalar_paths(n, off, p_dtype, g_dtype):
    """Aligned tensors take the 4-wide path with a scalar tail; views at odd offsets take the scalar kernel."""
    from ml_experiments_b200.ops.runtime import ops

    torch.manual_seed(n)
    p0 = torch.randn(n + off, device="cuda").to(p_dtype)[off:]
    g = (torch.randn(n + off, device="cuda") * 1e-2).to(g_dtype)[off:]
    m = torch.zeros(n + off, device="cuda")[off:]
    v = torch.zeros(n + off, device="cuda")[off:]
    p = p0.clone() if off == 0 else torch.cat([p0.new_zeros(off), p0])[off:]
    pf, mf, vf, gf = p.float().clone(), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda"), g.float()
    for step in range(1, 3):
        b1c, b2c = 1 - 0.8 ** step, 1 - 0.95 ** step
        ops().adam_step(p, g, m, v, 0.01, 0.8, 0.95, 1e-10, 0.1, b1c, b2c, 1.0)
        mf = 0.8 * mf + 0.2 * gf
        vf = 0.95 * vf + 0.05 * gf * gf
        pf = pf - 0.01 * 0.1 * pf
        pf = pf - (0.01 / b1c) * mf / (vf.sqrt() / b2c ** 0.5 + 1e-10)
        if p_dtype == torch.bfloat16:
            pf = pf.bfloat16().float()
    tol = 1e-2 if p_dtype == torch.bfloat16 else 1e-4
    assert torch.allclose(p.float(), pf, rtol=tol, atol=tol)
    assert torch.allclose(m, mf, rtol=1e-4, atol=1e-7) and torch.allclose(v, vf, rtol=1e-4, atol=1e-10)


def test_embed_scatter_add_two_sources():
    from ml_experiments_b200.ops.runtime import ops

    torch.manual_seed(9)
    t, c, rows = 1000, 768, 64
    idx = torch.randint(0, rows, (t,), device="cuda", dtype=torch.int32)
    a = torch.randn(t, c, device="cuda").bfloat16()
    b = torch.randn(t, c, device="cuda").bfloat16()
    table = torch.zeros(rows, c, device="cuda")
    ops().embed_scatter_add(idx, a, table, b)
    ref = torch.zeros(rows, c, device="cuda").index_add_(0, idx.long(), a.float() + b.float())
    assert torch.allclose(table, ref, rtol=1e-4, atol=1e-3)
    table.zero_()
    ops().embed_scatter_add(idx, a.float(), table)
    assert torch.allclose(table, torch.zeros(rows, c, device="cuda").index_add_(0, idx.long(), a.float()), rtol=1e-4, atol=1e-3)


@pytest.mark.parametrize("D,H,paired,strided", [(128, 6, False, True), (128, 6, True, True), (64, 4, False, False), (64, 4, True, True)])
def test_norm_rotary_kernel_matches_the_eager_composition(D, H, paired, strided):
    """RMS norm + rotary map of the current speedrun GPT in one kernel (forward, backward) against F.rms_norm + the table
    multiply in fp32; x is the q slice of a fused projection when ``strided``."""
    from ml_experiments_b200.models.gpt_head import Yarn
    from ml_experiments_b200.ops.norm_rope import norm_rotary, norm_rotary_ref

    torch.manual_seed(0)
    B, T = 1, 300
    yarn = Yarn(D, 512, paired=paired).cuda()
    base = torch.randn(B, T, 3 * H, D, device="cuda").bfloat16()
    leaf = base.clone().requires_grad_(True)
    x = leaf.chunk(3, dim=-2)[1] if strided else leaf[:, :, :H].contiguous()
    y = norm_rotary(x, yarn.factor1, yarn.factor2)
    w = torch.randn_like(y.float())
    (y.float() * w).sum().backward()
    ref_leaf = base.float().clone().requires_grad_(True)
    xr = ref_leaf.chunk(3, dim=-2)[1] if strided else ref_leaf[:, :, :H]
    yr = norm_rotary_ref(xr, yarn.factor1.float(), yarn.factor2.float(), eps=torch.finfo(torch.bfloat16).eps)
    (yr * w).sum().backward()
    rel = lambda a, b: ((a.float() - b.float()).norm() / b.float().norm()).item()
    assert rel(y, yr) < 1e-2 and rel(leaf.grad, ref_leaf.grad) < 1e-2, (rel(y, yr), rel(leaf.grad, ref_leaf.grad))


@pytest.mark.parametrize("D,with_a", [(128, True), (64, True), (128, False)])
def test_rowscale_add_kernel(D, with_a):
    from ml_experiments_b200.ops.rowops import rowscale_add

    torch.manual_seed(1)
    B, T, H = 1, 257, 6
    qkv = torch.randn(B, T, 3 * H, D, device="cuda").bfloat16().requires_grad_(True)
    g = torch.rand(B, T, H, device="cuda").bfloat16().requires_grad_(True)
    b = torch.randn(B, T, H, D, device="cuda").bfloat16().requires_grad_(True)
    a = qkv.chunk(3, dim=-2)[2] if with_a else None          # the strided v slice of a fused projection
    out = rowscale_add(a, g, b)
    w = torch.randn_like(out.float())
    (out.float() * w).sum().backward()
    got = [t.grad.clone() for t in (qkv, g, b)] if with_a else [None, g.grad.clone(), b.grad.clone()]
    q2, g2, b2 = (t.detach().float().requires_grad_(True) for t in (qkv, g, b))
    ref = (q2.chunk(3, dim=-2)[2] if with_a else 0) + g2.unsqueeze(-1) * b2
    (ref * w).sum().backward()
    rel = lambda x, y: ((x.float() - y.float()).norm() / y.float().norm().clamp_min(1e-12)).item()
    assert rel(out, ref) < 1e-2
    for x, y in zip(got, (q2.grad, g2.grad, b2.grad)):
        if x is not None:
            assert rel(x, y) < 1e-2


@pytest.mark.parametrize("terms", [2, 3])
def test_lincomb3_kernel(terms):
    from ml_experiments_b200.ops.rowops import lincomb3

    torch.manual_seed(2)
    xs = [torch.randn(1, 1000, 768, device="cuda").bfloat16().requires_grad_(True) for _ in range(terms)]
    c = torch.tensor([0.7, -1.3, 0.4][:terms], device="cuda", requires_grad=True)
    out = lincomb3(xs[0], xs[1], xs[2] if terms == 3 else None, c)
    w = torch.randn_like(out.float())
    (out.float() * w).sum().backward()
    xr = [t.detach().float().requires_grad_(True) for t in xs]
    cr = c.detach().clone().requires_grad_(True)
    ref = sum(cr[i] * xr[i] for i in range(terms))
    (ref * w).sum().backward()
    rel = lambda x, y: ((x.float() - y.float()).norm() / y.float().norm().clamp_min(1e-12)).item()
    assert rel(out, ref) < 1e-2 and rel(c.grad, cr.grad) < 1e-2
    for t, r in zip(xs, xr):
        assert rel(t.grad, r.grad) < 1e-2


def test_mlp_relu2_node_matches_autograd():
    from ml_experiments_b200.ops.linear import mlp_relu2

    torch.manual_seed(3)
    x = (torch.randn(1, 512, 256, device="cuda") * 0.5).bfloat16().requires_grad_(True)
    wf = (torch.randn(1024, 256, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    wp = (torch.randn(1024, 256, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    y = mlp_relu2(x, wf, wp)
    w = torch.randn_like(y.float())
    (y.float() * w).sum().backward()
    xr, fr, pr = (t.detach().float().requires_grad_(True) for t in (x, wf, wp))
    yr = torch.relu(xr @ fr.T).square() @ pr
    (yr * w).sum().backward()
    rel = lambda a, b: ((a.float() - b.float()).norm() / b.float().norm()).item()
    assert rel(y, yr) < 2e-2
    for a, b in ((x.grad, xr.grad), (wf.grad, fr.grad), (wp.grad, pr.grad)):
        assert rel(a, b) < 2e-2, rel(a, b)


def test_linear_pair_node_matches_autograd():
    """Two outputs from row ranges of one weight; the backward sums the two data gradients in a GEMM epilogue and
    writes both weight gradients into one buffer (unequal halves; one of them small enough for split-K)."""
    from ml_experiments_b200.ops.linear import linear_pair

    torch.manual_seed(11)
    x = (torch.randn(2, 1024, 256, device="cuda") * 0.5).bfloat16().requires_grad_(True)
    w = (torch.randn(512 + 128, 256, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    ya, yb = linear_pair(x, w, 512)
    assert ya.shape == (2, 1024, 512) and yb.shape == (2, 1024, 128) and ya.is_contiguous() and yb.is_contiguous()
    ga, gb = torch.randn_like(ya.float()), torch.randn_like(yb.float())
    ((ya.float() * ga).sum() + (yb.float() * gb).sum()).backward()
    xr, wr = (t.detach().float().requires_grad_(True) for t in (x, w))
    yr = xr @ wr.T
    ((yr[..., :512] * ga).sum() + (yr[..., 512:] * gb).sum()).backward()
    rel = lambda a, b: ((a.float() - b.float()).norm() / b.float().norm()).item()
    assert rel(ya, yr[..., :512]) < 1e-2 and rel(yb, yr[..., 512:]) < 1e-2
    assert rel(x.grad, xr.grad) < 2e-2 and rel(w.grad, wr.grad) < 2e-2


def test_linear_tee_adds_the_other_gradient_in_the_epilogue():
    from ml_experiments_b200.ops.linear import linear_tee

    torch.manual_seed(12)
    x = (torch.randn(2, 640, 256, device="cuda") * 0.5).bfloat16().requires_grad_(True)
    w = (torch.randn(96, 256, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    y, x2 = linear_tee(x, w)
    gy = torch.randn_like(y.float())
    ((y.float() * gy).sum() + x2.float().pow(2).sum()).backward()
    xr, wr = (t.detach().float().requires_grad_(True) for t in (x, w))
    ((xr @ wr.T * gy).sum() + xr.pow(2).sum()).backward()
    rel = lambda a, b: ((a.float() - b.float()).norm() / b.float().norm()).item()
    assert rel(y, xr.detach() @ wr.detach().T) < 1e-2 and rel(x.grad, xr.grad) < 1e-2 and rel(w.grad, wr.grad) < 2e-2


def test_embedding_op_matches_torch():
    from ml_experiments_b200.ops.fused import embedding

    torch.manual_seed(6)
    table = torch.randn(3000, 768, device="cuda").bfloat16().requires_grad_(True)
    idx = torch.randint(0, 3000, (4096,), device="cuda")
    idx[:64] = 7                                               # a heavily repeated row
    out = embedding(idx, table)
    w = torch.randn_like(out.float()).bfloat16()
    (out.float() * w.float()).sum().backward()
    ref_t = table.detach().float().requires_grad_(True)
    ref = torch.nn.functional.embedding(idx, ref_t)
    (ref * w.float()).sum().backward()
    assert torch.equal(out.float(), ref)
    assert ((table.grad.float() - ref_t.grad).norm() / ref_t.grad.norm()).item() < 5e-3


def test_linear_and_mlp_nodes_add_the_residual_in_the_epilogue():
    from ml_experiments_b200.ops.linear import linear, mlp_relu2

    torch.manual_seed(7)
    x = (torch.randn(1, 384, 256, device="cuda") * 0.5).bfloat16().requires_grad_(True)
    r = torch.randn(1, 384, 256, device="cuda").bfloat16().requires_grad_(True)
    w = (torch.randn(256, 256, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    wf = (torch.randn(1024, 256, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    wp = (torch.randn(1024, 256, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    rel = lambda a, b: ((a.float() - b.float()).norm() / b.float().norm()).item()
    for fused, plain in ((lambda: linear(x, w, residual=r), lambda: r + linear(x, w)),
                         (lambda: mlp_relu2(x, wf, wp, residual=r), lambda: r + mlp_relu2(x, wf, wp))):
        outs = []
        for f in (fused, plain):
            for t in (x, r, w, wf, wp):
                t.grad = None
            y = f()
            y.float().square().mean().backward()
            outs.append((y.detach(), x.grad.clone(), r.grad.clone()))
        (y1, dx1, dr1), (y2, dx2, dr2) = outs
        assert rel(y1, y2) < 1e-2 and rel(dx1, dx2) < 2e-2 and rel(dr1, dr2) < 1e-2
