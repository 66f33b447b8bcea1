"""HEAD speedrun GPT: attention layouts, multi-token loss and fp8 head."""
import pytest
import torch

from ml_experiments_b200.models import gpt_head as GH
from ml_experiments_b200.ops.fused import softcap_ce_mtp_ref, softcapped_cross_entropy


def _dense_window_attention(q, k, v, seqlens, window, scale):
    """Explicit oracle: causal, same document, keys i - window .. i."""
    T = q.shape[0]
    doc = torch.searchsorted(seqlens, torch.arange(T), right=True)
    i = torch.arange(T)
    ok = (i[:, None] >= i[None, :]) & (doc[:, None] == doc[None, :]) & (i[:, None] - i[None, :] <= window)
    s = torch.einsum("thd,shd->hts", q.float(), k.float()) * scale
    p = torch.softmax(s.masked_fill(~ok[None], float("-inf")), dim=-1)
    return torch.einsum("hts,shd->thd", p, v.float())


def test_token_exact_window_and_document_bounds():
    torch.manual_seed(0)
    T, H, D = 300, 2, 16
    q, k, v = torch.randn(3, T, H, D).unbind(0)
    seqlens = torch.tensor([0, 70, 71, 260, 300])
    ds, de = GH.doc_bounds(seqlens, T)
    assert ds[69] == 0 and ds[70] == 70 and de[70] == 71 and ds[71] == 71 and de[299] == 300
    for window in (5, 128, 200):
        got = GH._attend(q, k, v, seqlens, window, 0.3, 1)
        assert torch.allclose(got, _dense_window_attention(q, k, v, seqlens, window, 0.3), atol=1e-5)


def test_paired_head_attention_is_attention_over_the_interleaved_sequence():
    torch.manual_seed(1)
    T, H, D, dim = 96, 4, 16, 64
    attn = GH.PairedHeadCausalSelfAttention(dim, D, H)
    yarn = GH.Yarn(D, 128, paired=True)
    x = torch.randn(1, T, dim)
    w = torch.randn(4 * dim, dim) * 0.1
    seqlens = torch.tensor([0, 40, 96])
    args = GH.AttnArgs(None, torch.tensor([1.0, 1.0]), seqlens, 64, yarn, False, torch.randn(H, 12), None)
    got = attn(x, args, w)
    # oracle: build the 2T-token sequences by hand. The reference reinterprets the [T, H, D] buffer as [2T, H/2, D]
    # (train_gpt.py:1000-1011), which sends head h of token t to position 2t + h // (H/2) of head h % (H/2), while the
    # rotary angle of head h is that of position 2t + h % 2.
    qkv = torch.nn.functional.linear(x, w[:3 * dim]).view(1, T, 3 * H, D)
    q, k, v = qkv.chunk(3, dim=-2)
    q, k = GH.norm(q), GH.norm(k)
    rot = lambda t: yarn.rotary(t.reshape(1, T, H // 2, 2 * D)).reshape(T, H, D)

    def seq(thd):  # [T, H, D] -> [2T, H/2, D]
        out = torch.empty(2 * T, H // 2, D)
        for h in range(H):
            out[h // (H // 2)::2, h % (H // 2)] = thd[:, h]
        return out

    y2 = _dense_window_attention(seq(rot(q)), seq(rot(k)), seq(v[0]), 2 * seqlens, 64, yarn.attn_scale)
    y = torch.empty(1, T, H, D)
    for h in range(H):
        y[0, :, h] = y2[h // (H // 2)::2, h % (H // 2)]
    y = y * torch.sigmoid(torch.nn.functional.linear(x[..., :12], args.attn_gate_w)).view(1, T, H, 1)
    want = torch.nn.functional.linear(y.reshape(1, T, dim), w[3 * dim:])
    assert torch.allclose(got, want, atol=1e-4), (got - want).abs().max()


def test_key_offset_node_is_the_nested_concatenation():
    """Value and gradient of the shift of the keys' stationary half against the two ``cat`` calls it replaces."""
    from ml_experiments_b200.models.gpt_head import key_offset

    for T in (1, 2, 9):
        k = torch.randn(1, T, 3, 8, dtype=torch.float64, requires_grad=True)
        ref = torch.cat([k[..., :4], torch.cat([k[:, :1, :, 4:], k[:, :-1, :, 4:]], dim=1)], dim=-1)
        out = key_offset(k)
        w = torch.randn_like(out)
        g_ref, = torch.autograd.grad((ref * w).sum(), k)
        g_out, = torch.autograd.grad((out * w).sum(), k)
        assert torch.equal(ref, out) and torch.allclose(g_ref, g_out)


def test_mtp_loss_reference_matches_definition():
    torch.manual_seed(2)
    T, V = 7, 16
    logits, targets = torch.randn(T, V), torch.randint(0, V, (T,))
    w = torch.tensor([1.0, 0.5, 0.25])
    got = softcapped_cross_entropy(logits, targets, w)
    z = 23 * torch.sigmoid((logits + 5) / 7.5)
    lse = torch.logsumexp(z, -1)
    for t in range(T):
        want = sum(w[k] * (lse[t] - z[t, targets[t + k]]) for k in range(3) if t + k < T)
        assert torch.allclose(got[t], want, atol=1e-5)
    assert torch.allclose(softcap_ce_mtp_ref(logits, targets), lse - z.gather(1, targets[:, None]).squeeze(1), atol=1e-5)


def test_head_gpt_runs_and_has_reference_parameter_layout():
    torch.manual_seed(0)
    m = GH.GPT(vocab_size=300, num_heads=2, head_dim=16, model_dim=32, max_seq_len=512, bigram_vocab_size=100, use_fp8=False, world_size=8)
    shapes = {n: tuple(p.shape) for n, p in m.named_parameters()}
    assert shapes["attn_bank"] == (10, 128, 32) and m.attn_bank.reshape == (40, 32, 32) and m.attn_bank.label == "attn"
    assert shapes["mlp_bank"] == (12, 2, 128, 32) and m.mlp_bank.reshape == (24, 128, 32)
    assert shapes["scalars"] == (11 * 4 + 3 + 4,) and shapes["lm_head.weight"] == (32, 384) and shapes["attn_gate_bank"] == (10, 2, 12)
    T = 256
    x, y, big = torch.randint(0, 300, (T,)), torch.randint(0, 300, (T,)), torch.randint(0, 100, (T,))
    cfg = GH.ForwardScheduleConfig(torch.tensor([1.0, 0.5]), 1, 2)
    loss = m.train()(x, y, torch.tensor([0, 100, 256]), big, cfg)
    loss.backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in m.parameters())
    m.yarn.apply(1, 3)
    m.yarn_paired_head.apply(1, 3)
    assert abs(m.yarn.attn_scale - 0.1 * (0.2 * torch.log(torch.tensor(3.0)).item() + 1)) < 1e-6
    assert torch.isfinite(m.eval()(x, y, torch.tensor([0, 256]), big, cfg))


@pytest.mark.gpu
def test_fp8_mm_t_and_mtp_kernel_on_gpu():
    from ml_experiments_b200.ops.fp8_linear import mm_t, mm_t_ref

    torch.manual_seed(0)
    x = (torch.randn(256, 128, device="cuda") * 0.5).bfloat16().requires_grad_(True)
    w = (torch.randn(128, 512, device="cuda") * 0.02).bfloat16().requires_grad_(True)
    x_s, w_s, g_s = 4 / 448, 0.1 / 448, 8 / 448
    out = mm_t(x, w, x_s, w_s, g_s)
    ref = mm_t_ref(x, w, x_s, w_s)
    assert ((out.float() - ref).abs().max() / ref.abs().max()).item() < 2e-2
    g = torch.randn_like(out)
    out.backward(g)
    gx_ref, gw_ref = g.float() @ w.float().T, x.float().T @ g.float()
    assert ((x.grad.float() - gx_ref).norm() / gx_ref.norm()).item() < 0.1       # e5m2 gradients: 2 mantissa bits
    assert ((w.grad.float() - gw_ref).norm() / gw_ref.norm()).item() < 0.1
    # multi-token loss kernel
    T, V = 300, 512
    logits = (torch.randn(T, V, device="cuda") * 3).bfloat16().requires_grad_(True)
    targets = torch.randint(0, V, (T,), device="cuda")
    wts = torch.tensor([1.0, 0.5, 0.25], device="cuda")
    lr = logits.detach().float().requires_grad_(True)
    ref_l = softcap_ce_mtp_ref(lr, targets, wts)
    ref_l.sum().backward()
    got = softcapped_cross_entropy(logits, targets, wts)
    assert torch.allclose(got, ref_l, atol=2e-2, rtol=1e-3)
    got.sum().backward()
    assert ((logits.grad.float() - lr.grad).norm() / lr.grad.norm()).item() < 2e-2


@pytest.mark.gpu
def test_head_gpt_gpu_matches_cpu():
    import copy
    torch.manual_seed(0)
    m = GH.GPT(vocab_size=1000, num_heads=2, head_dim=128, model_dim=256, max_seq_len=1024, bigram_vocab_size=500, use_fp8=False)
    with torch.no_grad():
        for p in m.parameters():
            if p.abs().sum() == 0:
                p.normal_(0, 0.02)
    T = 512
    x, y, big = torch.randint(0, 1000, (T,)), torch.randint(0, 1000, (T,)), torch.randint(0, 500, (T,))
    seqlens = torch.tensor([0, 200, 512])
    cfg = GH.ForwardScheduleConfig(torch.tensor([1.0, 0.5]), 1, 2)
    want = m.train()(x, y, seqlens, big, cfg) / T
    g = copy.deepcopy(m).cuda().bfloat16()
    cfg_g = GH.ForwardScheduleConfig(cfg.mtp_weights.cuda(), 1, 2)
    got = g(x.cuda(), y.cuda(), seqlens.cuda(), big.cuda(), cfg_g) / T
    assert abs(got.item() - want.item()) / want.item() < 3e-2
    got.backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in g.parameters())
    g.lm_head.use_fp8 = True
    loss8 = g(x.cuda(), y.cuda(), seqlens.cuda(), big.cuda(), cfg_g) / T
    assert abs(loss8.item() - want.item()) / want.item() < 6e-2


def test_medium_track_model_trains_and_evaluates():
    from ml_experiments_b200.models.gpt_head import ForwardScheduleConfig
    from ml_experiments_b200.models.gpt_medium import GPTMedium

    torch.manual_seed(0)
    m = GPTMedium(vocab_size=300, num_heads=2, head_dim=16, model_dim=32, max_seq_len=256, world_size=8)
    assert m.scalars.numel() % 8 == 0 and m.scalars.numel() >= 16 * 3 + 5
    labels = {getattr(p, "label", None) for p in m.parameters()}
    assert {"attn", "mlp", "attn_gate", "value_embed_gate", "smear_gate", "skip_gate", "value_embed", "lm_head", "embed", "embed2",
            "x0_lambdas", "scalars"} <= labels
    for p in m.parameters():
        if p.ndim >= 2 and p.abs().sum() == 0:
            torch.nn.init.normal_(p, std=0.02)
    T = 128
    ids, tg = torch.randint(0, 300, (T,)), torch.randint(0, 300, (T,))
    seqlens = torch.tensor([0, 50, 128], dtype=torch.int32)
    cfg = ForwardScheduleConfig(mtp_weights=torch.tensor([1.0, 0.5]), ws_short=1, ws_long=2)
    loss = m(ids, tg, seqlens, cfg)
    loss.backward()
    missing = [n for n, p in m.named_parameters() if p.grad is None]
    assert missing == ["embed.weight"]          # tied to lm_head until split_embed
    m.eval()
    ev = m(ids, tg, seqlens, cfg)
    assert abs(ev.item() - loss.item() / T / 1.5) < 0.2
    # a document boundary isolates the two documents: changing document 2 leaves document 1's logits alone
    ids2 = ids.clone()
    ids2[60:] = (ids2[60:] + 1) % 300
    m.train()
    cfg1 = ForwardScheduleConfig(mtp_weights=None, ws_short=1, ws_long=2)
    l1 = m(ids[:50], tg[:50], torch.tensor([0, 50], dtype=torch.int32), cfg1)
    tg_mask = tg.clone()
    tg_mask[50:] = -1
    l2 = m(ids2, tg_mask, seqlens, cfg1)
    assert torch.allclose(l1, l2, rtol=1e-4)


@pytest.mark.gpu
def test_medium_track_model_gpu_matches_cpu_and_steps():
    """The medium-track GPT on the CUDA kernels (flash attention, tcgen05 linears, soft-capped CE) agrees with its fp32
    CPU evaluation, and a few Adam steps through its backward lower the loss."""
    import copy

    from ml_experiments_b200.models.gpt_head import ForwardScheduleConfig
    from ml_experiments_b200.models.gpt_medium import GPTMedium

    torch.manual_seed(0)
    m = GPTMedium(vocab_size=1000, num_heads=2, head_dim=128, model_dim=256, max_seq_len=1024, world_size=1)
    with torch.no_grad():
        for p in m.parameters():
            if p.ndim >= 2 and p.abs().sum() == 0:
                p.normal_(0, 0.02)
    T = 512
    x, y = torch.randint(0, 1000, (T,)), torch.randint(0, 1000, (T,))
    seqlens = torch.tensor([0, 200, 512], dtype=torch.int32)
    cfg = ForwardScheduleConfig(torch.tensor([1.0, 0.5]), 1, 2)
    want = m.train()(x, y, seqlens, cfg) / T
    g = copy.deepcopy(m).cuda().bfloat16()
    cfg_g = ForwardScheduleConfig(cfg.mtp_weights.cuda(), 1, 2)
    args = (x.cuda(), y.cuda(), seqlens.cuda(), cfg_g)
    got = g(*args) / T
    assert abs(got.item() - want.item()) / want.item() < 3e-2
    opt = torch.optim.Adam(g.parameters(), lr=3e-3)
    losses = []
    for _ in range(6):
        loss = g(*args) / T
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
        losses.append(loss.item())
    assert all(l == l for l in losses) and losses[-1] < losses[0] - 0.05, losses


@pytest.mark.gpu
def test_fused_head_and_loss_node_matches_the_two_operators():
    """fp8 projection + multi-token loss as one node against ``mm_t`` followed by ``softcapped_cross_entropy`` (same
    quantisation of x and w; the logit gradient is quantised to e5m2 before the incoming 1 / T instead of after it)."""
    from ml_experiments_b200.ops.fp8_linear import head_ce_loss, mm_t
    from ml_experiments_b200.ops.fused import softcapped_cross_entropy

    torch.manual_seed(5)
    T, K, V = 1024, 256, 2048
    x0 = torch.randn(T, K, device="cuda").bfloat16()
    w0 = (torch.randn(K, V, device="cuda") * 0.05).bfloat16()
    tg = torch.randint(0, V, (T,), device="cuda")
    mw = torch.tensor([1.0, 0.5, 0.25], device="cuda")
    scales = dict(x_s=100 / 448, w_s=1.6 / 448, grad_s=0.75 / 448)
    outs = []
    for fused in (True, False):
        x, w = x0.clone().requires_grad_(True), w0.clone().requires_grad_(True)
        if fused:
            loss = head_ce_loss(x, w, tg, mw, **scales) / T
        else:
            loss = softcapped_cross_entropy(mm_t(x, w, **scales), tg, mw).sum() / T
        loss.backward()
        outs.append((loss.item(), x.grad.float(), w.grad.float()))
    (l1, dx1, dw1), (l2, dx2, dw2) = outs
    rel = lambda a, b: ((a - b).norm() / b.norm()).item()
    assert abs(l1 - l2) < 1e-3 * abs(l2) and rel(dx1, dx2) < 8e-2 and rel(dw1, dw2) < 8e-2, (l1, l2, rel(dx1, dx2), rel(dw1, dw2))
