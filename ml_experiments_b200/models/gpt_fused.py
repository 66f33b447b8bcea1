"""Fused sm_100a forward + backward of :class:`ml_experiments_b200.models.gpt.GPT`.

The whole training step of the model is one autograd node. Its forward runs the network with the tcgen05 GEMM
(fused ReLU² / residual epilogues), the flash-attention kernel, the fused norm / RoPE / mixing row kernels and the
fp8 head + soft-capped cross entropy; when gradients are enabled it immediately runs the hand-scheduled backward
(data gradients with MN-major weights, weight gradients with both operands MN-major and split-K, attention
backward with TMEM-resident dK/dV) and keeps the parameter gradients for ``backward`` to hand out.

Activations are kept (a 12-layer, 49 152-token step holds ~20 GB of the 180 GB HBM3e), nothing is recomputed.
"""
from __future__ import annotations

import torch
from torch import Tensor

from ..ops import fused as Fz
from ..ops import gemm as G
from ..ops.attention import flash_attention_backward, flash_attention_forward
from ..ops.runtime import ops
from ..utils.shadow import shadow_of

EPS = Fz.BF16_EPS


class _Saved:
    __slots__ = ("x_in", "x_mix", "xn", "qkv", "qkvp", "y", "lse", "x_a", "xn2", "h", "skip", "skip_idx")


def _wgrad(dy: Tensor, x: Tensor, out_shape, out: Tensor | None = None) -> Tensor:
    """dW[out, in] = dyᵀ · x with both operands consumed MN-major; split-K fills the machine for small outputs.
    ``out``: an fp32 buffer of ``out_shape`` to write into (the optimizer's stacked gradient slot of this matrix)."""
    n_out, n_in = dy.shape[1], x.shape[1]
    sk = G.auto_split_k(n_out, n_in, dy.shape[0])
    if out is not None and (out.dtype != torch.float32 or not out.is_contiguous()):
        out = None
    dst = None if out is None else out.view(n_out, n_in)
    return G.gemm(dy, x, a_mn=True, b_mn=True, split_k=sk, out=dst, out_dtype=torch.float32).view(out_shape)


def _forward_backward(model, input_seq: Tensor, target_seq: Tensor, swb: int, need_grad: bool):
    c = model.config
    dev = input_seq.device
    T = input_seq.numel()
    H, D, C = c.num_heads, c.head_dim, c.model_dim
    HD = H * D
    o = ops()
    idx = input_seq.to(torch.int32).contiguous()
    doc_start, doc_end = model.document_bounds(input_seq)
    windows = model.layer_windows(swb)
    enc = model.num_encoder_layers
    ve_map = model.value_embeds.layer_map()

    def w16(p):
        return shadow_of(p, torch.bfloat16)

    # ------------------------------------------------------------------ forward
    x0 = Fz.embed_gather(idx, model.embed.weight, normalize=True)
    ves = [Fz.embed_gather(idx, e.weight) for e in model.value_embeds.embed]
    cos = sin = None
    for blk in model.blocks:
        if blk.attn is not None:
            cos, sin = blk.attn.rotary.cos, blk.attn.rotary.sin
            break
    saved: list[_Saved] = []
    skips: list[tuple[int, Tensor]] = []
    x = x0
    for i, blk in enumerate(model.blocks):
        s = _Saved()
        s.x_in = x
        s.skip, s.skip_idx = None, -1
        skip_w = None
        if i >= enc:
            s.skip_idx, s.skip = skips.pop()
            skip_w = model.skip_weights[i - enc:i - enc + 1]
        s.x_mix, s.xn = Fz.mix_norm(x, x0, blk.lambdas, s.skip, skip_w, EPS)
        if blk.attn is not None:
            a = blk.attn
            s.qkv = G.gemm(s.xn, w16(a.qkv_w).view(3 * HD, C))
            s.qkvp = torch.empty_like(s.qkv)
            ve = ves[ve_map[i]] if ve_map[i] is not None else None
            o.qkv_post_fwd(s.qkv, ve, a.lambdas, cos, sin, s.qkvp, H, D, EPS)
            q4 = s.qkvp.view(T, 3, H, D)
            s.y, s.lse = flash_attention_forward(q4[:, 0], q4[:, 1], q4[:, 2], doc_start, doc_end, a.attn_scale, windows[i])
            s.x_a = G.gemm(s.y.view(T, HD), w16(a.c_proj.weight), epilogue=G.EPI_AXPBY, aux=s.x_mix, beta=1.0)
        else:
            s.qkv = s.qkvp = s.y = s.lse = None
            s.x_a = s.x_mix
        s.xn2 = Fz.rmsnorm(s.x_a, EPS)
        s.h = G.gemm(s.xn2, w16(blk.mlp.c_fc.weight), epilogue=G.EPI_RELU2)
        x = G.gemm(s.h, w16(blk.mlp.c_proj.weight), epilogue=G.EPI_AXPBY, aux=s.x_a, beta=1.0)
        if i < enc:
            skips.append((i, x))
        saved.append(s)
    x_last = x
    xf = Fz.rmsnorm(x_last, EPS)
    head = model.lm_head
    V = head.weight.shape[0]
    if head.use_fp8:
        x8 = Fz.cast_fp8(xf, head.x_s, torch.float8_e4m3fn)
        w8 = shadow_of(head.weight, torch.float8_e4m3fn, head.w_s)
        logits = G.gemm(x8, w8, alpha=1.0 / (head.x_s * head.w_s))
    else:
        x8 = w8 = None
        logits = G.gemm(xf, w16(head.weight))
    grad_s = head.grad_s if head.use_fp8 else 1.0
    gl = None
    if need_grad:
        gl = torch.empty(T, V, dtype=torch.float8_e5m2 if head.use_fp8 else torch.bfloat16, device=dev)
    loss_rows = Fz.softcap_ce(logits, target_seq, gl, c.softcap, c.softcap_div, 1.0, grad_s / T)
    loss = loss_rows.mean()
    if not need_grad:
        return loss, None
    del logits

    # ------------------------------------------------------------------ backward
    grads: dict[int, Tensor] = {}
    # Optional hand-over to a distributed optimizer: ``model._grad_out`` maps id(param) -> a preallocated gradient
    # buffer (e.g. a view of a peer-mapped bucket) that the producing kernel writes directly; ``model._grad_hooks``
    # maps id(param) -> callable(param, grad) invoked as soon as that gradient is complete (the head's is at the very
    # start of backward, so its collective overlaps everything below). A buffer is only used while the parameter
    # holds no gradient yet (with gradient accumulation the second micro-batch must not overwrite the first).
    grad_out = getattr(model, "_grad_out", None) or {}
    grad_hooks = getattr(model, "_grad_hooks", None) or {}

    def out_buf(p):
        return grad_out.get(id(p)) if p.grad is None else None

    def new_grad(p):
        # embedding gradients are accumulated by fp32 atomics whatever the table's dtype; the cast to the parameter's
        # dtype at the end of the step lands in the hand-over buffer (see fused_gpt_step)
        return torch.zeros(p.shape, dtype=torch.float32, device=dev)

    def put(p, g):
        grads[id(p)] = g if id(p) not in grads else grads[id(p)] + g
        hook = grad_hooks.get(id(p))
        if hook is not None:
            hook(p, grads[id(p)])

    if head.use_fp8:
        dxf = G.gemm(gl, w8, b_mn=True, alpha=1.0 / (grad_s * head.w_s))
        put(head.weight, G.gemm(gl, x8, a_mn=True, b_mn=True, out=out_buf(head.weight), out_dtype=torch.float32,
                                alpha=1.0 / (grad_s * head.x_s)))
    else:
        dxf = G.gemm(gl, w16(head.weight), b_mn=True)
        put(head.weight, _wgrad(gl, xf, head.weight.shape))
    del gl
    dx = Fz.norm_bwd_add(dxf, x_last, None, EPS)

    dx0_acc = torch.zeros(T, C, dtype=torch.float32, device=dev)
    dskip_w = torch.zeros_like(model.skip_weights)
    dskips: dict[int, Tensor] = {}
    ve_grads = [None] * len(model.value_embeds.embed)
    dve_wait: dict[int, Tensor] = {}
    dq_acc = None
    for i in reversed(range(len(model.blocks))):
        blk, s = model.blocks[i], saved[i]
        if i in dskips:
            dx = dx + dskips.pop(i)
        mlp = blk.mlp
        dpre = G.gemm(dx, w16(mlp.c_proj.weight), b_mn=True, epilogue=G.EPI_RELU2_BWD, aux=s.h)
        put(mlp.c_proj.weight, _wgrad(dx, s.h, mlp.c_proj.weight.shape, out_buf(mlp.c_proj.weight)))
        dxn2 = G.gemm(dpre, w16(mlp.c_fc.weight), b_mn=True)
        put(mlp.c_fc.weight, _wgrad(dpre, s.xn2, mlp.c_fc.weight.shape, out_buf(mlp.c_fc.weight)))
        del dpre
        dx_a = Fz.norm_bwd_add(dxn2, s.x_a, dx, EPS)
        if blk.attn is not None:
            a = blk.attn
            dy = G.gemm(dx_a, w16(a.c_proj.weight), b_mn=True)
            put(a.c_proj.weight, _wgrad(dx_a, s.y.view(T, HD), a.c_proj.weight.shape, out_buf(a.c_proj.weight)))
            q4 = s.qkvp.view(T, 3, H, D)
            if dq_acc is None:
                dq_acc = torch.zeros(T, H, D, dtype=torch.float32, device=dev)
            else:
                dq_acc.zero_()
            dq, dk, dv = flash_attention_backward(q4[:, 0], q4[:, 1], q4[:, 2], s.y, dy.view(T, H, D), s.lse, doc_start,
                                                  doc_end, a.attn_scale, windows[i], dq_acc)
            dqkv = torch.empty_like(s.qkv)
            vi = ve_map[i]
            ve = ves[vi] if vi is not None else None
            dve = torch.empty(T, HD, dtype=torch.bfloat16, device=dev) if ve is not None else None
            dlam = torch.zeros(2, dtype=torch.float32, device=dev)
            o.qkv_post_bwd(dq, dk, dv, s.qkv, ve, a.lambdas, cos, sin, dqkv, dve, dlam, H, D, EPS)
            put(a.lambdas, dlam)
            if dve is not None:
                # a value embedding feeds several layers: the first gradient waits for the next one and the two are
                # summed inside one scatter; what is still waiting at the end is flushed below
                if vi in dve_wait:
                    if ve_grads[vi] is None:
                        ve_grads[vi] = new_grad(model.value_embeds.embed[vi].weight)
                    o.embed_scatter_add(idx, dve, ve_grads[vi], dve_wait.pop(vi))
                else:
                    dve_wait[vi] = dve
            dxn = G.gemm(dqkv, w16(a.qkv_w).view(3 * HD, C), b_mn=True)
            put(a.qkv_w, _wgrad(dqkv, s.xn, a.qkv_w.shape, out_buf(a.qkv_w)))
            dx_mix = Fz.norm_bwd_add(dxn, s.x_mix, dx_a, EPS)
        else:
            dx_mix = dx_a
        dx_prev = torch.empty_like(dx_mix)
        dlam_b = torch.zeros(2, dtype=torch.float32, device=dev)
        # the skip gradient waiting for the layer below is added inside this kernel, before dx_prev is rounded
        add_in = dskips.pop(i - 1, None)
        if s.skip is not None:
            dsk = torch.empty_like(dx_mix)
            j = i - enc
            o.mix_bwd(dx_mix, s.x_in, x0, s.skip, blk.lambdas, model.skip_weights[j:j + 1], dx_prev, dsk, dx0_acc, dlam_b,
                      dskip_w[j:j + 1], add_in)
            dskips[s.skip_idx] = dsk
        else:
            o.mix_bwd(dx_mix, s.x_in, x0, None, blk.lambdas, None, dx_prev, None, dx0_acc, dlam_b, None, add_in)
        put(blk.lambdas, dlam_b)
        dx = dx_prev
        saved[i] = None
    put(model.skip_weights, dskip_w)
    # embedding: x0 = rmsnorm(embed[idx]) receives the first block's input gradient plus every lambda[1] path
    dx0_total = (dx0_acc + dx.float()).to(torch.bfloat16)
    e_raw = Fz.embed_gather(idx, model.embed.weight)
    d_e = Fz.norm_bwd_add(dx0_total, e_raw, None, EPS)
    g_embed = new_grad(model.embed.weight)
    o.embed_scatter_add(idx, d_e, g_embed)
    put(model.embed.weight, g_embed)
    for vi, dve in dve_wait.items():
        if ve_grads[vi] is None:
            ve_grads[vi] = new_grad(model.value_embeds.embed[vi].weight)
        o.embed_scatter_add(idx, dve, ve_grads[vi])
    for vi, e in enumerate(model.value_embeds.embed):
        if ve_grads[vi] is not None:
            put(e.weight, ve_grads[vi])
    return loss, grads


class _FusedGPTLoss(torch.autograd.Function):
    @staticmethod
    def forward(ctx, model, input_seq, target_seq, swb, need_grad, *params):
        loss, grads = _forward_backward(model, input_seq, target_seq, swb, need_grad)
        ctx.grads = grads
        ctx.params = params
        return loss

    @staticmethod
    def backward(ctx, grad_out):
        if ctx.grads is None:
            raise RuntimeError("fused GPT loss was computed without gradients (torch.no_grad())")
        out, present = [], []
        for p in ctx.params:
            g = ctx.grads.get(id(p))
            if g is not None:
                g = g.view(p.shape)
                present.append(g)
            out.append(g)
        # every gradient is linear in the incoming loss gradient (a device scalar): one multi-tensor multiply
        if present:
            try:
                torch._foreach_mul_(present, grad_out)
            except (RuntimeError, TypeError):
                for g in present:
                    g.mul_(grad_out)
        out = [g if g is None or g.dtype == p.dtype else g.to(p.dtype) for g, p in zip(out, ctx.params)]
        ctx.grads = None
        return (None, None, None, None, None, *out)


def fused_gpt_loss(model, input_seq: Tensor, target_seq: Tensor, swb: int) -> Tensor:
    params = [p for p in model.parameters() if p.requires_grad]
    need_grad = torch.is_grad_enabled() and len(params) > 0
    return _FusedGPTLoss.apply(model, input_seq, target_seq, swb, need_grad, *params)


def fused_gpt_step(model, input_seq: Tensor, target_seq: Tensor, swb: int) -> Tensor:
    """Loss of one training step with the parameter gradients written straight into ``p.grad`` (accumulated when a
    gradient is already there): what ``fused_gpt_loss(...).backward()`` produces, without the autograd node and its
    multiply of every gradient by the incoming loss gradient (which is 1 for a plain ``backward()``)."""
    loss, grads = _forward_backward(model, input_seq, target_seq, swb, True)
    grad_out = getattr(model, "_grad_out", None) or {}
    for p in model.parameters():
        if not p.requires_grad:
            continue
        g = grads.get(id(p))
        if g is None:
            continue
        g = g.view(p.shape)
        buf = grad_out.get(id(p)) if p.grad is None else None
        if buf is not None and buf.data_ptr() != g.data_ptr():
            buf.copy_(g)                      # cast (if any) and hand-over in one pass
            g = buf
        elif g.dtype != p.dtype:
            g = g.to(p.dtype)
        if p.grad is None:
            p.grad = g
        else:
            p.grad.add_(g)
    return loss.detach()
