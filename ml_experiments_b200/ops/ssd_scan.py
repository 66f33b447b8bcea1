"""Chunk-parallel scan for state-space layers with a scalar decay per head (the "SSD" form).

Recurrence, per batch ``b`` and head ``h`` with state ``S [N, P]``::

    S_t = alpha_t * S_{t-1} + gamma_t * B_t (x) x_t + beta_t * B_{t-1} (x) x_{t-1}        y_t = C_t . S_t

``beta`` (the look-back term of the trapezoidal discretisation) is optional. This is the recurrence of the reference's
``SSMMixer3._ssm_scan`` (src/heuristic_secrets/models/backbone.py:1516-1595), which walks the chunks in a Python loop
and materialises the ``[B, L, H, N, P]`` outer products, and of the vendored Mamba-2 ``ssd_combined`` pipeline
(zoology/mixers/mamba_ssm/ops/triton/ssd_combined.py). Here every chunk is processed at once as batched matrix
products that land on the tensor cores -- intra-chunk ``(C B^T o decay) U``, per-chunk end states, a logarithmic-depth
inter-chunk state pass, and the carried-state contribution -- and nothing of size ``L*N*P`` is ever formed.
Differentiable through autograd. ``ssd_scan_ref`` is the sequential fp32 oracle.

On a B200 with bf16 inputs and supported shapes (``L % 128 == 0``, ``N`` and ``P`` in {64, 128}) the forward runs in ONE
hand-written kernel (``csrc/scan/ssd_sm100.cu``): a CTA per (batch, head) walks 128-step chunks with the four
products on tcgen05 and the running state resident in tensor memory. The backward is three more launches of the SAME
kernel (:class:`_SsdKernelGradFn`): the gradients of ``x`` and ``B`` are scans of the same form run backwards in time
with the roles of the operands exchanged, the gradient of ``C`` is one forwards in time, and the gradients of the
decays and weights are row / column sums that follow from ``y``, ``dy``, ``x`` and ``dx`` elementwise. Calls with an
initial or returned state differentiate the batched-GEMM formulation below instead. ``B200_SSD_KERNEL=0`` disables
the kernel path.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def ssd_scan_ref(x, B, C, log_alpha, gamma, beta=None, init_state=None):
    """Sequential oracle. ``x [b,L,H,P]``, ``B,C [b,L,H,N]``, ``log_alpha, gamma, beta [b,L,H]`` -> ``(y, final_state)``."""
    b, L, H, P = x.shape
    N = B.shape[-1]
    xf, Bf, Cf = x.float(), B.float().expand(b, L, H, N), C.float().expand(b, L, H, N)
    S = xf.new_zeros(b, H, N, P) if init_state is None else init_state.float().clone()
    ys = []
    for t in range(L):
        u = gamma[:, t, :, None, None].float() * Bf[:, t, :, :, None] * xf[:, t, :, None, :]
        if beta is not None and t > 0:
            u = u + beta[:, t, :, None, None].float() * Bf[:, t - 1, :, :, None] * xf[:, t - 1, :, None, :]
        S = torch.exp(log_alpha[:, t].float())[:, :, None, None] * S + u
        ys.append(torch.einsum("bhnp,bhn->bhp", S, Cf[:, t]))
    return torch.stack(ys, 1).to(x.dtype), S


def _decay_matrix(cs):
    """``cs [..., Q]`` inclusive cumulative log-decay -> ``exp(cs_i - cs_j)`` for ``i >= j`` else 0, ``[..., Q, Q]``."""
    Q = cs.shape[-1]
    d = cs.unsqueeze(-1) - cs.unsqueeze(-2)
    keep = torch.ones(Q, Q, dtype=torch.bool, device=cs.device).tril()
    return torch.exp(d.masked_fill(~keep, float("-inf")))


def _exclusive_state_pass(log_a, s, s0=None, block: int = 64):
    """Linear recurrence over dim 1: ``S_in[c+1] = exp(log_a[c]) * S_in[c] + s[c]`` with ``S_in[0] = s0``.

    ``log_a [b, n, H]``, ``s [b, n, H, D]`` -> ``(S_in [b, n, H, D], S_final [b, H, D])``. Blocks of ``block`` steps are
    solved with a decay matrix; block totals recurse, so the depth is ``log_block(n)``.
    """
    b, n, H, D = s.shape
    if n <= block:
        cs = torch.cumsum(log_a.float(), dim=1)  # inclusive
        M = _decay_matrix(cs.transpose(1, 2))  # [b, H, n, n]: exp(cs_i - cs_j), i >= j
        # state after step i (inclusive) = sum_{j<=i} exp(cs_i - cs_j) s_j  (+ exp(cs_i) s0)
        incl = torch.einsum("bhij,bjhd->bihd", M.to(s.dtype), s)
        if s0 is not None:
            incl = incl + torch.exp(cs).to(s.dtype).unsqueeze(-1) * s0.unsqueeze(1)
        first = torch.zeros_like(s[:, :1]) if s0 is None else s0.unsqueeze(1)
        return torch.cat([first, incl[:, :-1]], dim=1), incl[:, -1]
    pad = (-n) % block
    if pad:
        log_a = F.pad(log_a, (0, 0, 0, pad))
        s = F.pad(s, (0, 0, 0, 0, 0, pad))
    nb = (n + pad) // block
    la = log_a.view(b, nb, block, H)
    sb = s.view(b, nb, block, H, D)
    # within-block inclusive states from a zero start, all blocks at once
    cs = torch.cumsum(la.float(), dim=2)
    M = _decay_matrix(cs.permute(0, 1, 3, 2))  # [b, nb, H, blk, blk]
    incl = torch.einsum("bchij,bcjhd->bcihd", M.to(s.dtype), sb)
    tot_log = cs[:, :, -1]  # [b, nb, H]
    carry_in, final = _exclusive_state_pass(tot_log, incl[:, :, -1], s0, block)  # state entering each block
    incl = incl + torch.exp(cs).to(s.dtype).unsqueeze(-1) * carry_in.unsqueeze(2)
    first = carry_in.unsqueeze(2)
    excl = torch.cat([first, incl[:, :, :-1]], dim=2).reshape(b, nb * block, H, D)[:, :n]
    if pad:  # padded steps have log_a = 0, s = 0: the state is unchanged, `final` is already right
        pass
    return excl, final


def kernel_supported(x, B, C) -> bool:
    """True when the tcgen05 kernel takes this call: CUDA, supported shapes, and bf16 compute asked for (bf16 inputs, or
    fp32 / fp16 inputs inside a bf16 autocast region: the operands are then rounded to bf16 for the tensor cores, the
    state and all accumulations stay fp32)."""
    import os

    if not x.is_cuda or os.environ.get("B200_SSD_KERNEL", "1") != "1" or B.shape != C.shape or x.dim() != 4 or B.dim() != 4:
        return False
    bf16_compute = x.dtype == torch.bfloat16 or (torch.is_autocast_enabled() and torch.get_autocast_gpu_dtype() == torch.bfloat16)
    b, L, H, P = x.shape
    Hb = B.shape[2]
    return bf16_compute and L % 128 == 0 and B.shape[-1] in (64, 128) and P in (64, 128) and Hb > 0 and H % Hb == 0


def _fold_weights(log_alpha, gamma, beta):
    """``(g_off, g_diag)`` of the kernel: the look-back term ``beta_t B_{t-1} x_{t-1}`` is the outer product of step
    ``t-1`` entering one step late and without that step's decay, i.e. weight ``beta_t / alpha_t`` on top of
    ``gamma_{t-1}`` for every later output and for the state."""
    g = gamma.float()
    if beta is None:
        return g.contiguous(), g.contiguous()
    late = beta.float() * torch.exp(-log_alpha.float().clamp_min(-80.0))
    return (g + F.pad(late[:, 1:], (0, 0, 0, 1))).contiguous(), g.contiguous()


def ssd_forward_kernel(x, B, C, log_alpha, gamma, beta=None, init_state=None, return_state: bool = False):
    """Forward only, on the tcgen05 kernel. Shapes as :func:`ssd_chunk_scan`; ``x, B, C`` bf16."""
    from .runtime import ops, status

    g_off, g_diag = _fold_weights(log_alpha, gamma, beta)
    out_dtype = x.dtype
    x, B, C = (t if t.dtype == torch.bfloat16 else t.to(torch.bfloat16) for t in (x, B, C))
    y = torch.empty_like(x)
    b, L, H, P = x.shape
    N = B.shape[-1]
    fin = torch.empty(b, H, N, P, dtype=torch.float32, device=x.device) if return_state else None
    init = None if init_state is None else init_state.float().contiguous()
    ops().ssd_fwd(x.contiguous(), B.contiguous(), C.contiguous(), log_alpha.float().contiguous(), g_off, g_diag, y, init, fin,
                  status(x.device))
    if y.dtype != out_dtype:
        y = y.to(out_dtype)
    return (y, fin) if return_state else y


_Q = 128      # steps per chunk of the kernel


def _launch(x, B, C, log_a, g_off, g_diag, states: bool = False):
    """One launch of the kernel; with ``states`` also the fp32 state after every 128-step chunk ``[b, H, L/128, N, P]``."""
    from .runtime import add_launches, ops, status

    y = torch.empty_like(x)
    b, L, H, P = x.shape
    st = torch.empty(b, H, L // _Q, B.shape[-1], P, dtype=torch.float32, device=x.device) if states else None
    ops().ssd_fwd(x, B, C, log_a, g_off, g_diag, y, None, None, status(x.device), st)
    add_launches(1)
    return (y, st) if states else y


class _SsdKernelGradFn(torch.autograd.Function):
    """``y_i = g_diag_i (C_i.B_i) x_i + sum_{j<i} exp(cs_i - cs_j) g_off_j (C_i.B_j) x_j`` with ``cs`` the running sum of
    ``log_a``; forward and backward on the tcgen05 kernel.

    With ``E_ij = exp(cs_i - cs_j) (C_i.B_j)`` for ``j < i``:

    * ``dx_j = g_off_j sum_{i>j} E_ij dy_i + diag``: the same scan backwards in time, "queries" ``B``, "keys" ``C``,
      values ``dy`` (the decay between reversed neighbours ``t'-1, t'`` is ``log_a`` of the later original step);
    * ``dC_i = sum_{j<i} E_ij g_off_j (dy_i.x_j) B_j + diag``: forwards in time, queries ``dy``, keys ``x``, values ``B``
      (state of shape ``[P, N]`` instead of ``[N, P]``);
    * ``dB_j = g_off_j sum_{i>j} E_ij (dy_i.x_j) C_i + diag``: backwards in time, queries ``x``, keys ``dy``, values ``C``;
    * ``d g_off_j = x_j . DX_j`` with ``DX`` the first scan before its ``g_off`` factor, ``d g_diag_i = (C_i.B_i)(dy_i.x_i)``;
    * every pair ``j < t <= i`` sees ``log_a_t``, so ``d log_a_t = sum_{i>=t} R_i - sum_{j>=t} K_j`` with the row sums
      ``R_i = dy_i . (y_i - diag_i)`` and column sums ``K_j = g_off_j d g_off_j`` (pairs on one side of ``t`` cancel).
      The cancellation is only left to the sums inside a chunk: the part of later chunks is the number of pairs that
      straddle the chunk's end, and that is the inner product of the forward state at that boundary with the state of
      the backwards-in-time scan there (both are written by the kernel in fp32), so the rounding noise of ``y`` and
      ``dx`` (bf16) does not accumulate along the sequence.
    """

    @staticmethod
    def forward(ctx, x, B, C, log_a, g_off, g_diag):
        bf = lambda t: (t if t.dtype == torch.bfloat16 else t.to(torch.bfloat16)).contiguous()
        f32 = lambda t: t.float().contiguous()
        xb, Bb, Cb, la, go, gd = bf(x), bf(B), bf(C), f32(log_a), f32(g_off), f32(g_diag)
        need_grad = any(t.requires_grad for t in (x, B, C, log_a, g_off, g_diag))
        y, S = _launch(xb, Bb, Cb, la, go, gd, states=True) if need_grad else (_launch(xb, Bb, Cb, la, go, gd), None)
        ctx.save_for_backward(xb, Bb, Cb, la, go, gd, y, S)
        ctx.dtypes = (x.dtype, B.dtype, C.dtype, log_a.dtype, g_off.dtype, g_diag.dtype)
        return y if y.dtype == x.dtype else y.to(x.dtype)

    @staticmethod
    def backward(ctx, dy):
        from .runtime import add_launches, ops

        x, B, C, la, go, gd, y, S = ctx.saved_tensors
        b, L, H, P = x.shape
        Hb, N = B.shape[2], B.shape[3]
        rep = H // Hb
        o = ops()
        flip = o.ssd_flip_time                                   # time reversal of a contiguous [b, L, ...] tensor
        dyb = dy.to(torch.bfloat16).contiguous()
        heads = lambda t: t if rep == 1 else t.repeat_interleave(rep, dim=2).contiguous()
        ones, zeros = torch.ones_like(la), torch.zeros_like(la)
        la_r = torch.cat([zeros[:, :1], la[:, 1:].flip(1)], dim=1).contiguous()   # decay between reversed neighbours
        dy_r, B_r, C_r = flip(dyb), flip(B), flip(C)
        dx_rev, Lam = _launch(dy_r, C_r, B_r, la_r, ones, zeros, states=True)                     # [b, L, H, P], reversed
        dC_h = _launch(heads(B), x, dyb, la, go, gd)                                              # [b, L, H, N]
        dB_rev = _launch(heads(C_r), dy_r, flip(x), la_r, ones, zeros)                            # [b, L, H, N], reversed
        dx, dB, dC = torch.empty_like(x), torch.empty_like(B), torch.empty_like(C)
        d_goff, d_gdiag, inner = torch.empty_like(la), torch.empty_like(la), torch.empty_like(la)
        o.ssd_bwd_post(x, dyb, y, dx_rev, dB_rev, dC_h, B, C, go, gd, dx, dB, dC, d_goff, d_gdiag, inner)
        add_launches(5)
        nc = L // _Q
        inner = inner.view(b, nc, _Q, H).flip(2).cumsum(2).flip(2)                                # sums to the chunk's end
        if nc > 1:
            # pairs (i, j) on the two sides of the boundary after chunk c: <forward state after c, backwards state
            # reaching the first step of chunk c+1> times that step's decay
            pairs = (S[:, :, :nc - 1] * Lam[:, :, :nc - 1].flip(2)).sum((-1, -2)).permute(0, 2, 1)          # [b, nc-1, H]
            later = torch.cat([torch.exp(la[:, _Q::_Q]) * pairs, zeros[:, :1]], dim=1)
            inner = inner + later.unsqueeze(2)
        d_la = inner.reshape(b, L, H)
        outs = (dx, dB, dC, d_la, d_goff, d_gdiag)
        return tuple(t.to(dt) if need else None for t, dt, need in zip(outs, ctx.dtypes, ctx.needs_input_grad))


class _SsdKernelFn(torch.autograd.Function):
    """Kernel forward; backward = autograd through the batched-GEMM formulation on the saved inputs."""

    @staticmethod
    def forward(ctx, x, B, C, log_alpha, gamma, beta, init_state, return_state):
        ctx.save_for_backward(x, B, C, log_alpha, gamma, beta, init_state)
        ctx.return_state = return_state
        out = ssd_forward_kernel(x, B, C, log_alpha, gamma, beta, init_state, return_state)
        return out if return_state else (out, None)

    @staticmethod
    def backward(ctx, dy, dstate):
        saved = ctx.saved_tensors
        with torch.enable_grad():
            ins = [None if t is None else t.detach().requires_grad_(t.is_floating_point()) for t in saved]
            x, B, C, la, g, bt, s0 = ins
            out = _ssd_chunk_scan_torch(x, B, C, la, g, bt, 64, s0, ctx.return_state)
            y, st = out if ctx.return_state else (out, None)
            outs, gouts = [y], [dy]
            if st is not None and dstate is not None:
                outs.append(st)
                gouts.append(dstate.to(st.dtype))
            need = [t for t, n in zip(ins, ctx.needs_input_grad[:7]) if t is not None and n]
            grads = iter(torch.autograd.grad(outs, need, gouts, allow_unused=True))
        res = [next(grads) if (t is not None and n) else None for t, n in zip(ins, ctx.needs_input_grad[:7])]
        return (*res, None)


def ssd_chunk_scan(x, B, C, log_alpha, gamma, beta=None, chunk: int = 64, init_state=None, return_state: bool = False):
    """Chunk-parallel evaluation of the recurrence in the module docstring.

    ``x [b,L,H,P]``; ``B, C [b,L,H,N]`` (a size-1 head dim broadcasts: grouped B/C); ``log_alpha, gamma, beta [b,L,H]``.
    Returns ``y [b,L,H,P]`` (and the final state ``[b,H,N,P]`` if ``return_state``).
    """
    if kernel_supported(x, B, C):
        if init_state is None and not return_state:
            g_off, g_diag = _fold_weights(log_alpha, gamma, beta)      # differentiable: beta's look-back folds into g_off
            return _SsdKernelGradFn.apply(x, B, C, log_alpha, g_off, g_diag)
        y, st = _SsdKernelFn.apply(x, B, C, log_alpha, gamma, beta, init_state, return_state)
        return (y, st) if return_state else y
    return _ssd_chunk_scan_torch(x, B, C, log_alpha, gamma, beta, chunk, init_state, return_state)


def _ssd_chunk_scan_torch(x, B, C, log_alpha, gamma, beta=None, chunk: int = 64, init_state=None, return_state: bool = False):
    b, L, H, P = x.shape
    N = B.shape[-1]
    B = B.expand(b, L, H, N)
    C = C.expand(b, L, H, N)
    dt = x.dtype
    u1 = gamma.to(dt).unsqueeze(-1) * x
    if beta is not None:
        u2 = beta.to(dt).unsqueeze(-1) * F.pad(x[:, :-1], (0, 0, 0, 0, 1, 0))
        Bp = F.pad(B[:, :-1], (0, 0, 0, 0, 1, 0))
    pad = (-L) % chunk
    if pad:
        padl = lambda t: F.pad(t, (0, 0) * (t.dim() - 2) + (0, pad))
        u1, B, C, log_alpha = padl(u1), padl(B), padl(C), padl(log_alpha)
        if beta is not None:
            u2, Bp = padl(u2), padl(Bp)
    nc, Q = (L + pad) // chunk, chunk
    c5 = lambda t: t.reshape(b, nc, Q, H, t.shape[-1]).permute(0, 1, 3, 2, 4)  # [b, nc, H, Q, *]
    Cc, Bc, U1 = c5(C), c5(B), c5(u1)
    cs = torch.cumsum(log_alpha.float().view(b, nc, Q, H).permute(0, 1, 3, 2), dim=-1)  # [b, nc, H, Q]
    dec = _decay_matrix(cs).to(dt)
    to_end = torch.exp(cs[..., -1:] - cs).to(dt).unsqueeze(-1)  # decay from step j to the chunk end
    y = torch.matmul(torch.matmul(Cc, Bc.transpose(-1, -2)) * dec, U1)
    S = torch.matmul((Bc * to_end).transpose(-1, -2), U1)  # [b, nc, H, N, P]
    if beta is not None:
        Bpc, U2 = c5(Bp), c5(u2)
        y = y + torch.matmul(torch.matmul(Cc, Bpc.transpose(-1, -2)) * dec, U2)
        S = S + torch.matmul((Bpc * to_end).transpose(-1, -2), U2)
    s0 = None if init_state is None else init_state.to(dt).reshape(b, H, N * P)
    S_in, S_fin = _exclusive_state_pass(cs[..., -1], S.reshape(b, nc, H, N * P), s0)
    S_in = S_in.view(b, nc, H, N, P)
    y = y + torch.exp(cs).to(dt).unsqueeze(-1) * torch.matmul(Cc, S_in)
    y = y.permute(0, 1, 3, 2, 4).reshape(b, nc * Q, H, P)[:, :L]
    if return_state:
        return y, S_fin.view(b, H, N, P)
    return y
