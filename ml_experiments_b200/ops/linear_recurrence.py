"""Matrix-state linear recurrences of the recall-harness mixers, in chunk-parallel form (batched GEMMs) with step-by-step
oracles. State ``S [dk, dv]`` per (batch, head); inputs ``[B, T, H, d]``.

* gated linear attention  ``S_t = diag(exp(g_t)) S_{t-1} + k_tᵀ v_t``, ``o_t = q_t S_t``
  (the ``chunk_gla`` / ``fused_recurrent_gla`` calls of zoology/mixers/gla.py:227-257);
* (gated) delta rule      ``S_t = a_t (I - b_t k_tᵀ k_t) S_{t-1} + b_t k_tᵀ v_t`` with scalar ``a_t = exp(g_t)``
  (``chunk_delta_rule``, zoology/mixers/delta_net.py:247-270; ``chunk_gated_delta_rule``, gated_delta_net.py:229-253);
* diagonal-plus-low-rank  ``S_t = S_{t-1} (diag(exp(w_t)) + a_tᵀ b_t) + v_tᵀ k_t`` (RWKV-7, zoology/mixers/rwkv7.py:178-190),
  time-stepped.

The reference takes these from the external ``fla`` Triton package; here they are restated on PyTorch GEMMs.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def _pad_chunks(t, C):
    T = t.shape[1]
    pad = (-T) % C
    return F.pad(t, (0, 0) * (t.dim() - 2) + (0, pad)) if pad else t


# ------------------------------------------------------------------------------------------------ GLA
def gla_recurrent(q, k, v, g, scale=None, initial_state=None):
    B, T, H, dk = q.shape
    scale = dk ** -0.5 if scale is None else scale
    S = q.new_zeros(B, H, dk, v.shape[-1], dtype=torch.float32) if initial_state is None else initial_state.float()
    out = []
    for t in range(T):
        S = S * g[:, t].float().exp().unsqueeze(-1) + k[:, t].float().unsqueeze(-1) * v[:, t].float().unsqueeze(-2)
        out.append(torch.einsum("bhk,bhkv->bhv", q[:, t].float() * scale, S))
    return torch.stack(out, 1).to(v.dtype), S


def chunk_gla(q, k, v, g, scale=None, initial_state=None, chunk: int = 64, sub: int = 16):
    """``g`` = per-key-channel log decay (<= 0). Two-level chunking: inside a chunk, sub-block pairs are evaluated
    relative to the first row of the query sub-block so every exponent is <= 0."""
    B, T, H, dk = q.shape
    dv = v.shape[-1]
    scale = dk ** -0.5 if scale is None else scale
    C = min(chunk, max(sub, (T + sub - 1) // sub * sub))
    qf, kf, vf, gf = (_pad_chunks(t.float(), C) for t in (q, k, v, g))
    N = qf.shape[1] // C
    r = lambda t: t.view(B, N, C, H, -1).permute(0, 3, 1, 2, 4)  # [B,H,N,C,d]
    qf, kf, vf, gf = r(qf) * scale, r(kf), r(vf), r(gf)
    G = gf.cumsum(-2)                                              # inclusive
    Gend = G[..., -1:, :]
    # intra-chunk scores
    A = qf.new_zeros(B, H, N, C, C)
    ns = C // sub
    for I in range(ns):
        sl = slice(I * sub, (I + 1) * sub)
        ref = G[..., I * sub:I * sub + 1, :]
        qi = qf[..., sl, :] * (G[..., sl, :] - ref).exp()
        if I > 0:
            kj = kf[..., :I * sub, :] * (ref - G[..., :I * sub, :]).exp()
            A[..., sl, :I * sub] = qi @ kj.transpose(-1, -2)
        d = (G[..., sl, None, :] - G[..., None, sl, :])           # [.., sub, sub, dk]
        tri = torch.ones(sub, sub, device=q.device, dtype=torch.bool).tril()
        d = d.masked_fill(~tri[..., None], float("-inf"))
        A[..., sl, sl] = torch.einsum("...id,...ijd,...jd->...ij", qf[..., sl, :], d.exp(), kf[..., sl, :])
    o = A @ vf
    # inter-chunk
    k_end = kf * (Gend - G).exp()
    dS = k_end.transpose(-1, -2) @ vf                              # [B,H,N,dk,dv]
    decay = Gend.squeeze(-2).exp()                                 # [B,H,N,dk]
    S = qf.new_zeros(B, H, dk, dv) if initial_state is None else initial_state.float()
    states = []
    for n in range(N):
        states.append(S)
        S = S * decay[:, :, n].unsqueeze(-1) + dS[:, :, n]
    S0 = torch.stack(states, 2)
    o = o + (qf * G.exp()) @ S0
    o = o.permute(0, 2, 3, 1, 4).reshape(B, N * C, H, dv)[:, :T]
    if N * C != T:  # the padded tail (g = 0, k = 0) left the state untouched
        pass
    return o.to(v.dtype), S


# ------------------------------------------------------------------------------------------------ delta rule
def delta_rule_recurrent(q, k, v, beta, g=None, scale=None, initial_state=None):
    B, T, H, dk = q.shape
    scale = dk ** -0.5 if scale is None else scale
    S = q.new_zeros(B, H, dk, v.shape[-1], dtype=torch.float32) if initial_state is None else initial_state.float()
    out = []
    for t in range(T):
        kt, vt, bt = k[:, t].float(), v[:, t].float(), beta[:, t].float()[..., None]
        if g is not None:
            S = S * g[:, t].float().exp()[..., None, None]
        u = bt * (vt - torch.einsum("bhk,bhkv->bhv", kt, S))
        S = S + kt.unsqueeze(-1) * u.unsqueeze(-2)
        out.append(torch.einsum("bhk,bhkv->bhv", q[:, t].float() * scale, S))
    return torch.stack(out, 1).to(v.dtype), S


def chunk_delta_rule(q, k, v, beta, g=None, scale=None, initial_state=None, chunk: int = 64):
    """WY-form chunked (gated) delta rule. With ``gamma_i = exp(sum_{j<=i} g_j)`` inside a chunk, the pseudo-values solve
    ``(I + tril(diag(beta) (gamma_i/gamma_j) K Kᵀ, -1)) U = diag(beta) (V - diag(gamma) K S_0)``; then
    ``o_i = gamma_i q_i S_0 + sum_{j<=i} (gamma_i/gamma_j)(q_i.k_j) u_j`` and
    ``S_C = gamma_C S_0 + sum_j (gamma_C/gamma_j) k_jᵀ u_j``."""
    B, T, H, dk = q.shape
    dv = v.shape[-1]
    scale = dk ** -0.5 if scale is None else scale
    C = min(chunk, T)
    qf, kf, vf = (_pad_chunks(t.float(), C) for t in (q, k, v))
    bf = _pad_chunks(beta.float().unsqueeze(-1), C)
    gf = _pad_chunks(g.float().unsqueeze(-1), C) if g is not None else torch.zeros_like(bf)
    N = qf.shape[1] // C
    r = lambda t: t.view(B, N, C, H, -1).permute(0, 3, 1, 2, 4)
    qf, kf, vf, bf, gf = r(qf) * scale, r(kf), r(vf), r(bf), r(gf)
    Gc = gf.cumsum(-2)                                             # [B,H,N,C,1] log gamma
    ratio = (Gc - Gc.transpose(-1, -2))                            # log(gamma_i / gamma_j)
    tri = torch.ones(C, C, device=q.device, dtype=torch.bool).tril()
    ratio = ratio.masked_fill(~tri, float("-inf")).exp()           # zero above the diagonal
    KK = kf @ kf.transpose(-1, -2)
    Amat = (bf * KK * ratio).tril(-1)
    eye = torch.eye(C, device=q.device)
    Tm = torch.linalg.solve_triangular(eye + Amat, eye.expand_as(Amat), upper=False)
    Uv = Tm @ (bf * vf)                                            # T diag(beta) V
    Wk = Tm @ (bf * Gc.exp() * kf)                                 # T diag(beta) diag(gamma) K
    QK = (qf @ kf.transpose(-1, -2)) * ratio                       # lower-triangular incl. diagonal
    k_end = kf * (Gc[..., -1:, :] - Gc).exp()
    q_g = qf * Gc.exp()
    g_end = Gc[..., -1, :].exp().unsqueeze(-1)                     # [B,H,N,1,1]
    S = qf.new_zeros(B, H, dk, dv) if initial_state is None else initial_state.float()
    outs = []
    for n in range(N):
        U = Uv[:, :, n] - Wk[:, :, n] @ S
        outs.append(q_g[:, :, n] @ S + QK[:, :, n] @ U)
        S = S * g_end[:, :, n] + k_end[:, :, n].transpose(-1, -2) @ U
    o = torch.stack(outs, 2).permute(0, 2, 3, 1, 4).reshape(B, N * C, H, dv)[:, :T]
    return o.to(v.dtype), S


# ------------------------------------------------------------------------------------------------ DPLR (RWKV-7)
def dplr_recurrent(r, w, k, v, a, b, scale: float = 1.0, initial_state=None):
    """``S [dv, dk]``: ``S_t = S_{t-1} diag(exp(w_t)) + (S_{t-1} a_t) b_tᵀ + v_t k_tᵀ``; ``o_t = S_t r_t``."""
    B, T, H, dk = r.shape
    S = r.new_zeros(B, H, v.shape[-1], dk, dtype=torch.float32) if initial_state is None else initial_state.float()
    out = []
    wf = w.float().exp()
    for t in range(T):
        Sa = torch.einsum("bhvk,bhk->bhv", S, a[:, t].float())
        S = S * wf[:, t].unsqueeze(-2) + Sa.unsqueeze(-1) * b[:, t].float().unsqueeze(-2) \
            + v[:, t].float().unsqueeze(-1) * k[:, t].float().unsqueeze(-2)
        out.append(torch.einsum("bhvk,bhk->bhv", S, r[:, t].float() * scale))
    return torch.stack(out, 1).to(v.dtype), S
