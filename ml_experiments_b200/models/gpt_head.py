"""The current (HEAD) speedrun GPT: 11 layers, d = 768, 6 heads x 128, parameter banks, paired-head attention, bigram
hash embedding, gated value embeddings, smear / skip / back-out gates, fp8 transposed lm_head and the multi-token
soft-capped loss (modded-nanogpt/train_gpt.py:916-1300).

Differences in mechanism, not in function: attention runs on this package's flash kernel with per-token document
bounds derived from ``seqlens`` (the reference calls a Hopper FlashAttention-3 binary with ``cu_seqlens``); the paired
heads are the same kernel on the ``2T``-token interleaved view; the linear layers are the tcgen05 GEMM autograd ops
(ReLU^2 fused into the epilogue); nothing is traced or compiled. Parameter names, shapes, labels and the ``reshape``
hints on the banks match, so the optimizer tables and checkpoints carry over.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops.attention import attention_reference, flash_attention
from ..ops.fp8_linear import CastedLinearT, head_ce_loss
from ..ops.fused import embedding, softcapped_cross_entropy
from ..ops.linear import linear, linear_t, mlp_relu2
from ..ops.norm_act import rms_norm_act, rms_norm_act_skip
from ..ops.norm_rope import norm_rotary
from ..ops.rowops import lincomb3, rowscale_add

BLOCK = 128  # attention block / window granularity in tokens


_ONES: dict = {}


def _ones(n: int, device) -> torch.Tensor:
    key = (n, str(device))
    if key not in _ONES:
        _ONES[key] = torch.ones(n, device=device)
    return _ONES[key]


def norm(x):
    if x.is_cuda and x.dtype == torch.bfloat16:   # weightless RMSNorm on the row kernel (unit weights, eps of the dtype)
        return rms_norm_act(x, _ones(x.size(-1), x.device), torch.finfo(x.dtype).eps)
    return F.rms_norm(x, (x.size(-1),))


def norm_skip(x, lead_cols: int = 0):
    """``(norm(x), x[, norm(x)[..., :lead_cols]])`` for ``x + f(norm(x))``: on CUDA the skip's gradient (and that of the
    leading columns, the gates' input) joins the norm's in one backward kernel."""
    if x.is_cuda and x.dtype == torch.bfloat16:
        return rms_norm_act_skip(x, _ones(x.size(-1), x.device), torch.finfo(x.dtype).eps, lead_cols=lead_cols)
    h = F.rms_norm(x, (x.size(-1),))
    return (h, x, h[..., :lead_cols]) if lead_cols else (h, x)


def next_multiple_of_n(v, *, n: int) -> int:
    return -(-int(v) // n) * n


@dataclass
class ForwardScheduleConfig:
    mtp_weights: torch.Tensor | None
    ws_short: int
    ws_long: int


class Yarn(nn.Module):
    """Half-truncated rotary tables (``cos``, sign-alternated ``sin``) applied as ``f1 * x + f2 * flip_pairs(x)``, with the
    YaRN frequency rescale at window changes. ``paired`` builds the tables of the paired-head layout, where one row
    holds the even and the odd interleaved position side by side."""

    def __init__(self, head_dim: int, max_seq_len: int, paired: bool = False, block_size: int = BLOCK):
        super().__init__()
        self.head_dim, self.max_seq_len, self.paired, self.block_size = head_dim, max_seq_len, paired, block_size
        self.register_buffer("factor1", torch.empty(0), persistent=False)
        self.register_buffer("factor2", torch.empty(0), persistent=False)
        self.reset()

    def _tables(self):
        dev = self.angular_freq.device
        t = torch.arange(2 * self.max_seq_len, dtype=torch.float32, device=dev)
        if self.paired:
            th = torch.cat((torch.outer(2 * t, self.angular_freq), torch.outer(2 * t + 1, self.angular_freq)), dim=-1)
        else:
            th = torch.outer(t, self.angular_freq)
        f1, f2 = th.cos().to(torch.bfloat16), th.sin().to(torch.bfloat16)
        f2[..., 1::2] *= -1
        self.factor1, self.factor2 = f1, f2

    def reset(self, device=None):
        device = device or self.factor1.device
        freq = (1 / 1024) ** torch.linspace(0, 1, steps=self.head_dim // 4, dtype=torch.float32, device=device)
        self.angular_freq = torch.cat([freq.repeat_interleave(2), freq.new_zeros(self.head_dim // 2)])
        self.attn_scale = 0.1
        self._tables()

    def _apply(self, fn, *a, **k):  # keep the plain-tensor frequency vector on the module's device
        out = super()._apply(fn, *a, **k)
        self.angular_freq = fn(self.angular_freq)
        return out

    def rotary(self, x_BTHD):
        T = x_BTHD.size(-3)
        f1, f2 = self.factor1[None, :T, None, :].to(x_BTHD.dtype), self.factor2[None, :T, None, :].to(x_BTHD.dtype)
        flip = x_BTHD.view(*x_BTHD.shape[:-1], x_BTHD.shape[-1] // 2, 2).flip(-1).view(x_BTHD.shape)
        return f1 * x_BTHD + f2 * flip

    def apply(self, old_window: int, new_window: int, alpha: int = 1, beta: int = 32):
        rotations = self.block_size * old_window * self.angular_freq / (2 * torch.pi)
        scale = old_window / new_window
        interp = torch.clamp((rotations - alpha) / (beta - alpha), 0, 1)
        self.angular_freq = self.angular_freq * (scale + interp * (1 - scale))
        self._tables()
        self.attn_scale *= 0.2 * math.log(new_window / old_window) + 1


def doc_bounds(seqlens: torch.Tensor, T: int, factor: int = 1):
    """Per-token ``(doc_start, doc_end)`` (int32) from cumulative sequence lengths; ``factor`` 2 for the paired layout."""
    cu = (seqlens.to(torch.int64) * factor).clamp(max=T)
    pos = torch.arange(T, device=seqlens.device)
    idx = torch.searchsorted(cu, pos, right=True).clamp(1, len(cu) - 1)
    return cu[idx - 1].to(torch.int32), cu[idx].to(torch.int32)


def _attend(q, k, v, seqlens, window_tokens: int, scale: float, factor: int):
    """``q, k, v [T', H', D]`` -> causal, document-local attention where query ``i`` sees keys ``i - window .. i`` (the
    ``window_size=(w, 0)`` rule of the reference's varlen call). The token-exact window is folded into the per-token
    lower / upper bounds the kernel already takes; its block window only has to be wide enough to cover it."""
    Tp = q.shape[0]
    ds, de = doc_bounds(seqlens, Tp, factor)
    pos = torch.arange(Tp, device=q.device, dtype=torch.int32)
    ds = torch.maximum(ds, pos - window_tokens)
    de = torch.minimum(de, pos + window_tokens + 1)
    blocks = -(-window_tokens // BLOCK) + 1
    if q.is_cuda and q.shape[-1] == 128 and q.dtype == torch.bfloat16:
        # the kernel reads rows through a token stride: a [T, H, D] slice of the fused QKV output needs no copy
        rows = lambda t: t if (t.stride(2) == 1 and t.stride(1) == t.shape[2] and t.stride(0) % 8 == 0) else t.contiguous()
        return flash_attention(rows(q), rows(k), rows(v), ds, de, scale, blocks)
    return attention_reference(q, k, v, ds, scale, blocks).to(q.dtype)


class _KeyOffset(torch.autograd.Function):
    """The stationary (second) half of every key row replaced by that of the previous token (token 0 keeps its own):
    ``cat([k[..., :D/2], cat([k[:, :1, :, D/2:], k[:, :-1, :, D/2:]], 1)], -1)`` as one copy + one shifted half-row
    copy, and the same two copies in the backward (the nested ``cat`` costs two unaligned concatenations forward and three
    zero-filled full-size slice gradients plus their sums backward)."""

    @staticmethod
    def forward(ctx, k):
        h = k.shape[-1] // 2
        out = k.clone(memory_format=torch.contiguous_format)
        out[:, 1:, :, h:] = k[:, :-1, :, h:]
        return out

    @staticmethod
    def backward(ctx, g):
        h = g.shape[-1] // 2
        dk = g.clone(memory_format=torch.contiguous_format)
        T = g.shape[1]
        if T > 1:
            dk[:, :-1, :, h:] = g[:, 1:, :, h:]
            dk[:, 0, :, h:] += g[:, 0, :, h:]
            dk[:, -1, :, h:] = 0
        return dk


def key_offset(k: torch.Tensor) -> torch.Tensor:
    """``k [B, T, H, D]``: shift the second half of the head dimension one token forward."""
    return _KeyOffset.apply(k)


@dataclass
class AttnArgs:
    ve: torch.Tensor | None
    sa_lambdas: torch.Tensor
    seqlens: torch.Tensor
    bm_size: int
    yarn: Yarn
    key_offset: bool
    attn_gate_w: torch.Tensor
    ve_gate_w: torch.Tensor | None


class CausalSelfAttention(nn.Module):
    def __init__(self, dim: int, head_dim: int, num_heads: int, paired: bool = False):
        super().__init__()
        self.num_heads, self.head_dim, self.dim, self.paired = num_heads, head_dim, dim, paired
        assert num_heads * head_dim == dim, "num_heads * head_dim must equal model_dim"

    def forward(self, x, a: AttnArgs, qkvo_w, residual=None, gate_in=None):
        """``residual``: added to the output inside the output projection's GEMM (the block's skip connection).
        ``gate_in``: ``x[..., :12]`` when the caller already has it as a tensor of its own."""
        B, T = x.shape[:2]
        assert B == 1, "packed variable-length sequences need B == 1"
        H, D = self.num_heads, self.head_dim
        q, k, v = linear(x, a.sa_lambdas[0] * qkvo_w[:self.dim * 3].type_as(x)).view(B, T, 3, H, D).unbind(2)   # unbind: one stack in the backward
        gate_in = x[..., :12] if gate_in is None else gate_in
        f1, f2 = a.yarn.factor1, a.yarn.factor2          # QK norm and the rotary map are one kernel on CUDA
        # value-embedding mix v + 2 sigmoid(gate) * ve: one kernel in the [T, H, D] layout (reinterpreting the result as
        # [2T, H/2, D] afterwards is the same flat order the reference mixes in)
        if a.ve is not None:
            v = rowscale_add(v, 2 * torch.sigmoid(F.linear(gate_in, a.ve_gate_w)).view(B, T, H), a.ve.view(B, T, H, D))
        if self.paired:
            # [T, H, D] reinterpreted as [2T, H/2, D] exactly as the reference does (a flat view: head h of token t lands at
            # position 2t + h // (H/2) of head h % (H/2)); rotary angles come from the paired table (positions 2t, 2t+1)
            q = norm_rotary(q, f1, f2).view(B, 2 * T, H // 2, D)
            k = norm_rotary(k, f1, f2).view(B, 2 * T, H // 2, D)
            v = v.reshape(B, 2 * T, H // 2, D)
            y = _attend(q[0], k[0], v[0], a.seqlens, a.bm_size, a.yarn.attn_scale, 2)
        else:
            q, k = norm_rotary(q, f1, f2), norm_rotary(k, f1, f2)
            if a.key_offset:  # shift the stationary half of the key one token forward: one-layer induction
                k = key_offset(k)
            y = _attend(q[0], k[0], v[0], a.seqlens, a.bm_size, a.yarn.attn_scale, 1)
        y = rowscale_add(None, torch.sigmoid(F.linear(gate_in, a.attn_gate_w)).view(B, T, H), y.reshape(B, T, H, D))
        return linear(y.reshape(B, T, H * D), a.sa_lambdas[1] * qkvo_w[self.dim * 3:].type_as(y), residual=residual)


class PairedHeadCausalSelfAttention(CausalSelfAttention):
    def __init__(self, dim: int, head_dim: int, num_heads: int):
        super().__init__(dim, head_dim, num_heads, paired=True)


class MLP(nn.Module):
    def forward(self, x, c_fc, c_proj, residual=None):
        """``relu(x @ c_fc.T)^2 @ c_proj (+ residual)`` with both weights stored ``[4 d, d]``."""
        return mlp_relu2(x, c_fc.type_as(x), c_proj.type_as(x), residual)


class Block(nn.Module):
    def __init__(self, dim: int, head_dim: int, num_heads: int, has_attn: bool, has_mlp: bool, use_paired_head: bool):
        super().__init__()
        self.attn = (PairedHeadCausalSelfAttention if use_paired_head else CausalSelfAttention)(dim, head_dim, num_heads) if has_attn else None
        self.mlp = MLP() if has_mlp else None

    def forward(self, x, attn_args, qkvo_w=None, c_fc=None, c_proj=None):
        if self.attn is not None:      # the skip connections are added in the epilogue of each branch's last GEMM
            h, skip, gate_in = norm_skip(x, 12)
            x = self.attn(h, attn_args, qkvo_w, residual=skip, gate_in=gate_in)
        if self.mlp is not None:
            h, skip = norm_skip(x)
            x = self.mlp(h, c_fc, c_proj, residual=skip)
        return x


class GPT(nn.Module):
    def __init__(self, vocab_size: int = 50257, num_layers: int = 11, num_heads: int = 6, head_dim: int = 128, model_dim: int = 768,
                 max_seq_len: int = 2048 * 16, bigram_vocab_size: int = 50304 * 5, world_size: int = 1, use_fp8: bool = True,
                 block_size: int = BLOCK):
        super().__init__()
        self.num_layers, self.block_size = num_layers, block_size
        vocab_size = next_multiple_of_n(vocab_size, n=128)

        def labelled(p, label, reshape=None):
            p.label = label
            if reshape is not None:
                p.reshape = reshape
            return p

        self.smear_gate = nn.Linear(12, 1, bias=False)
        self.skip_gate = nn.Linear(12, 1, bias=False)
        for gate, label in ((self.smear_gate, "smear_gate"), (self.skip_gate, "skip_gate")):
            nn.init.zeros_(gate.weight)
            labelled(gate.weight, label)
        self.value_embeds = nn.ModuleList([nn.Embedding(vocab_size, model_dim) for _ in range(5)])
        for i, ve in enumerate(self.value_embeds):
            nn.init.zeros_(ve.weight)
            labelled(ve.weight, f"ve{i}")
        n_attn = num_layers - 1  # the layer at index 6 has no attention
        self.attn_gate_bank = labelled(nn.Parameter(torch.zeros(n_attn, num_heads, 12)), "attn_gate_bank")
        self.ve_gate_bank = labelled(nn.Parameter(torch.zeros(5, num_heads, 12)), "ve_gate_bank")
        self.attn_layer_indices = [i for i in range(num_layers) if i != 6]
        self.mlp_layer_indices = list(range(num_layers))
        self.layer_to_attn_idx = {l: b for b, l in enumerate(self.attn_layer_indices)}
        self.layer_to_mlp_idx = {l: b for b, l in enumerate(self.mlp_layer_indices)}
        hdim, mlp_hdim = num_heads * head_dim, 4 * model_dim
        # banks: every matrix of one kind in one parameter, so that the sharded optimizer sees (40, d, d) and (24, 4d, d)
        self.attn_bank = labelled(nn.Parameter(torch.empty(n_attn, 4 * model_dim, hdim)), "attn", (n_attn * 4, hdim, hdim))
        n_mlp = len(self.mlp_layer_indices) + 1  # one padding slot: 24 matrices divide over 8 ranks
        self.mlp_bank = labelled(nn.Parameter(torch.empty(n_mlp, 2, mlp_hdim, model_dim)), "mlp", (n_mlp * 2, mlp_hdim, model_dim))
        attn_bound = (3 ** 0.5) * model_dim ** -0.5
        mlp_bound = (3 ** 0.5) * 0.5 * model_dim ** -0.5
        with torch.no_grad():
            self.attn_bank[:, :model_dim * 3].uniform_(-attn_bound, attn_bound)
            self.attn_bank[:, model_dim * 3:].zero_()
            self.mlp_bank[:, 0].uniform_(-mlp_bound, mlp_bound)
            self.mlp_bank[:, 1].zero_()
        self.paired_head_layers = [0, 2, 5, 9]
        self.blocks = nn.ModuleList([Block(model_dim, head_dim, num_heads, has_attn=i in self.layer_to_attn_idx,
                                           has_mlp=i in self.layer_to_mlp_idx, use_paired_head=i in self.paired_head_layers)
                                     for i in range(num_layers)])
        self.yarn = Yarn(head_dim, max_seq_len, block_size=block_size)
        self.yarn_paired_head = Yarn(head_dim, max_seq_len, paired=True, block_size=block_size)
        self.lm_head = CastedLinearT(model_dim, vocab_size, use_fp8=use_fp8, x_s=100 / 448, w_s=1.6 / 448, grad_s=0.75 / 448)
        nn.init.normal_(self.lm_head.weight, mean=0, std=0.005)
        labelled(self.lm_head.weight, "lm_head")
        self.embed = nn.Embedding(vocab_size, model_dim)
        labelled(self.embed.weight, "embed")
        with torch.no_grad():
            self.embed.weight.copy_(self.lm_head.weight.T)
        self.bigram_embed = nn.Embedding(bigram_vocab_size, model_dim)
        nn.init.zeros_(self.bigram_embed.weight)
        labelled(self.bigram_embed.weight, "bigram_embed")
        self.x0_lambdas = labelled(nn.Parameter(torch.zeros(num_layers)), "x0_lambdas")
        pad = (-num_layers * 3 - 3) % world_size  # the reference's padding rule, kept for identical parameter shapes
        self.scalars = labelled(nn.Parameter(torch.cat([
            1.1 * torch.ones(num_layers),                                    # residual lambdas
            *[torch.tensor([0.5, 1.0]) for _ in range(num_layers)],          # attention in / out lambdas
            0.1 * torch.ones(num_layers),                                    # bigram lambdas
            torch.zeros(1), 0.5 * torch.ones(1), -1.5 * torch.ones(1),       # smear, back-out, skip
            torch.ones(pad)])), "scalars")

    def forward(self, input_seq, target_seq, seqlens, bigram_input_seq, schedule_cfg: ForwardScheduleConfig):
        assert input_seq.ndim == 1
        L = self.num_layers
        resid = self.scalars[:L]
        sa = self.scalars[L:3 * L].view(-1, 2)
        bigram_l = self.scalars[3 * L:4 * L]
        smear_l, backout_l, skip_l = self.scalars[4 * L], self.scalars[4 * L + 1], self.scalars[4 * L + 2]
        short_bm, long_bm = schedule_cfg.ws_short * self.block_size, schedule_cfg.ws_long * self.block_size
        bm = [short_bm] * L
        for i in (3, L - 1):
            bm[i] = long_bm
        bm[6] = None
        key_offset = [b == long_bm for b in bm]
        x = embedding(input_seq, self.embed.weight)
        x0_bigram = embedding(bigram_input_seq, self.bigram_embed.weight)[None]
        ve = [embedding(input_seq, e.weight) for e in self.value_embeds]
        ve = [ve[0], ve[1]] + [None] * (L - 5) + [ve[2], ve[3], ve[4]]
        smear = smear_l * torch.sigmoid(self.smear_gate(x[1:, :12]))
        x = torch.cat([x[:1], x[1:] + smear * x[:-1]])
        x = x0 = norm(x[None])
        ag = [w.to(x.dtype) for w in self.attn_gate_bank.unbind(0)]
        veg = [w.to(x.dtype) for w in self.ve_gate_bank.unbind(0)]
        attn_gates = ag[:6] + [None] + ag[6:]
        ve_gates = [veg[0], veg[1]] + [None] * (L - 5) + [veg[2], veg[3], veg[4]]
        attn_w = self.attn_bank.unbind(0)
        fcs, projs = self.mlp_bank[:, 0].unbind(0), self.mlp_bank[:, 1].unbind(0)
        skips, x_backout = [], None
        for i in range(L):
            args = AttnArgs(ve[i], sa[i], seqlens, bm[i], self.yarn_paired_head if i in self.paired_head_layers else self.yarn,
                            key_offset[i], attn_gates[i], ve_gates[i])
            if i == 6:
                x = x + torch.sigmoid(skip_l) * 2 * torch.sigmoid(self.skip_gate(x0[..., :12])) * skips.pop()
            if i == 0:   # x is x0 here: its two coefficients add up
                x = lincomb3(x, x0_bigram, None, torch.stack([resid[0] + self.x0_lambdas[0], bigram_l[0]]))
            else:
                x = lincomb3(x, x0, x0_bigram, torch.stack([resid[i], self.x0_lambdas[i], bigram_l[i]]))
            x = self.blocks[i](x, args, attn_w[self.layer_to_attn_idx[i]] if i in self.layer_to_attn_idx else None,
                               fcs[self.layer_to_mlp_idx[i]], projs[self.layer_to_mlp_idx[i]])
            if i == 3:
                skips.append(x)
            if i == 7:
                x_backout = x
        x = norm(x - backout_l * x_backout)
        head = self.lm_head
        if self.training and head.use_fp8 and x.is_cuda:      # projection + loss as one node (no [T, V] gradient passes)
            return head_ce_loss(x.flatten(0, -2), head.weight, target_seq, schedule_cfg.mtp_weights, head.x_s, head.w_s, head.grad_s)
        logits = head(x)
        if self.training:
            return softcapped_cross_entropy(logits.view(-1, logits.size(-1)), target_seq, schedule_cfg.mtp_weights).sum()
        z = 23 * torch.sigmoid((logits.float() + 5) / 7.5)
        return F.cross_entropy(z.view(-1, z.size(-1)), target_seq, reduction="mean")
