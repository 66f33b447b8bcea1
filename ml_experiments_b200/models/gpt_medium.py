"""The medium-track speedrun GPT: 16 layers, d = 1024, 8 heads x 128 (modded-nanogpt/train_gpt_medium.py:925-1218).

Per-block parameters instead of banks: ``qkvo_w [4 d, d]`` (Q, K, V rows then the output projection, zero-initialised),
``c_fc`` / ``c_proj [4 d, d]``; sparse attention gate and value-embedding gate on the first 16 channels; partial key
offset on the long-window layers (the stationary quarter-bands of the key are shifted one token forward); five value
embeddings on the first and last five layers; a second token embedding ``embed2`` mixed into every layer through
``x0_lambdas[:, 1]``; three gated U-net skips (2 -> 11, 4 -> 10, 6 -> 9); back-out of layer 11; lm_head tied to the
embedding until ``split_embed``; multi-token soft-capped loss in training, four-chunk mean loss in eval.
Attention, linear layers and the loss run on this package's kernels exactly as in :mod:`.gpt_head`.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops.fused import softcapped_cross_entropy
from ..ops.linear import linear, linear_t, mlp_relu2
from ..ops.norm_rope import norm_rotary
from ..ops.rowops import lincomb3, rowscale_add
from .gpt import CastedLinear
from .gpt_head import BLOCK, ForwardScheduleConfig, Yarn, _attend, next_multiple_of_n, norm, norm_skip

VE_LAYERS = (0, 1, 2, 3, 4, 11, 12, 13, 14, 15)
LONG_LAYERS = (0, 4, 11, 15)
SKIP_IN, SKIP_OUT, BACKOUT_LAYER = (2, 4, 6), (9, 10, 11), 11


def _label(p, label, lr_mul=None, wd_mul=None):
    p.label = label
    if lr_mul is not None:
        p.lr_mul = lr_mul
    if wd_mul is not None:
        p.wd_mul = wd_mul
    return p


class CausalSelfAttention(nn.Module):
    def __init__(self, dim: int, head_dim: int, num_heads: int, layer_idx: int):
        super().__init__()
        assert num_heads * head_dim == dim, "num_heads * head_dim must equal model_dim"
        self.num_heads, self.head_dim, self.dim = num_heads, head_dim, dim
        bound = (3 ** 0.5) * dim ** -0.5
        self.qkvo_w = _label(nn.Parameter(torch.empty(dim * 4, dim)), "attn")
        with torch.no_grad():
            self.qkvo_w[: dim * 3].uniform_(-bound, bound)
            self.qkvo_w[dim * 3:].zero_()
        self.attn_gate = CastedLinear(16, num_heads)
        _label(self.attn_gate.weight, "attn_gate", lr_mul=0.1)
        if layer_idx in VE_LAYERS:
            self.value_embed_gate = CastedLinear(16, num_heads)
            _label(self.value_embed_gate.weight, "value_embed_gate", lr_mul=0.1)

    def forward(self, x, ve, sa_lambdas, seqlens, bm_size: int, yarn: Yarn, key_offset: bool, residual=None, gate_in=None):
        """``residual`` (the block's skip connection) is added in the output projection's GEMM epilogue; ``gate_in`` is
        ``x[..., :16]`` when the caller already holds it as a tensor of its own."""
        B, T = x.shape[:2]
        assert B == 1, "packed variable-length sequences need B == 1"
        H, D = self.num_heads, self.head_dim
        q, k, v = linear(x, sa_lambdas[0] * self.qkvo_w[: self.dim * 3].type_as(x)).view(B, T, 3, H, D).unbind(2)
        q, k = norm_rotary(q, yarn.factor1, yarn.factor2), norm_rotary(k, yarn.factor1, yarn.factor2)
        if key_offset:  # the two stationary quarter-bands of the key move one token forward
            prev = torch.cat([k[:, :1], k[:, :-1]], dim=1)
            band = torch.zeros(D, dtype=torch.bool, device=k.device)
            band[D // 4: D // 2] = True
            band[3 * D // 4:] = True
            k = torch.where(band, prev, k)
        gate_in = x[..., :16] if gate_in is None else gate_in
        if ve is not None:
            v = rowscale_add(v, 2 * torch.sigmoid(self.value_embed_gate(gate_in)).view(B, T, H), ve.view(B, T, H, D))
        y = _attend(q[0], k[0], v[0], seqlens, bm_size, yarn.attn_scale, 1)
        y = rowscale_add(None, torch.sigmoid(self.attn_gate(gate_in)).view(B, T, H), y.reshape(B, T, H, D))
        return linear(y.reshape(B, T, H * D), sa_lambdas[1] * self.qkvo_w[self.dim * 3:].type_as(y), residual=residual)


class MLP(nn.Module):
    def __init__(self, dim: int):
        super().__init__()
        bound = (3 ** 0.5) * 0.5 * dim ** -0.5
        self.c_fc = _label(nn.Parameter(torch.empty(4 * dim, dim).uniform_(-bound, bound)), "mlp")
        self.c_proj = _label(nn.Parameter(torch.zeros(4 * dim, dim)), "mlp", lr_mul=2.0)

    def forward(self, x, residual=None):
        return mlp_relu2(x, self.c_fc.type_as(x), self.c_proj.type_as(x), residual)


class Block(nn.Module):
    def __init__(self, dim: int, head_dim: int, num_heads: int, layer_idx: int):
        super().__init__()
        self.attn, self.mlp = CausalSelfAttention(dim, head_dim, num_heads, layer_idx), MLP(dim)

    def forward(self, x, **attn_args):
        h, skip, gate_in = norm_skip(x, 16)       # skip and gate-input gradients join the norm's backward kernel
        x = self.attn(h, residual=skip, gate_in=gate_in, **attn_args)
        h, skip = norm_skip(x)
        return self.mlp(h, residual=skip)


class GPTMedium(nn.Module):
    def __init__(self, vocab_size: int = 50257, num_layers: int = 16, num_heads: int = 8, head_dim: int = 128, model_dim: int = 1024,
                 max_seq_len: int = 65536, world_size: int = 1, block_size: int = BLOCK):
        super().__init__()
        assert num_layers == 16, "the skip / value-embedding / window layout is defined for 16 layers"
        self.num_layers, self.block_size = num_layers, block_size
        vocab_size = next_multiple_of_n(vocab_size, n=128)
        self.smear_gate = CastedLinear(16, 1)
        _label(self.smear_gate.weight, "smear_gate", 0.01, 0.0)
        self.skip_gates = nn.ModuleList([CastedLinear(16, 1) for _ in range(3)])
        for sg in self.skip_gates:
            _label(sg.weight, "skip_gate", 0.01, 0.0)
        self.value_embeds = nn.ModuleList([nn.Embedding(vocab_size, model_dim) for _ in range(5)])
        for e in self.value_embeds:
            nn.init.zeros_(e.weight)
            _label(e.weight, "value_embed", 75.0, 5.0)
        self.blocks = nn.ModuleList([Block(model_dim, head_dim, num_heads, i) for i in range(num_layers)])
        self.yarn = Yarn(head_dim, max_seq_len)
        self.lm_head = CastedLinear(model_dim, vocab_size)
        nn.init.normal_(self.lm_head.weight, mean=0, std=0.005)
        _label(self.lm_head.weight, "lm_head", wd_mul=150.0)
        self.embed, self.embed2 = nn.Embedding(vocab_size, model_dim), nn.Embedding(vocab_size, model_dim)
        _label(self.embed.weight, "embed", wd_mul=150.0)
        _label(self.embed2.weight, "embed2", 75.0, 5.0)
        self.x0_lambdas = _label(nn.Parameter(torch.zeros(2 * num_layers)), "x0_lambdas", 5.0, 0.0)
        pad = (-num_layers * 3 - 5) % world_size
        self.scalars = _label(nn.Parameter(torch.cat([1.05 * torch.ones(num_layers), *[torch.tensor([0.5, 1.0]) for _ in range(num_layers)],
                                                      torch.zeros(1), 0.5 * torch.ones(1), -1.5 * torch.ones(3), torch.ones(pad)])),
                              "scalars", 5.0, 0.0)
        self.split_embed = False   # training starts with the embedding tied to lm_head

    def forward(self, input_seq, target_seq, seqlens, schedule_cfg: ForwardScheduleConfig):
        assert input_seq.ndim == 1
        L = self.num_layers
        resid, x0l, sa = self.scalars[:L], self.x0_lambdas.view(-1, 2), self.scalars[L:3 * L].view(-1, 2)
        smear_l, backout_l, skip_l = self.scalars[3 * L], self.scalars[3 * L + 1], self.scalars[3 * L + 2:3 * L + 5]
        short_bm, long_bm = schedule_cfg.ws_short * self.block_size, schedule_cfg.ws_long * self.block_size
        x = self.embed(input_seq) if self.split_embed else F.embedding(input_seq, self.lm_head.weight)
        ve = [e(input_seq) for e in self.value_embeds]
        ve = ve + [None] * (L - 10) + ve
        x = torch.cat([x[:1], x[1:] + smear_l * torch.sigmoid(self.smear_gate(x[1:, :16])) * x[:-1]])
        x = x0 = norm(x[None])
        x02 = norm(self.embed2(input_seq)[None])
        skips, x_backout, skip_idx = [], None, 0
        for i in range(L):
            if i in SKIP_OUT:
                gate = torch.sigmoid(skip_l[skip_idx]) * 2 * torch.sigmoid(self.skip_gates[skip_idx](x0[..., :16]))
                skip_idx += 1
                x = x + gate * skips.pop()
            if i == 0:   # x is x0 here: its two coefficients add up
                x = lincomb3(x, x02, None, torch.stack([resid[0] + x0l[0, 0], x0l[0, 1]]))
            else:
                x = lincomb3(x, x0, x02, torch.stack([resid[i], x0l[i, 0], x0l[i, 1]]))
            x = self.blocks[i](x, ve=ve[i], sa_lambdas=sa[i], seqlens=seqlens, bm_size=long_bm if i in LONG_LAYERS else short_bm,
                               yarn=self.yarn, key_offset=i in LONG_LAYERS)
            if i in SKIP_IN:
                skips.append(x)
            if i == BACKOUT_LAYER:
                x_backout = x
        x = norm(x - backout_l * x_backout)
        if not self.training:
            loss = 0
            for xc, tc in zip(x.flatten(end_dim=1).chunk(4), target_seq.chunk(4)):
                z = 23 * torch.sigmoid((F.linear(xc, self.lm_head.weight.to(xc.dtype)).float() + 5) / 7.5)
                loss = loss + F.cross_entropy(z, tc, reduction="mean") / 4
            return loss
        logits = self.lm_head(x)
        return softcapped_cross_entropy(logits.view(-1, logits.size(-1)), target_seq, schedule_cfg.mtp_weights).sum()
