"""GPT-2 style decoder of the modded-nanogpt "classic" speedrun trainer, generic in
``(num_layers, num_heads, head_dim, model_dim)``.

Module tree, parameter names / shapes / dtypes and the forward signature follow the reference
(modded-nanogpt/records/track_1_short/2025-01-26_BatchSize/c44090cc-...txt, classes ``CastedLinear``, ``Rotary``,
``CausalSelfAttention``, ``MLP``, ``Block``, ``ValueEmbedding``, ``GPT``), so its ``state_dict`` loads here and vice versa:
merged ``qkv_w (3, H*D, dim)``, zero-initialised ``c_proj`` and ``lm_head``, value embeddings in the 012...012 pattern,
U-net skips with ``skip_weights``, per-block ``lambdas``, half-truncated RoPE, QK RMSNorm, attention scale 0.12,
document-causal attention with long/short block windows, logits ``30 * sigmoid(z / 7.5)``, fp8 ``lm_head``
(``x_s=2, w_s=2**9, grad_s=2**19``).

Two execution paths share the parameters:

* ``forward`` on CPU tensors (or with ``fused=False``): plain PyTorch autograd, the numerical oracle;
* ``forward`` on CUDA tensors: one autograd node (:class:`_FusedGPTLoss`) that runs the whole forward and backward with
  the sm_100a kernels of :mod:`ml_experiments_b200.ops` (tcgen05 GEMMs with fused epilogues, flash attention, fused
  norm / RoPE / mixing kernels, fp8 head + soft-capped cross entropy).
"""
from __future__ import annotations

from dataclasses import dataclass, asdict

import torch
import torch.nn.functional as F
from torch import Tensor, nn

from ..ops import fused as Fz
from ..ops.attention import attention_mask, doc_bounds_from_starts, doc_bounds_from_tokens  # noqa: F401

BOS_ID = 50256


def next_multiple_of_n(v: float | int, *, n: int) -> int:
    return next(x for x in range(n, int(v) + 1 + n, n) if x >= v)


def norm(x: Tensor) -> Tensor:
    return F.rms_norm(x, (x.size(-1),))


@dataclass
class GPTConfig:
    vocab_size: int = 50257
    num_layers: int = 12
    num_heads: int = 6
    model_dim: int = 768
    head_dim: int = 128
    max_seq_len: int = 65536
    num_value_embeds: int = 3
    skip_attn_layers: tuple = (7,)
    attn_scale: float = 0.12
    softcap: float = 30.0
    softcap_div: float = 7.5
    use_fp8_head: bool = True
    x_s: float = 2.0
    w_s: float = 2.0 ** 9
    grad_s: float = 2.0 ** 19
    uniform_doc_len: int | None = None   # set when every document has this length (documents then start every N tokens)

    def to_dict(self):
        return asdict(self)

    @classmethod
    def gpt2_small(cls, **kw):
        return cls(**kw)

    @classmethod
    def gpt2_medium(cls, **kw):
        base = dict(num_layers=24, num_heads=16, model_dim=1024, head_dim=64, skip_attn_layers=())
        base.update(kw)
        return cls(**base)

    @classmethod
    def medium_track(cls, **kw):
        """Shape of the reference's medium-track trainer (modded-nanogpt/train_gpt_medium.py:1688-1695)."""
        base = dict(num_layers=16, num_heads=8, model_dim=1024, head_dim=128, skip_attn_layers=())
        base.update(kw)
        return cls(**base)


class CastedLinear(nn.Linear):
    def __init__(self, in_features: int, out_features: int, use_fp8: bool = False, x_s: float = 1.0, w_s: float = 1.0,
                 grad_s: float = 1.0):
        super().__init__(in_features, out_features, bias=False)
        self.use_fp8, self.x_s, self.w_s, self.grad_s = use_fp8, x_s, w_s, grad_s

    def reset_parameters(self) -> None:
        std = 0.5 * (self.in_features ** -0.5)
        bound = (3 ** 0.5) * std
        with torch.no_grad():
            self.weight.uniform_(-bound, bound)

    def forward(self, x: Tensor) -> Tensor:
        return F.linear(x, self.weight.type_as(x))


class Rotary(nn.Module):
    def __init__(self, dim: int, max_seq_len: int):
        super().__init__()
        cos, sin = Fz.rotary_tables(dim, max_seq_len)
        self.cos = nn.Buffer(cos, persistent=False)
        self.sin = nn.Buffer(sin, persistent=False)

    def forward(self, x_BTHD: Tensor) -> Tensor:
        t = x_BTHD.size(-3)
        cos, sin = self.cos[None, :t, None, :], self.sin[None, :t, None, :]
        x1, x2 = x_BTHD.to(dtype=torch.float32).chunk(2, dim=-1)
        return torch.cat((x1 * cos + x2 * sin, x1 * (-sin) + x2 * cos), 3).type_as(x_BTHD)


class CausalSelfAttention(nn.Module):
    def __init__(self, dim: int, num_heads: int, max_seq_len: int, head_dim: int = 128, attn_scale: float = 0.12):
        super().__init__()
        self.num_heads, self.head_dim = num_heads, head_dim
        hdim = num_heads * head_dim
        bound = (3 ** 0.5) * 0.5 * (dim ** -0.5)
        self.qkv_w = nn.Parameter(torch.empty(3, hdim, dim).uniform_(-bound, bound))
        self.lambdas = nn.Parameter(torch.tensor([0.5, 0.5]))
        self.rotary = Rotary(head_dim, max_seq_len)
        self.c_proj = CastedLinear(hdim, dim)
        self.c_proj.weight.detach().zero_()
        self.attn_scale = attn_scale

    def forward(self, x: Tensor, ve: Tensor | None, mask: Tensor) -> Tensor:
        B, T = x.size(0), x.size(1)
        q, k, v = F.linear(x, self.qkv_w.flatten(end_dim=1).type_as(x)).view(B, T, 3 * self.num_heads, self.head_dim).chunk(3, dim=-2)
        q, k = norm(q), norm(k)
        q, k = self.rotary(q), self.rotary(k)
        if ve is not None:
            v = self.lambdas[0] * v + self.lambdas[1] * ve.view_as(v)
        else:
            v = self.lambdas[0] * v
        y = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2).type_as(q),
                                           attn_mask=mask, scale=self.attn_scale).transpose(1, 2)
        y = y.contiguous().view(B, T, self.num_heads * self.head_dim)
        return self.c_proj(y)


class MLP(nn.Module):
    def __init__(self, dim: int):
        super().__init__()
        self.c_fc = CastedLinear(dim, 4 * dim)
        self.c_proj = CastedLinear(4 * dim, dim)
        self.c_proj.weight.detach().zero_()

    def forward(self, x: Tensor) -> Tensor:
        return self.c_proj(F.relu(self.c_fc(x)).square())


class Block(nn.Module):
    def __init__(self, dim: int, num_heads: int, layer_idx: int, max_seq_len: int, head_dim: int = 128,
                 has_attn: bool = True, attn_scale: float = 0.12):
        super().__init__()
        self.attn = CausalSelfAttention(dim, num_heads, max_seq_len, head_dim, attn_scale) if has_attn else None
        self.mlp = MLP(dim)
        self.lambdas = nn.Parameter(torch.tensor([1., 0.]))

    def forward(self, x: Tensor, ve: Tensor | None, x0: Tensor, mask: Tensor) -> Tensor:
        x = self.lambdas[0] * x + self.lambdas[1] * x0
        if self.attn is not None:
            x = x + self.attn(norm(x), ve, mask)
        x = x + self.mlp(norm(x))
        return x


class ValueEmbedding(nn.Module):
    def __init__(self, vocab_size: int, embedding_dim: int, num_layers: int, num_embeddings: int = 3):
        super().__init__()
        self.num_layers, self.num_embeddings = num_layers, num_embeddings
        self.embed = nn.ModuleList([nn.Embedding(vocab_size, embedding_dim) for _ in range(num_embeddings)])

    def layer_map(self) -> list[int | None]:
        n = self.num_embeddings
        return list(range(n)) + [None] * (self.num_layers - 2 * n) + list(range(n))

    def forward(self, input_seq: Tensor) -> list[Tensor | None]:
        ve = [emb(input_seq) for emb in self.embed]
        return [None if j is None else ve[j] for j in self.layer_map()]


def window_pattern(num_layers: int) -> list[bool]:
    """``True`` where a layer uses the long window. Encoder half ``[L,S,S,S,L,S]`` (cyclic for other depths),
    decoder half mirrored, as in the reference ``GPT.forward``."""
    enc = num_layers // 2
    base = [True, False, False, False, True, False]
    enc_pat = [base[i % 6] for i in range(enc)]
    dec_pat = list(reversed(enc_pat))
    dec = num_layers - enc
    dec_pat = (dec_pat + [False] * dec)[:dec]
    return enc_pat + dec_pat


class GPT(nn.Module):
    def __init__(self, vocab_size: int = 50257, num_layers: int = 12, num_heads: int = 6, model_dim: int = 768,
                 max_seq_len: int = 65536, head_dim: int = 128, config: GPTConfig | None = None):
        super().__init__()
        if config is None:
            config = GPTConfig(vocab_size=vocab_size, num_layers=num_layers, num_heads=num_heads, model_dim=model_dim,
                               head_dim=head_dim, max_seq_len=max_seq_len,
                               skip_attn_layers=(7,) if num_layers == 12 else ())
        self.config = c = config
        self.embed = nn.Embedding(c.vocab_size, c.model_dim)
        self.value_embeds = ValueEmbedding(c.vocab_size, c.num_heads * c.head_dim, c.num_layers, c.num_value_embeds)
        self.blocks = nn.ModuleList([
            Block(c.model_dim, c.num_heads, i, c.max_seq_len, c.head_dim, has_attn=i not in c.skip_attn_layers,
                  attn_scale=c.attn_scale) for i in range(c.num_layers)])
        self.num_encoder_layers = c.num_layers // 2
        self.num_decoder_layers = c.num_layers - self.num_encoder_layers
        self.skip_weights = nn.Parameter(torch.ones(self.num_decoder_layers))
        self.lm_head = CastedLinear(c.model_dim, next_multiple_of_n(c.vocab_size, n=128), use_fp8=c.use_fp8_head,
                                    x_s=c.x_s, w_s=c.w_s, grad_s=c.grad_s)
        self.lm_head.weight.detach().zero_()
        self.fused = True
        self._shadow = None  # low-precision parameter copies for the fused path

    # -------------------------------------------------------------------------------------------- helpers
    def cast_embeddings_bf16(self) -> "GPT":
        """Embedding tables are kept in bf16 by the reference trainer (``m.bfloat16()`` on every ``nn.Embedding``)."""
        for m in self.modules():
            if isinstance(m, nn.Embedding):
                m.bfloat16()
        return self

    def document_bounds(self, input_seq: Tensor):
        return doc_bounds_from_tokens(input_seq, BOS_ID)

    def layer_windows(self, sliding_window_num_blocks: int) -> list[int]:
        long_w = int(sliding_window_num_blocks)
        short_w = max(long_w // 2, 1)
        return [long_w if is_long else short_w for is_long in window_pattern(self.config.num_layers)]

    # -------------------------------------------------------------------------------------------- forward
    def forward(self, input_seq: Tensor, target_seq: Tensor, sliding_window_num_blocks) -> Tensor:
        assert input_seq.ndim == 1
        swb = int(sliding_window_num_blocks)
        if input_seq.is_cuda and self.fused:
            from .gpt_fused import fused_gpt_loss
            return fused_gpt_loss(self, input_seq, target_seq, swb)
        return self.forward_reference(input_seq, target_seq, swb)

    def loss_and_grad(self, input_seq: Tensor, target_seq: Tensor, sliding_window_num_blocks) -> Tensor:
        """``loss = self(...); loss.backward()`` in one call; returns the detached loss. The fused CUDA path fills
        ``p.grad`` directly."""
        swb = int(sliding_window_num_blocks)
        if input_seq.is_cuda and self.fused and torch.is_grad_enabled():
            from .gpt_fused import fused_gpt_step
            return fused_gpt_step(self, input_seq, target_seq, swb)
        loss = self(input_seq, target_seq, swb)
        loss.backward()
        return loss.detach()

    def forward_reference(self, input_seq: Tensor, target_seq: Tensor, sliding_window_num_blocks: int) -> Tensor:
        """Plain PyTorch path (dense masks; meant for CPU tests and small sequences)."""
        c = self.config
        doc_start, _ = self.document_bounds(input_seq)
        windows = self.layer_windows(sliding_window_num_blocks)
        masks = {w: attention_mask(doc_start, w) for w in set(windows)}
        x = x0 = norm(self.embed(input_seq)[None])
        ve = self.value_embeds(input_seq)
        skips = []
        for i in range(self.num_encoder_layers):
            x = self.blocks[i](x, ve[i], x0, masks[windows[i]])
            skips.append(x)
        for i in range(self.num_decoder_layers):
            x = x + self.skip_weights[i] * skips.pop()
            li = self.num_encoder_layers + i
            x = self.blocks[li](x, ve[li], x0, masks[windows[li]])
        x = norm(x)
        logits = self.lm_head(x)
        logits = c.softcap * torch.sigmoid(logits.float() / c.softcap_div)
        return F.cross_entropy(logits.view(-1, logits.size(-1)), target_seq)

    # -------------------------------------------------------------------------------------------- param groups
    def param_groups(self):
        """``(hidden_matrix, embed, scalar, head)`` parameter lists exactly as the reference trainer splits them."""
        hidden = [p for n, p in self.blocks.named_parameters() if p.ndim >= 2 and "embed" not in n]
        embed = [p for n, p in self.named_parameters() if "embed" in n]
        scalar = [p for p in self.parameters() if p.ndim < 2]
        head = [self.lm_head.weight]
        return hidden, embed, scalar, head
