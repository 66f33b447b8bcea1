"""``UnifiedLayer`` / ``UnifiedModel`` / ``Model`` and their configuration dataclasses.

Structure follows src/heuristic_secrets/models/composed.py:39-151 (configs with dict round-trip), :154-170,319-379
(poolers, heuristic embedding, gated MLP, feature integration), :574-837 (layer), :840-912 (model, wrapper). One
deliberate difference: with ``head_type="mask"`` the reference applies ``MaskHead`` to the pooled vector and so returns
one logit per sample, which its own trainer's mask loss (``[B, L]`` logits) cannot consume; here the mask head is
applied per position.
"""
from __future__ import annotations

from dataclasses import dataclass, fields
from typing import Literal

import torch
import torch.nn as nn
import torch.nn.functional as F

from .attention import AttentionBlock, ContextualAttentionBlock
from .deform import AdaptiveConvBiases, BiasProjection
from .layers import ByteEmbedding, ClassifierHead, LearnedPooler, MaskHead, RMSNorm, query_pool
from .ssm import MultiKernelSSMBlock, SSMBlock3

_TUPLE_FIELDS = ("conv_kernel_sizes", "ssm_kernel_sizes", "adaptive_init_sigmas")


class _DictConfig:
    def to_dict(self) -> dict:
        d = dict(self.__dict__)
        for k in _TUPLE_FIELDS:
            if d.get(k) is not None:
                d[k] = list(d[k])
        return d

    @classmethod
    def from_dict(cls, d: dict):
        known = {f.name for f in fields(cls)}
        kw = {k: v for k, v in d.items() if k in known}
        for k in _TUPLE_FIELDS:
            if kw.get(k) is not None:
                kw[k] = tuple(kw[k])
        return cls(**kw)


@dataclass
class LayerConfig(_DictConfig):
    embed_width: int = 32
    dropout: float = 0.1
    arch_type: Literal["conv", "attn", "ssm", "both", "conv_ssm", "unified"] = "both"
    conv_kernel_sizes: tuple[int, ...] = (3, 5, 7, 9)
    conv_groups: int = 2
    use_attention: bool = True
    attn_depth: int = 2
    attn_heads: int = 2
    attn_ffn_mult: int = 4
    attn_window_size: int = 768
    attn_use_rope: bool = True
    num_attn_features: int = 4
    ssm_depth: int = 2
    ssm_state_size: int = 64
    ssm_n_heads: int = 4
    ssm_conv_kernel: int = 7
    ssm_kernel_sizes: tuple[int, ...] = (3, 5, 7, 9)
    ssm_expand: int = 2
    num_ssm_features: int = 4
    ssm_version: Literal[2, 3] = 3
    ssm_conv_type: Literal["none", "deform_se"] = "none"
    adaptive_conv: bool = False
    n_adaptive_branches: int = 3
    adaptive_kernel_size: int = 15
    adaptive_init_sigmas: tuple[float, ...] | None = None
    adaptive_min_sigma: float = 0.05
    adaptive_max_sigma: float = 0.5
    depthwise_conv: bool = False
    bias_ffn_mult: int = 2
    context_dim: int = 16
    num_embed_features: int = 4
    mlp_hidden_mult: int = 4
    mlp_output_dim: int = 32
    num_precomputed_features: int = 0
    num_heuristic_features: int = 4
    num_hidden_features: int = 8


@dataclass
class HeadConfig(_DictConfig):
    head_type: Literal["classifier", "mask"] = "classifier"
    n_classes: int = 2


@dataclass
class ModelConfig:
    n_layers: int = 1
    layer: LayerConfig | None = None
    head: HeadConfig | None = None

    def __post_init__(self):
        self.layer = self.layer or LayerConfig()
        self.head = self.head or HeadConfig()

    def to_dict(self) -> dict:
        return {"n_layers": self.n_layers, "layer": self.layer.to_dict(), "head": self.head.to_dict()}

    @classmethod
    def from_dict(cls, d: dict) -> "ModelConfig":
        return cls(n_layers=d.get("n_layers", 1), layer=LayerConfig.from_dict(d.get("layer", {})),
                   head=HeadConfig.from_dict(d.get("head", {})))


class EmbedPooler(nn.Module):
    def __init__(self, width: int, num_features: int):
        super().__init__()
        self.pooler = LearnedPooler(width, num_queries=1)
        self.proj = nn.Sequential(nn.Linear(width, num_features), nn.SiLU())

    def forward(self, h, mask=None):
        return self.proj(self.pooler(h, mask))


class PooledGate(nn.Module):
    """A backbone over the sequence, one learned-query pooling of its output, and two heads on the pooled vector:
    ``num_features`` features of this branch and one bias per feature of the whole model (the branch's own included).
    The attention and state-space "gates" of the reference's earlier two-branch classifier
    (src/heuristic_secrets/models/composed.py:206-316) are this module with different backbones."""

    def __init__(self, backbone: nn.Module, width: int, num_other_features: int, num_features: int = 4):
        super().__init__()
        self.backbone, self.pooler = backbone, LearnedPooler(width, num_queries=1)
        self.feature_proj = nn.Linear(width, num_features)
        self.bias_proj = nn.Linear(width, num_other_features + num_features)

    def forward(self, h, mask=None):
        pooled = self.pooler(self.backbone(h, mask), mask)
        return self.feature_proj(pooled), self.bias_proj(pooled)


class AttentionGate(PooledGate):
    def __init__(self, width: int, depth: int, num_heads: int, ffn_mult: int, dropout: float, num_other_features: int, num_attn_features: int = 4):
        from .attention import AttentionBackbone
        super().__init__(AttentionBackbone(width, depth, num_heads, ffn_mult, dropout), width, num_other_features, num_attn_features)
        self.num_attn_features = num_attn_features


class SSMGate(PooledGate):
    def __init__(self, width: int, depth: int, state_size: int, conv_kernel: int, conv_groups: int, expand: int, dropout: float,
                 num_other_features: int, num_ssm_features: int = 4):
        from .ssm import SSMBackbone
        super().__init__(SSMBackbone(width, depth, state_size, conv_kernel, conv_groups, expand, dropout), width, num_other_features, num_ssm_features)
        self.num_ssm_features = num_ssm_features


class SSMGate3(PooledGate):
    def __init__(self, width: int, depth: int, state_size: int, n_heads: int, expand: int, dropout: float, num_other_features: int,
                 num_ssm_features: int = 4, use_conv: bool = False, conv_kernel: int = 7, conv_groups: int = 4):
        from .ssm import SSMBackbone3
        super().__init__(SSMBackbone3(width, depth, state_size, n_heads, expand, dropout, use_conv, conv_kernel, conv_groups), width,
                         num_other_features, num_ssm_features)
        self.num_ssm_features = num_ssm_features


class HeuristicEmbed(nn.Module):
    """Scalar heuristic (one precomputed number per sample) -> small feature vector."""

    def __init__(self, output_dim: int = 4, hidden_dim: int = 16):
        super().__init__()
        self.net = nn.Sequential(nn.Linear(1, hidden_dim), nn.SiLU(), nn.Linear(hidden_dim, hidden_dim), nn.SiLU(),
                                 nn.Linear(hidden_dim, output_dim))

    def forward(self, x):
        return self.net(x.unsqueeze(-1) if x.dim() == 1 else x)


class GatedMLP(nn.Module):
    def __init__(self, input_dim: int, hidden_mult: int = 4, output_dim: int | None = None, dropout: float = 0.1):
        super().__init__()
        hidden = input_dim * hidden_mult
        self.gate_proj = nn.Linear(input_dim, hidden)
        self.up_proj = nn.Linear(input_dim, hidden)
        self.down_proj = nn.Linear(hidden, output_dim or input_dim)
        self.dropout = nn.Dropout(dropout)

    def forward(self, x):
        return self.dropout(self.down_proj(F.silu(self.gate_proj(x)) * self.up_proj(x)))


class FeatureIntegration(nn.Module):
    """Broadcast-add a projection of the per-sample feature vector onto every position, then RMSNorm."""

    def __init__(self, width: int, feature_dim: int, dropout: float = 0.1):
        super().__init__()
        self.proj = nn.Sequential(nn.Linear(feature_dim, width), nn.SiLU(), nn.Linear(width, width))
        self.norm = RMSNorm(width)
        self.dropout = nn.Dropout(dropout)

    def forward(self, h, features, mask=None):
        return self.norm(h + self.dropout(self.proj(features).unsqueeze(1)))


def _spread_sigmas(cfg: LayerConfig) -> tuple[float, ...]:
    if cfg.adaptive_init_sigmas is not None:
        return cfg.adaptive_init_sigmas
    n, lo, hi = cfg.n_adaptive_branches, cfg.adaptive_min_sigma, cfg.adaptive_max_sigma
    return tuple(lo + (hi - lo) * i / (n - 1) for i in range(n)) if n > 1 else ((lo + hi) / 2,)


class UnifiedLayer(nn.Module):
    def __init__(self, config: LayerConfig):
        super().__init__()
        self.config = c = config
        w = c.embed_width
        self.uses_adaptive_conv, self.use_attention = c.adaptive_conv, c.use_attention
        init_sigmas = _spread_sigmas(c) if c.adaptive_conv else None
        n_branches = len(init_sigmas) if c.adaptive_conv else len(c.ssm_kernel_sizes)
        self.multi_kernel_ssm = n_branches > 1
        ctx_dim = c.context_dim if c.adaptive_conv else 0
        if c.use_attention:
            if c.adaptive_conv:
                self.attn_block = ContextualAttentionBlock(w, c.attn_heads, n_branches, ctx_dim, c.attn_ffn_mult, c.dropout,
                                                           window_size=c.attn_window_size, use_rope=c.attn_use_rope)
                self.attn_pooler = None
            else:
                self.attn_block = AttentionBlock(w, c.attn_heads, c.attn_ffn_mult, c.dropout,
                                                 window_size=c.attn_window_size, use_rope=c.attn_use_rope)
                self.attn_pooler = LearnedPooler(w, num_queries=1)
            self.attn_proj = nn.Sequential(nn.Linear(w, c.num_attn_features), nn.SiLU())
        elif c.adaptive_conv:
            self.bias_proj = BiasProjection(w, n_branches, ctx_dim)
        if self.multi_kernel_ssm:
            self.ssm_block = MultiKernelSSMBlock(
                w, c.ssm_kernel_sizes, c.ssm_state_size, c.ssm_n_heads, c.ssm_expand, c.dropout, c.conv_groups,
                c.num_ssm_features, adaptive_conv=c.adaptive_conv, depthwise_conv=c.depthwise_conv, context_dim=ctx_dim,
                bias_ffn_mult=c.bias_ffn_mult, adaptive_kernel_size=c.adaptive_kernel_size, init_sigmas=init_sigmas,
                min_sigma=c.adaptive_min_sigma, max_sigma=c.adaptive_max_sigma, attn_window_size=c.attn_window_size,
                attn_use_rope=c.attn_use_rope, use_merge_attention=c.use_attention)
            self.ssm_pooler = self.ssm_proj = None
        else:
            if not c.adaptive_conv and c.ssm_kernel_sizes == (0,):
                self.ssm_block = SSMBlock3(w, c.ssm_state_size, c.ssm_n_heads, c.ssm_expand, c.dropout, use_conv=False)
            else:
                kernel = c.adaptive_kernel_size if c.adaptive_conv else (c.ssm_kernel_sizes[0] if c.ssm_kernel_sizes else c.ssm_conv_kernel)
                self.ssm_block = SSMBlock3(
                    w, c.ssm_state_size, c.ssm_n_heads, c.ssm_expand, c.dropout, use_conv=True, conv_kernel=kernel,
                    conv_groups=c.conv_groups, adaptive_conv=c.adaptive_conv, depthwise_conv=c.depthwise_conv,
                    init_sigma=init_sigmas[0] if init_sigmas else 0.3, min_sigma=c.adaptive_min_sigma,
                    max_sigma=c.adaptive_max_sigma)
            self.ssm_pooler = LearnedPooler(w, num_queries=1)
            self.ssm_proj = nn.Sequential(nn.Linear(w, c.num_ssm_features), nn.SiLU())
        self.embed_pooler = EmbedPooler(w, c.num_embed_features)
        self.hidden_pooler = LearnedPooler(w, num_queries=1)
        self.hidden_proj = nn.Sequential(nn.Linear(w, c.num_hidden_features), nn.SiLU())
        self.heuristic_embed = HeuristicEmbed(c.num_heuristic_features)
        self.total_features = ((c.num_attn_features if c.use_attention else 0) + c.num_ssm_features + c.num_embed_features
                               + c.num_hidden_features + c.num_heuristic_features)
        self.feature_integration = FeatureIntegration(w, self.total_features, c.dropout)
        self._attn_pool_query = nn.Parameter(torch.randn(1, w))
        self._attn_pool_scale = w ** -0.5

    def forward(self, h, mask=None, precomputed=None):
        biases = context = None
        feats = []
        if self.use_attention:
            if self.uses_adaptive_conv:
                h, biases, context = self.attn_block(h, mask)
                pooled = query_pool(h, self._attn_pool_query.unsqueeze(0), mask, self._attn_pool_scale).squeeze(1)
            else:
                h = self.attn_block(h, mask)
                pooled = self.attn_pooler(h, mask)
            feats.append(self.attn_proj(pooled))
        elif self.uses_adaptive_conv:
            biases, context = self.bias_proj(h, mask)
        if self.multi_kernel_ssm:
            h, ssm_features, aux = self.ssm_block(h, h, mask, biases, context)
        else:
            single = None
            if self.uses_adaptive_conv and biases is not None:
                single = AdaptiveConvBiases(biases.sigma[:, 0], biases.offset_scale[:, 0], biases.omega[:, 0])
            h, aux = self.ssm_block(h, mask, single)
            ssm_features = self.ssm_proj(self.ssm_pooler(h, mask))
        feats += [ssm_features, self.embed_pooler(h, mask), self.hidden_proj(self.hidden_pooler(h, mask))]
        if precomputed is not None:
            feats.append(self.heuristic_embed(precomputed))
        else:
            feats.append(h.new_zeros(h.shape[0], self.config.num_heuristic_features))
        features = torch.cat(feats, dim=-1)
        return self.feature_integration(h, features, mask), features, aux


class UnifiedModel(nn.Module):
    def __init__(self, config: ModelConfig):
        super().__init__()
        self.config = config
        w = config.layer.embed_width
        self.embedding = ByteEmbedding(w, config.layer.dropout)
        self.layers = nn.ModuleList([UnifiedLayer(config.layer) for _ in range(config.n_layers)])
        self.output_pooler = LearnedPooler(w, num_queries=1)
        if config.head.head_type == "classifier":
            self.head = ClassifierHead(w, config.head.n_classes)
        elif config.head.head_type == "mask":
            self.head = MaskHead(w)
        else:
            raise ValueError(f"Unknown head type: {config.head.head_type}")

    def forward(self, x, mask=None, precomputed=None):
        aux_all = {}
        h = self.embedding(x)
        for i, layer in enumerate(self.layers):
            h, _, aux = layer(h, mask, precomputed)
            aux_all.update({f"layer{i}_{k}": v for k, v in aux.items()})
        if self.config.head.head_type == "mask":
            return self.head(h), aux_all
        return self.head(self.output_pooler(h, mask)), aux_all


class Model(nn.Module):
    """Public wrapper: ``forward -> (logits, aux_losses)``, ``predict -> {0,1}`` decisions."""

    def __init__(self, config: ModelConfig):
        super().__init__()
        self.config = config
        self._impl = UnifiedModel(config)

    def forward(self, x, mask=None, precomputed=None):
        return self._impl(x, mask, precomputed)

    @torch.no_grad()
    def predict(self, x, threshold: float = 0.5, mask=None, precomputed=None):
        return (torch.sigmoid(self.forward(x, mask, precomputed)[0]) >= threshold).long()
