"""Language models assembled from configured mixers (zoology/model.py:11-339 of the reference).

``TokenEmbeddings`` (default / spherical / normal init, optional learned positions), the pre-norm ``TransformerBlock``
in residual-stream form (the block returns ``(hidden, residual)`` so the add lands right before the next norm) with
stochastic depth, ``LMBackbone``, ``LanguageModel`` (tied head) and ``ContinuousInputModel``; GPT-2 style scaled
initialisation of the residual output projections; recurrent-state accounting via the mixers' ``state_size``.
"""
from __future__ import annotations

import math
from functools import partial

import torch
import torch.nn as nn

from .config import ModelConfig


class StochasticDepth(nn.Module):
    """Drop whole rows (samples) of a residual branch with probability ``p`` during training, rescaling the rest."""

    def __init__(self, p: float, mode: str = "row"):
        super().__init__()
        self.p, self.mode = p, mode

    def forward(self, x):
        if not self.training or self.p == 0.0:
            return x
        shape = [x.shape[0]] + [1] * (x.dim() - 1) if self.mode == "row" else [1] * x.dim()
        keep = torch.empty(shape, dtype=x.dtype, device=x.device).bernoulli_(1.0 - self.p)
        return x * keep / (1.0 - self.p)


class TokenEmbeddings(nn.Module):
    def __init__(self, embed_dim, vocab_size, max_position_embeddings, padding_idx=None, word_embed_proj_dim=None,
                 learnable: bool = True, init_type: str = "default", device=None, dtype=torch.float32):
        super().__init__()
        dim = word_embed_proj_dim or embed_dim
        self.word_embeddings = nn.Embedding(vocab_size, dim, padding_idx=padding_idx, device=device, dtype=dtype)
        self._init_embeddings(self.word_embeddings, init_type, padding_idx)
        self.project_in = nn.Linear(word_embed_proj_dim, embed_dim, bias=False, device=device, dtype=dtype) if word_embed_proj_dim else None
        if not learnable:
            self.word_embeddings.weight.requires_grad = False
        self.max_position_embeddings = max_position_embeddings
        if max_position_embeddings > 0:
            self.position_embeddings = nn.Embedding(max_position_embeddings, embed_dim, device=device, dtype=dtype)

    @staticmethod
    def _init_embeddings(embedding: nn.Embedding, init_type: str, padding_idx=None):
        if init_type == "default":
            return  # the model-wide initialiser sets N(0, 0.02)
        with torch.no_grad():
            if init_type == "spherical":
                v = torch.randn_like(embedding.weight)
                embedding.weight.copy_(v / v.norm(dim=1, keepdim=True))
            elif init_type == "normal":
                embedding.weight.normal_(0.0, 1.0)
            else:
                raise ValueError(f"Unknown init_type: {init_type}. Choose from 'default', 'spherical', 'normal'")
            if padding_idx is not None:
                embedding.weight[padding_idx].zero_()
        embedding._no_reinit = True

    def forward(self, input_ids, position_ids=None):
        emb = self.word_embeddings(input_ids)
        if self.project_in is not None:
            emb = self.project_in(emb)
        if self.max_position_embeddings > 0:
            if position_ids is None:
                position_ids = torch.arange(input_ids.shape[1], dtype=torch.long, device=input_ids.device)
            emb = emb + self.position_embeddings(position_ids)
        return emb


def _init_weights(module, n_layers, block_type, initializer_range=0.02, rescale_prenorm_residual=True, n_residuals_per_layer=1):
    mamba = "Mamba" in block_type
    if isinstance(module, nn.Linear):
        if not mamba:
            nn.init.normal_(module.weight, std=initializer_range)
        if module.bias is not None and not getattr(module.bias, "_no_reinit", False):
            nn.init.zeros_(module.bias)
    elif isinstance(module, nn.Embedding):
        if not getattr(module, "_no_reinit", False):
            nn.init.normal_(module.weight, std=initializer_range)
    if not rescale_prenorm_residual:
        return
    # residual output projections shrink with depth (GPT-2): std / sqrt(2 * n_layers)
    for name, p in module.named_parameters():
        if mamba:
            if name in ("out_proj.weight", "fc2.weight"):
                nn.init.kaiming_uniform_(p, a=math.sqrt(5))
                with torch.no_grad():
                    p /= math.sqrt(n_residuals_per_layer * n_layers)
        elif "out_proj.weight" in name or "fc2.weight" in name or "output_linear.0.weight" in name:
            nn.init.normal_(p, mean=0.0, std=initializer_range / math.sqrt(2 * n_layers))


class TransformerBlock(nn.Module):
    def __init__(self, config: ModelConfig, layer_idx: int):
        super().__init__()
        self.sequence_mixer = config.sequence_mixer.instantiate(d_model=config.d_model, layer_idx=layer_idx)
        self.state_mixer = config.state_mixer.instantiate(d_model=config.d_model, layer_idx=layer_idx)
        self.dropout1 = nn.Dropout(config.embed_dropout if layer_idx == 0 else config.resid_dropout)
        self.drop_path1 = StochasticDepth(config.drop_path, mode="row")
        self.norm1 = nn.LayerNorm(config.d_model)
        self.dropout2 = nn.Dropout(config.resid_dropout)
        self.drop_path2 = StochasticDepth(config.drop_path, mode="row")
        self.norm2 = nn.LayerNorm(config.d_model)

    def forward(self, hidden_states, residual=None):
        dropped = self.drop_path1(self.dropout1(hidden_states))
        residual = dropped if residual is None else dropped + residual
        hidden_states = self.sequence_mixer(self.norm1(residual.to(self.norm1.weight.dtype)))
        dropped = self.drop_path2(self.dropout2(hidden_states))
        residual = dropped + residual
        return self.state_mixer(self.norm2(residual.to(self.norm2.weight.dtype))), residual


def _block_class(block_type: str):
    if block_type == "TransformerBlock":
        return TransformerBlock
    if block_type == "MambaBlock":
        from .mixers.mamba import MambaBlock
        return MambaBlock
    if block_type == "Mamba2Block":
        from .mixers.mamba2 import Mamba2Block
        return Mamba2Block
    raise ValueError(f"unknown block_type {block_type}")


class LMBackbone(nn.Module):
    def __init__(self, config: ModelConfig):
        super().__init__()
        self.embeddings = TokenEmbeddings(config.d_model, config.vocab_size, config.max_position_embeddings,
                                          learnable=config.learnable_word_embeddings, init_type=config.embedding_init_type)
        block = _block_class(config.block_type)
        self.layers = nn.ModuleList([block(config=config, layer_idx=i) for i in range(config.n_layers)])
        self.drop_f = nn.Dropout(config.resid_dropout)
        self.ln_f = nn.LayerNorm(config.d_model, eps=config.layer_norm_epsilon)
        self.apply(partial(_init_weights, n_layers=config.n_layers, block_type=config.block_type))

    def layers_forward(self, hidden_states):
        residual = None
        for layer in self.layers:
            hidden_states, residual = layer(hidden_states, residual)
        dropped = self.drop_f(hidden_states)
        residual = dropped if residual is None else dropped + residual
        return self.ln_f(residual.to(self.ln_f.weight.dtype))

    def forward(self, input_ids, position_ids=None):
        return self.layers_forward(self.embeddings(input_ids, position_ids=position_ids))


def _compute_state_size(layers, sequence_length: int):
    total = 0
    for layer in layers:
        mixer = getattr(layer, "mixer", None) or getattr(layer, "sequence_mixer", None)
        if mixer is None or not hasattr(mixer, "state_size"):
            return None
        total += mixer.state_size(sequence_length=sequence_length)
    return total * 4  # bytes of fp32 state


class LanguageModel(nn.Module):
    """Token ids -> vocabulary logits (head tied to the word embeddings when those are learnable)."""

    def __init__(self, config: ModelConfig):
        super().__init__()
        if config.vocab_size % config.pad_vocab_size_multiple:
            config.vocab_size += config.pad_vocab_size_multiple - config.vocab_size % config.pad_vocab_size_multiple
        self.backbone = LMBackbone(config)
        self.lm_head = nn.Linear(config.d_model, config.vocab_size, bias=False)
        self.apply(partial(_init_weights, n_layers=config.n_layers, block_type=config.block_type))
        if config.learnable_word_embeddings:
            self.lm_head.weight = self.backbone.embeddings.word_embeddings.weight

    def forward(self, input_ids, position_ids=None, state=None, return_embeddings: bool = False):
        hidden = self.backbone(input_ids, position_ids=position_ids)
        return hidden if return_embeddings else self.lm_head(hidden)

    def state_size(self, sequence_length: int):
        return _compute_state_size(self.backbone.layers, sequence_length)


class ContinuousInputModel(nn.Module):
    """Inputs are concatenated (key, value) embedding pairs ``[B, L, 2 d]``; outputs live in embedding space."""

    def __init__(self, config: ModelConfig):
        super().__init__()
        config = config.model_copy()
        self.input_proj = nn.Linear(config.d_model * 2, config.d_model)
        self.backbone = LMBackbone(config)
        self.output_proj = nn.Linear(config.d_model, config.d_model)

    def forward(self, x):
        return self.output_proj(self.backbone.layers_forward(self.input_proj(x)))

    def state_size(self, sequence_length: int):
        return _compute_state_size(self.backbone.layers, sequence_length)
