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
import torch.nn.functional as F

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
    """Word embeddings (optionally of a narrower width with an input projection, optionally frozen) plus optional
    learned absolute positions. ``init_type``: ``default`` leaves the table to the model-wide initialiser;
    ``spherical`` puts every row on the unit sphere; ``normal`` draws N(0, 1)."""

    def __init__(self, embed_dim, vocab_size, max_position_embeddings, padding_idx=None, word_embed_proj_dim=None,
                 learnable: bool = True, init_type: str = "default", device=None, dtype=torch.float32):
        super().__init__()
        kw = dict(device=device, dtype=dtype)
        narrow = word_embed_proj_dim is not None and word_embed_proj_dim > 0
        self.word_embeddings = nn.Embedding(vocab_size, word_embed_proj_dim if narrow else embed_dim, padding_idx=padding_idx, **kw)
        self.project_in = nn.Linear(word_embed_proj_dim, embed_dim, bias=False, **kw) if narrow else None
        self.max_position_embeddings = max_position_embeddings
        if max_position_embeddings > 0:
            self.position_embeddings = nn.Embedding(max_position_embeddings, embed_dim, **kw)
        self._init_embeddings(self.word_embeddings, init_type, padding_idx)
        self.word_embeddings.weight.requires_grad_(learnable)

    @staticmethod
    def _init_embeddings(embedding: nn.Embedding, init_type: str, padding_idx=None):
        draw = {"default": None, "spherical": lambda w: F.normalize(torch.randn_like(w), dim=1),
                "normal": lambda w: torch.randn_like(w)}
        if init_type not in draw:
            raise ValueError(f"Unknown init_type: {init_type}. Choose from 'default', 'spherical', 'normal'")
        if draw[init_type] is None:
            return
        with torch.no_grad():
            embedding.weight.copy_(draw[init_type](embedding.weight))
            if padding_idx is not None:
                embedding.weight[padding_idx] = 0
        embedding._no_reinit = True      # the model-wide initialiser must not overwrite it

    def forward(self, input_ids, position_ids=None):
        x = self.word_embeddings(input_ids)
        if self.project_in is not None:
            x = self.project_in(x)
        if self.max_position_embeddings > 0:
            pos = position_ids if position_ids is not None else torch.arange(input_ids.shape[1], device=input_ids.device)
            x = x + self.position_embeddings(pos)
        return x


# Parameters that write into the residual stream: their initial scale shrinks with depth.
_RESIDUAL_OUTPUTS = ("out_proj.weight", "fc2.weight", "output_linear.0.weight")


def _init_weights(module, n_layers, block_type, initializer_range=0.02, rescale_prenorm_residual=True, n_residuals_per_layer=1):
    """Applied to every sub-module (``nn.Module.apply``): N(0, ``initializer_range``) for linear and embedding
    weights, zero biases, and GPT-2's 1/sqrt(2 n_layers) shrink of everything that writes into the residual stream.
    Mamba blocks keep their own linear initialisation; their residual outputs are re-drawn Kaiming-uniform and
    divided by sqrt(n_residuals_per_layer * n_layers). Tensors marked ``_no_reinit`` are left alone."""
    is_mamba = "Mamba" in block_type
    skip = lambda t: t is None or getattr(t, "_no_reinit", False)
    if isinstance(module, nn.Embedding) and not skip(module):
        nn.init.normal_(module.weight, std=initializer_range)
    if isinstance(module, nn.Linear):
        if not is_mamba:
            nn.init.normal_(module.weight, std=initializer_range)
        if not skip(module.bias):
            nn.init.zeros_(module.bias)
    if not rescale_prenorm_residual:
        return
    for name, p in module.named_parameters():
        if is_mamba and name in _RESIDUAL_OUTPUTS[:2]:
            nn.init.kaiming_uniform_(p, a=math.sqrt(5))
            with torch.no_grad():
                p.div_(math.sqrt(n_residuals_per_layer * n_layers))
        elif not is_mamba and any(tag in name for tag in _RESIDUAL_OUTPUTS):
            nn.init.normal_(p, mean=0.0, std=initializer_range / math.sqrt(2 * n_layers))


def _join_stream(branch, residual, dropout, drop_path, norm):
    """Residual-stream bookkeeping shared by the blocks and the backbone's last norm: regularise the branch output,
    add it to the stream (which starts as the first branch output), return ``(norm(stream), stream)``."""
    branch = drop_path(dropout(branch)) if drop_path is not None else dropout(branch)
    stream = branch if residual is None else branch + residual
    return norm(stream.to(norm.weight.dtype)), stream


class TransformerBlock(nn.Module):
    """Pre-norm block in residual-stream form: it receives the previous branch output and the stream, and returns its
    own last branch output and the updated stream, so every add sits right before the norm that consumes it."""

    def __init__(self, config: ModelConfig, layer_idx: int):
        super().__init__()
        d = config.d_model
        self.sequence_mixer = config.sequence_mixer.instantiate(d_model=d, layer_idx=layer_idx)
        self.state_mixer = config.state_mixer.instantiate(d_model=d, layer_idx=layer_idx)
        self.dropout1 = nn.Dropout(config.embed_dropout if layer_idx == 0 else config.resid_dropout)
        self.dropout2 = nn.Dropout(config.resid_dropout)
        self.drop_path1, self.drop_path2 = StochasticDepth(config.drop_path, mode="row"), StochasticDepth(config.drop_path, mode="row")
        self.norm1, self.norm2 = nn.LayerNorm(d), nn.LayerNorm(d)

    def forward(self, hidden_states, residual=None):
        normed, residual = _join_stream(hidden_states, residual, self.dropout1, self.drop_path1, self.norm1)
        normed, residual = _join_stream(self.sequence_mixer(normed), residual, self.dropout2, self.drop_path2, self.norm2)
        return self.state_mixer(normed), residual


def _block_class(block_type: str):
    if block_type == "TransformerBlock":
        return TransformerBlock
    lazy = {"MambaBlock": ".mixers.mamba", "Mamba2Block": ".mixers.mamba2"}
    if block_type not in lazy:
        raise ValueError(f"unknown block_type {block_type}")
    import importlib

    return getattr(importlib.import_module(lazy[block_type], __package__), block_type)


class LMBackbone(nn.Module):
    def __init__(self, config: ModelConfig):
        super().__init__()
        self.embeddings = TokenEmbeddings(config.d_model, config.vocab_size, config.max_position_embeddings,
                                          learnable=config.learnable_word_embeddings, init_type=config.embedding_init_type)
        block = _block_class(config.block_type)
        self.layers = nn.ModuleList(block(config=config, layer_idx=i) for i in range(config.n_layers))
        self.drop_f = nn.Dropout(config.resid_dropout)
        self.ln_f = nn.LayerNorm(config.d_model, eps=config.layer_norm_epsilon)
        self.apply(partial(_init_weights, n_layers=config.n_layers, block_type=config.block_type))

    def layers_forward(self, hidden_states):
        residual = None
        for layer in self.layers:
            hidden_states, residual = layer(hidden_states, residual)
        return _join_stream(hidden_states, residual, self.drop_f, None, self.ln_f)[0]

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
