"""Ensemble of identically configured models evaluated in one vectorised call.

As in src/heuristic_secrets/models/ensemble.py:9-38 the members' parameters are stacked with
``torch.func.stack_module_state`` and a single ``vmap(functional_call)`` produces all members' logits; the ensemble
returns the mean (and variance) of their probabilities. The stacked state is cached between calls in eval mode.
"""
from __future__ import annotations

import copy

import torch
import torch.nn as nn
from torch.func import functional_call, stack_module_state

from .composed import Model, ModelConfig


class Ensemble(nn.Module):
    def __init__(self, config: ModelConfig, n_members: int = 5):
        super().__init__()
        self.config, self.n_members = config, n_members
        self.models = nn.ModuleList([Model(config) for _ in range(n_members)])
        self._stacked = None

    def train(self, mode: bool = True):
        self._stacked = None
        return super().train(mode)

    def _member_probs(self, x, mask, precomputed):
        if self.training or self._stacked is None:
            self._stacked = stack_module_state(list(self.models))
        params, buffers = self._stacked
        template = copy.deepcopy(self.models[0]).to("meta")

        def one(p, b, x, mask, precomputed):
            return functional_call(template, (p, b), (x, mask, precomputed))[0]

        logits = torch.vmap(one, in_dims=(0, 0, None, None, None), randomness="different")(params, buffers, x, mask, precomputed)
        return torch.sigmoid(logits)

    def forward(self, x, mask=None, precomputed=None):
        return self._member_probs(x, mask, precomputed).mean(dim=0)

    def forward_with_variance(self, x, mask=None, precomputed=None):
        p = self._member_probs(x, mask, precomputed)
        return p.mean(dim=0), p.var(dim=0)
