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
        self._loop = False
        self._streams = None

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

        if not self._loop:
            try:
                logits = torch.vmap(one, in_dims=(0, 0, None, None, None), randomness="different")(params, buffers, x, mask, precomputed)
                return torch.sigmoid(logits)
            except (RuntimeError, NotImplementedError):
                # a hand-written CUDA op without a batching rule: run the members one after another on side streams
                self._loop = True
        return torch.sigmoid(self._member_logits_loop(x, mask, precomputed))

    def _member_logits_loop(self, x, mask, precomputed):
        if not x.is_cuda:
            return torch.stack([m(x, mask, precomputed)[0] for m in self.models])
        cur = torch.cuda.current_stream(x.device)
        if self._streams is None or len(self._streams) != self.n_members:
            self._streams = [torch.cuda.Stream(x.device) for _ in range(self.n_members)]
        outs = []
        for m, st in zip(self.models, self._streams):
            st.wait_stream(cur)
            with torch.cuda.stream(st):
                outs.append(m(x, mask, precomputed)[0])
        for st in self._streams:
            cur.wait_stream(st)
        return torch.stack(outs)

    def forward(self, x, mask=None, precomputed=None):
        return self._member_probs(x, mask, precomputed).mean(dim=0)

    def forward_with_variance(self, x, mask=None, precomputed=None):
        p = self._member_probs(x, mask, precomputed)
        return p.mean(dim=0), p.var(dim=0)
