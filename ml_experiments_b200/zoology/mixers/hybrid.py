"""``Hybrid``: picks one of several mixer configs by layer index (zoology/mixers/hybrid.py:12-39)."""
from typing import List

import torch.nn as nn

from ..config import ModuleConfig


class Hybrid(nn.Module):
    def __init__(self, d_model: int, configs: List, layer_idx: int = None, **kwargs):
        super().__init__()
        self.d_model = d_model
        cfg = configs[layer_idx % len(configs)]
        cfg = cfg if isinstance(cfg, ModuleConfig) else ModuleConfig(**cfg)
        self.mixer = cfg.instantiate(d_model=d_model, layer_idx=layer_idx)

    def forward(self, u, *args, **kwargs):
        return self.mixer(u, *args, **kwargs)

    def state_size(self, **kwargs):
        return self.mixer.state_size(**kwargs)
