"""``BaseConv``: ``conv(u) * proj(u) + u`` with a short or (implicit) long convolution (zoology/mixers/base_conv.py:14-65)."""
from __future__ import annotations

from typing import List, Union

import torch.nn as nn

from .convolution import ImplicitLongConvolution, LongConvolution, ShortConvolution


class BaseConv(nn.Module):
    def __init__(self, d_model: int, l_max: int, kernel_size: Union[int, List[int]] = 3, layer_idx: int = None,
                 implicit_long_conv: bool = True, use_act: bool = False, **kwargs):
        super().__init__()
        self.d_model, self.l_max, self.layer_idx, self.use_act = d_model, l_max, layer_idx, use_act
        self.projection = nn.Linear(d_model, d_model)
        if use_act:
            self.act = nn.SiLU()
        if isinstance(kernel_size, (list, tuple)):
            if layer_idx is None or layer_idx >= len(kernel_size):
                raise ValueError("kernel_size must be an int or a list of ints with length equal to the number of layers")
            kernel_size = kernel_size[layer_idx]
        if kernel_size == -1:
            self.conv = (ImplicitLongConvolution if implicit_long_conv else LongConvolution)(d_model, l_max=l_max)
        else:
            self.conv = ShortConvolution(d_model, kernel_size=kernel_size)

    def forward(self, u, *args, **kwargs):
        c, p = self.conv(u), self.projection(u)
        return (self.act(c) * self.act(p) if self.use_act else c * p) + u

    def state_size(self, sequence_length: int):
        return self.conv.state_size(sequence_length=sequence_length)
