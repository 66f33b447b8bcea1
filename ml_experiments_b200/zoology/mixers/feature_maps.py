"""Query / key feature maps for linear attention (zoology/mixers/feature_maps/*.py): identity, positive ELU, ReLU,
square, the 2nd-order Taylor expansion of ``exp`` (Based), learned polynomial maps, Performer random features
(FAVOR+) and the cosFormer position re-weighting. All map ``[B, H, L, D] -> [B, H, L, expanded_size()]``."""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F


class FeatureMap(nn.Module):
    def __init__(self, input_dim: int, temp: float | None = None, head_dim_idx: int = -1, eps: float = 1e-12, **kwargs):
        super().__init__()
        self.input_dim, self.head_dim_idx, self.eps = input_dim, head_dim_idx, eps
        self.temp = 1.0 if temp is None else temp

    def forward(self, x):
        return x

    def expanded_size(self) -> int:
        return self.input_dim


Identity = FeatureMap


class PosELU(FeatureMap):
    def forward(self, x):
        return F.elu(x * self.temp) + 1


class ReLU(FeatureMap):
    def forward(self, x):
        return F.relu(x * self.temp).clamp(min=self.eps)


class Square(FeatureMap):
    def forward(self, x):
        return x ** 2


class SquaredMap(FeatureMap):
    def forward(self, x):
        return x * x / math.sqrt(2)


class TaylorExp(FeatureMap):
    """``f(x) . f(y) = 1 + x.y / sqrt(d) + (x.y)^2 / (2 d)``: features ``[1, x / d^(1/4), vec(x x^T) / (sqrt(2) sqrt(d))]``."""

    def __init__(self, input_dim: int, **kwargs):
        super().__init__(input_dim, **kwargs)
        self.r2, self.rd = math.sqrt(2), math.sqrt(input_dim)
        self.rrd = math.sqrt(self.rd)

    def forward(self, x):
        x2 = (x.unsqueeze(-1) * x.unsqueeze(-2)).flatten(start_dim=-2) / self.r2
        return torch.cat([torch.ones_like(x[..., :1]), x / self.rrd, x2 / self.rd], dim=self.head_dim_idx)

    def expanded_size(self) -> int:
        return 1 + self.input_dim + self.input_dim ** 2


class AllPolyMap(FeatureMap):
    """Learned degree-2 map ``(W1 x)^2 + W2 (x^2)``."""

    def __init__(self, input_dim: int, output_dim: int | None = None, init: str = "randn", learnable: bool = True, **kwargs):
        super().__init__(input_dim, **kwargs)
        self.output_dim = output_dim if output_dim is not None else input_dim
        self.proj_1 = nn.Linear(input_dim, self.output_dim, bias=False)
        self.proj_2 = nn.Linear(input_dim, self.output_dim, bias=False)
        with torch.no_grad():
            if init == "randn":
                nn.init.normal_(self.proj_1.weight, std=1 / math.sqrt(input_dim))
                nn.init.normal_(self.proj_2.weight, std=1 / math.sqrt(input_dim))
            elif init == "plusminus":
                for p in (self.proj_1, self.proj_2):
                    p.weight.copy_((torch.rand_like(p.weight) > 0.5) * 2.0 - 1.0)
            elif init != "kaiming":
                raise ValueError(f"Invalid init method: {init}")
        if not learnable:
            for p in self.parameters():
                p.requires_grad = False

    def forward(self, x):
        return (self.proj_1(x) ** 2 + self.proj_2(x ** 2)) / math.sqrt(2)

    def expanded_size(self) -> int:
        return self.output_dim


class PerformerFeatureMap(FeatureMap):
    """Positive orthogonal random features: ``exp(-|x|^2 / 2) / sqrt(m) * exp(W x)`` with block-orthogonal ``W``."""

    def __init__(self, input_dim: int = 16, expanded_dim: int = 256, **kwargs):
        super().__init__(input_dim=input_dim, **kwargs)
        self.expanded_dim = expanded_dim
        blocks, left = [], expanded_dim
        while left > 0:
            q, _ = torch.linalg.qr(torch.randn(input_dim, input_dim))
            blocks.append(q.T[:min(left, input_dim)])
            left -= input_dim
        w = torch.cat(blocks) / math.sqrt(expanded_dim / input_dim)
        self.register_buffer("random_feats", w)

    def forward(self, x):
        x = x / x.shape[-1] ** 0.25
        h = torch.exp(-x.pow(2).sum(dim=-1, keepdim=True) / 2)
        return h / math.sqrt(self.expanded_dim) * torch.exp(x @ self.random_feats.T.to(x.dtype))

    def expanded_size(self) -> int:
        return self.expanded_dim


class CosFormerFeatureMap(FeatureMap):
    """``[act(x) sin(pi i / 2L), act(x) cos(pi i / 2L)]`` for position ``i`` of ``L``."""

    def __init__(self, act_fun: str = "relu", *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.act_fun = F.relu if act_fun == "relu" else (lambda t: 1 + F.elu(t))

    def forward(self, x):
        L = x.shape[2]
        idx = (math.pi / 2 * torch.arange(1, L + 1, device=x.device, dtype=x.dtype) / L).view(1, 1, L, 1)
        x = self.act_fun(x)
        return torch.cat([x * torch.sin(idx), x * torch.cos(idx)], dim=-1)

    def expanded_size(self) -> int:
        return 2 * self.input_dim


class FullSpaceMap(nn.Module):
    """``[x, -x]`` along the feature dimension, clamped positive: lets a positive map see both signs of its input."""

    def __init__(self, head_dim_idx: int = -1, eps: float = 1e-12, **kwargs):
        super().__init__()
        self.head_dim_idx, self.eps = head_dim_idx, eps

    def forward(self, x, fmap=None):
        return torch.cat([x, -x], dim=self.head_dim_idx).clamp(min=self.eps)


class ExpDim(FeatureMap):
    """The "spiky" maps of the feature-map ablations (zoology/mixers/feature_maps/exp_dim.py): an exponential of the
    (temperature-scaled) input per element or normalised over the feature dimension. ``fullspace`` doubles the
    features with the negated input. Sub-classes choose the normalisation."""
    normalise = "none"          # none | max | softmax | abs-softmax
    halfspace = False           # only the positive half (no doubling)

    def __init__(self, fullspace: bool = True, **kwargs):
        super().__init__(**kwargs)
        self.fs_map = FullSpaceMap(head_dim_idx=self.head_dim_idx, eps=self.eps) if fullspace else nn.Identity()

    def forward(self, x):
        d = self.head_dim_idx
        if self.normalise == "abs-softmax":            # softmax of |x|, routed to the half of its sign
            w = x.abs().softmax(dim=d) if self.halfspace else (x * self.temp).abs().softmax(dim=d)
            if self.halfspace:
                return ((x >= 0) * w).clamp(min=self.eps)
            xs = x * self.temp
            return torch.stack([(xs >= 0) * w, (xs < 0) * w], dim=-1).flatten(-2).clamp(min=self.eps)
        x = x * self.temp
        if self.normalise == "softmax":
            pos = torch.softmax(x, dim=d)
            return (pos if self.halfspace else torch.cat([pos, torch.softmax(-x, dim=d)], dim=d)).clamp(min=self.eps)
        if self.normalise == "max":
            x = x - x.amax(d, keepdim=True)
        return torch.exp(self.fs_map(x))

    def expanded_size(self) -> int:
        doubled = (self.normalise in ("softmax", "abs-softmax") and not self.halfspace) or \
                  (self.normalise in ("none", "max") and isinstance(self.fs_map, FullSpaceMap))
        return self.input_dim * (2 if doubled else 1)


class ExpMaxNorm(ExpDim):
    normalise = "max"


class SoftmaxDim(ExpDim):
    normalise = "softmax"


class SoftmaxDimHalfspace(ExpDim):
    normalise, halfspace = "softmax", True


class ExpSumNorm(ExpDim):
    normalise = "abs-softmax"


class ExpSumNormHalfspace(ExpDim):
    normalise, halfspace = "abs-softmax", True


_MAPS = {None: FeatureMap, "none": FeatureMap, "identity": FeatureMap, "taylor_exp": TaylorExp, "performer": PerformerFeatureMap,
         "cosformer": CosFormerFeatureMap, "pos_elu": PosELU, "relu": ReLU, "square": Square, "all_poly": AllPolyMap}


def init_feature_map(feature_map="none", **kwargs):
    if feature_map in _MAPS:
        return _MAPS[feature_map](**kwargs)
    from ..utils import import_from_str
    return import_from_str(feature_map)(**kwargs)
