"""``heuristic_secrets.models.backbone2d``: 2-D building blocks (image grids) (reference:
src/heuristic_secrets/models/backbone2d.py). Re-exports."""
# ruff: noqa: F401
from ...models.ripple_ops import RMSNorm
from ...models.unified.layers import SwiGLU, check_nan
from ...models.unified.two_d import (
    AdaptiveConvBiases2d, AdaptiveConvBranch2d, AdaptiveDeformConv2d, AttentionBlock2d, BiasProjection2d, ContextualAttentionBlock2d,
    DeformConv2d, MultiKernelSSMBlock2d, RotaryEmbedding2d, SEBlock2d, SSMBlock3_2d, apply_rotary_pos_emb_2d, apply_rotary_pos_emb_qk_2d
)
