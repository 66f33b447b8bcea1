"""``heuristic_secrets.models.backbone``: 1-D building blocks: deformable / adaptive convolutions, attention blocks, S6
and scalar-decay state-space mixers and backbones (reference: src/heuristic_secrets/models/backbone.py). Re-exports."""
# ruff: noqa: F401
from ...models.scatter import Sine
from ...models.unified.attention import AttentionBackbone, AttentionBlock, ContextualAttentionBlock
from ...models.unified.deform import (
    AdaptiveConvBiases, AdaptiveConvBranch, AdaptiveDeformConv1d, BiasProjection, ConvBackbone, ConvBlock, DeformConv1d, KernelNet1d,
    SIRENLayer
)
from ...models.unified.layers import (
    RMSNorm, RotaryEmbedding, SEBlock, SwiGLU, apply_rotary_emb, apply_rotary_pos_emb_qk, check_nan, chunked_local_attention
)
from ...models.unified.ssm import MultiKernelSSMBlock, SSMBackbone, SSMBackbone3, SSMBlock, SSMBlock3, SSMMixer, SSMMixer3
