"""``heuristic_secrets.models.ripple_attention``: Ripple attention, blocks and classifier (reference:
src/heuristic_secrets/models/ripple_attention.py). Re-exports."""
# ruff: noqa: F401
from ...models.ripple import (
    CrossLayerAttention, LayerHistoryAccumulator, LearnedSinusoidal2DEmbed, RippleAttention, RippleBlock, RippleClassifier
)
from ...models.ripple_channel import ChannelMixer, ChannelSegment, RippleChannelClassifier
from ...models.ripple_ops import CausalSelfAttention, ReLUSquared, relu_squared

HAS_TRITON = True   # "a fused kernel path exists": the CUDA kernels of this package stand where the reference has Triton programs
