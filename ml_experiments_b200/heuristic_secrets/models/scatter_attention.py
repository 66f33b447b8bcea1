"""``heuristic_secrets.models.scatter_attention``: scatter / local / hierarchical / SGSB / flat-ripple family, MIMO-
Jacobi state-space model (reference: src/heuristic_secrets/models/scatter_attention.py). Re-exports."""
# ruff: noqa: F401
from ...models.jacobi import MIMOJacobiBlock, MIMOJacobiBlock_ND, MIMOJacobiSSM, MIMOJacobiSSM_ND
from ...models.ripple_ops import LowRankAttention
from ...models.scatter import (
    AdaptiveConvND, FlatRipple, FlatRippleClassifier, FlatRippleClassifierND, FlatRippleND, GatedMerge, HierarchicalLocalAttention,
    HierarchicalLocalAttentionND, HierarchicalLocalBlock, HierarchicalLocalBlockND, KernelNetND, LearnedMerge, LocalAttention,
    LocalAttentionND, LocalBlock, LowRankAttentionMerge, LowRankAttentionMergeND, LowRankAttentionND, LowRankCollapseMerge, RMSNorm,
    RippleClassifierND, RippleLayer, RippleLayerND, RippleModel, RippleModelND, SEBlock1d, SGSBAttention, SGSBAttentionND, SGSBBlock,
    SGSBBlockND, SGSBClassifier, SGSBClassifierND, SGSBModel, SGSBModelND, SIRENDownsampleND, SIRENUpsampleND, ScatterAttention1d, Sine,
    SqueezeExciteND, apply_rope, avg_pool_nd, interpolate_nd, relu_squared, sinusoidal_pos_embed, sinusoidal_pos_embed_nd
)
from ...models.unified.two_d import SEBlock2d
from ...models.scatter import LayerwiseRippleClassifier as RippleClassifier   # the reference's name for the 1-D layerwise classifier

HAS_TRITON = True   # "a fused kernel path exists": the CUDA kernels of this package stand where the reference has Triton programs
HAS_TRITON_ADAPTIVE = True
