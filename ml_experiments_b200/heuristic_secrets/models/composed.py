"""``heuristic_secrets.models.composed``: the unified byte model: configs, layers, feature integration, Model (reference:
src/heuristic_secrets/models/composed.py). Re-exports."""
# ruff: noqa: F401
from ...models.unified.composed import (
    AttentionGate, EmbedPooler, FeatureIntegration, GatedMLP, HeadConfig, HeuristicEmbed, LayerConfig, Model, ModelConfig, SSMGate,
    SSMGate3, UnifiedLayer, UnifiedModel
)
from ...models.unified.features import ConvBranch
from ...models.unified.layers import LearnedPooler, check_nan
