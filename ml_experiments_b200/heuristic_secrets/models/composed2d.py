"""``heuristic_secrets.models.composed2d``: the unified image model (reference:
src/heuristic_secrets/models/composed2d.py). Re-exports."""
# ruff: noqa: F401
from ...models.unified.two_d import (
    EmbedPooler2d, FeatureIntegration2d, HeadConfig2d, LayerConfig2d, LearnedPooler2d, Model2d, ModelConfig2d, UnifiedLayer2d,
    UnifiedModel2d
)
