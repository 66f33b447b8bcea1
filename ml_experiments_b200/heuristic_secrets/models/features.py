"""``heuristic_secrets.models.features``: feature makers of the earlier feature-combining classifier (reference:
src/heuristic_secrets/models/features.py). Re-exports."""
# ruff: noqa: F401
from ...models.unified.features import AttentionFeature, ConvBranch, ConvFeature, FeatureMaker, HeuristicFeature, PrecomputedFeature
