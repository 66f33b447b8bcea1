"""``heuristic_secrets.models.combiner``: feature combiner (reference: src/heuristic_secrets/models/combiner.py). Re-
exports."""
# ruff: noqa: F401
from ...models.unified.features import FeatureCombiner
