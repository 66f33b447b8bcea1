"""``heuristic_secrets.models.ponder``: ponder wrapper and its trainer (reference:
src/heuristic_secrets/models/ponder.py). Re-exports."""
# ruff: noqa: F401
from ...models.unified.ponder import InternalLossNetwork, PonderTrainConfig, PonderTrainer, PonderWrapper, SiLUAttentionBlock
