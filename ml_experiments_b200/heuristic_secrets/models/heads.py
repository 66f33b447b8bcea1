"""``heuristic_secrets.models.heads``: classifier and mask heads (reference: src/heuristic_secrets/models/heads.py). Re-
exports."""
# ruff: noqa: F401
from ...models.unified.layers import BinaryHead, ClassifierHead, MaskHead
