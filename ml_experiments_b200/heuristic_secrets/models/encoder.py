"""``heuristic_secrets.models.encoder``: byte embedding (reference: src/heuristic_secrets/models/encoder.py). Re-exports."""
# ruff: noqa: F401
from ...models.unified.layers import ByteEmbedding, RMSNorm
