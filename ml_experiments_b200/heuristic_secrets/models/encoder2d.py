"""``heuristic_secrets.models.encoder2d``: pixel embeddings (reference: src/heuristic_secrets/models/encoder2d.py). Re-
exports."""
# ruff: noqa: F401
from ...models.unified.two_d import PixelEmbedding2d, PixelEmbedding2dLearned, RMSNorm2d, get_2d_sinusoidal_pos_embed
