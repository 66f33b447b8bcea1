"""``heuristic_secrets.models.adaptive_local_conv``: adaptive local convolution (reference:
src/heuristic_secrets/models/adaptive_local_conv.py). Re-exports."""
# ruff: noqa: F401
from ...models.ripple_ops import AdaptiveLocalConv, AdaptiveLocalConvBlock, SqueezeExcite1D, llama_rmsnorm
