# ruff: noqa: F401
from ...norms import RMSNorm, layer_norm_fn, rms_norm_fn
