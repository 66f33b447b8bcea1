"""Residual-fused RMSNorm / LayerNorm (zoology/mixers/mamba_ssm/ops/triton/layer_norm.py, layernorm.py)."""
# ruff: noqa: F401
from ....norms import RMSNorm, layer_norm_fn, layer_norm_ref, rms_norm_fn, rms_norm_ref
