"""``zoology.mixers.gla`` of the reference (zoology/mixers/gla.py): the same public names, implemented in the modules imported below."""
# ruff: noqa: F401
from .linear_attn import GatedLinearAttention
