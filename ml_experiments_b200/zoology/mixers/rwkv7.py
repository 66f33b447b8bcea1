"""``zoology.mixers.rwkv7`` of the reference (zoology/mixers/rwkv7.py): the same public names, implemented in the modules imported below."""
# ruff: noqa: F401
from .linear_attn import RWKV7Attention
