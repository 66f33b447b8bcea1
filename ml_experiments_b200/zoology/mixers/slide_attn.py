"""``zoology.mixers.slide_attn`` of the reference (zoology/mixers/slide_attn.py): the same public names, implemented in the modules imported below."""
# ruff: noqa: F401
from .attention import SlidingAttn, SlidingSelfAttention
