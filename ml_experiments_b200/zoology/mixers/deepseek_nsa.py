"""``zoology.mixers.deepseek_nsa`` of the reference (zoology/mixers/deepseek_nsa.py): the same public names, implemented in the modules imported below."""
# ruff: noqa: F401
from .nsa import SparseAttention
