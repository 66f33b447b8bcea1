"""``zoology.mixers.delta_net`` of the reference (zoology/mixers/delta_net.py): the same public names, implemented in the modules imported below."""
# ruff: noqa: F401
from .linear_attn import elu_p1, sum_norm, DeltaNet
