"""``zoology.mixers.rwkv5`` of the reference (zoology/mixers/rwkv5.py): the same public names, implemented in the modules imported below."""
# ruff: noqa: F401
from .rwkv import RWKVTimeMixer, RWKV_ChannelMix
