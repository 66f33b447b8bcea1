"""``zoology.mixers.scatterbrain_new`` of the reference (zoology/mixers/scatterbrain_new.py): the same public names, implemented in the modules imported below."""
# ruff: noqa: F401
from .feature_maps import init_feature_map
from .scatterbrain import ScatterBrain
