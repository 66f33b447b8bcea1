"""Optimizers: Muon (classic), NorMuon+Adam, DistAdam, Dion, fused Adam."""
from .adam import FusedAdam  # noqa: F401
from .muon import Muon  # noqa: F401
from .dion import Dion  # noqa: F401
