"""``zoology.mixers.listing`` of the reference (zoology/mixers/listing.py): the same public names, implemented in the modules imported below."""
# ruff: noqa: F401
from .base_conv import BaseConv
from .convolution import PositionalEmbedding, fft_conv
