"""Temporal filtering (mirror of ``lava.lib.dl.slayer.utils.filter``)."""

from .conv import conv, corr
from .fir import FIR, FIRBank

__all__ = ['conv', 'corr', 'FIR', 'FIRBank']
