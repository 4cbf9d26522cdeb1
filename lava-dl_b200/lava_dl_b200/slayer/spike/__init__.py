"""Spike mechanisms (mirror of ``lava.lib.dl.slayer.spike``)."""

from .spike import Spike
from . import complex

__all__ = ['Spike', 'complex']
