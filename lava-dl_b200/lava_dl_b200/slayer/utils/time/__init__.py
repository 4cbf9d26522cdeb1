"""Time-axis manipulation (mirror of ``lava.lib.dl.slayer.utils.time``)."""

from .shift import shift
from .replicate import replicate

__all__ = ['shift', 'replicate']
