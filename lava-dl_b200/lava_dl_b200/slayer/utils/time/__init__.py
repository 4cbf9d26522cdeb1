"""Time-axis manipulation (mirror of ``lava.lib.dl.slayer.utils.time``)."""

from .shift import shift

__all__ = ['shift']
