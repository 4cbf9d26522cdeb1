"""Axon models (mirror of ``lava.lib.dl.slayer.axon``)."""

from .delay import delay, Delay
from .delta import Delta

__all__ = ['delay', 'Delay', 'Delta']
