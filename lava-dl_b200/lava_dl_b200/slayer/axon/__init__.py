"""Axonal delay (mirror of ``lava.lib.dl.slayer.axon``)."""

from .delay import delay, Delay

__all__ = ['delay', 'Delay']
