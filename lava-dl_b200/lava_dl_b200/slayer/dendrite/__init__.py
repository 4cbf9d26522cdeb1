"""Dendrite models (mirror of ``lava.lib.dl.slayer.dendrite``)."""

from .sigma import Sigma

__all__ = ['Sigma']
