"""Blocks: synapse + neuron + delay (mirror of ``lava.lib.dl.slayer.block`` for
the real-valued neuron families)."""

from . import base, cuba, alif

__all__ = ['base', 'cuba', 'alif']
