"""Blocks: synapse + neuron + delay (mirror of ``lava.lib.dl.slayer.block`` for
the real-valued neuron families)."""

from . import base, cuba, alif, sigma_delta

__all__ = ['base', 'cuba', 'alif', 'sigma_delta']
