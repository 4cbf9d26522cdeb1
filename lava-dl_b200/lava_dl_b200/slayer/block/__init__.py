"""Blocks: synapse + neuron + delay (mirror of ``lava.lib.dl.slayer.block``)."""

from . import base, cuba, alif, rf, adrf, rf_iz, adrf_iz, sigma_delta

__all__ = ['base', 'cuba', 'alif', 'rf', 'adrf', 'rf_iz', 'adrf_iz', 'sigma_delta']
