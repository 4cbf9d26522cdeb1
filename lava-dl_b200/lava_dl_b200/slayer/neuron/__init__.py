"""Neuron models on the hot path (mirror of ``lava.lib.dl.slayer.neuron``)."""

from . import dynamics, base, cuba, alif, rf, rf_iz, adrf, adrf_iz, sigma_delta  # noqa: F401

__all__ = ['dynamics', 'base', 'cuba', 'alif', 'rf', 'rf_iz', 'adrf', 'adrf_iz', 'sigma_delta']
