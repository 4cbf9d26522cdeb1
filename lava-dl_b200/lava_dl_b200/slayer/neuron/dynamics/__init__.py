"""Neuron dynamics primitives (mirror of ``lava.lib.dl.slayer.neuron.dynamics``)."""

from . import leaky_integrator, adaptive_threshold, resonator, adaptive_phase_th, adaptive_resonator

__all__ = ['leaky_integrator', 'adaptive_threshold', 'resonator', 'adaptive_phase_th', 'adaptive_resonator']
