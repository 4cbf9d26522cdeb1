"""Drop-in mirror of the hot-path part of ``lava.lib.dl.slayer``."""

from . import jitconfig, utils, axon, dendrite, spike, neuron, synapse, block  # noqa: F401

__all__ = ['jitconfig', 'utils', 'axon', 'dendrite', 'spike', 'neuron', 'synapse', 'block']
