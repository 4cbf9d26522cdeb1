"""Synapses (mirror of the real-valued part of ``lava.lib.dl.slayer.synapse``).

These sit next to the hot path, not on it: they are thin ``torch.nn.Conv3d``
subclasses with a unit time kernel and run in cuDNN, exactly as in the
reference (``src/lava/lib/dl/slayer/synapse/layer.py``).  They exist so that
the blocks, and through them whole networks, can be assembled around the
neuron kernels.
"""

from .layer import Dense, Conv, Pool

__all__ = ['Dense', 'Conv', 'Pool']
