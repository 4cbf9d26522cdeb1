"""CUBA-LIF blocks (``src/lava/lib/dl/slayer/block/cuba.py``); 8-bit quantisation ready."""

from ._family import make_blocks
from ..neuron import cuba

Dense, Conv, Pool, Flatten = make_blocks(cuba.Neuron)

__all__ = ['Dense', 'Conv', 'Pool', 'Flatten']
