"""Adaptive-LIF blocks (``src/lava/lib/dl/slayer/block/alif.py``); 8-bit quantisation ready."""

from ._family import make_blocks
from ..neuron import alif

Dense, Conv, Pool, Flatten = make_blocks(alif.Neuron)

__all__ = ['Dense', 'Conv', 'Pool', 'Flatten']
