"""Adaptive-LIF blocks (``src/lava/lib/dl/slayer/block/alif.py``); 8-bit quantisation ready."""

from ._family import make_family
from ..neuron import alif

_blocks = make_family(alif.Neuron)
Input, Flatten, Average = _blocks['Input'], _blocks['Flatten'], _blocks['Average']
Dense, Conv, Pool = _blocks['Dense'], _blocks['Conv'], _blocks['Pool']
KWTA, Recurrent = _blocks['KWTA'], _blocks['Recurrent']

__all__ = ['Input', 'Flatten', 'Average', 'Dense', 'Conv', 'Pool', 'KWTA', 'Recurrent']
