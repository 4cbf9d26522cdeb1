"""CUBA-LIF blocks (``src/lava/lib/dl/slayer/block/cuba.py``); 8-bit quantisation ready.
The recurrent and winner-takes-all blocks run their walk over time as one kernel launch per
direction for up to 1024 neurons (``utils.recurrent``)."""

from ._family import make_family
from ..neuron import cuba

_blocks = make_family(cuba.Neuron)
Input, Flatten, Average = _blocks['Input'], _blocks['Flatten'], _blocks['Average']
Dense, Conv, Pool = _blocks['Dense'], _blocks['Conv'], _blocks['Pool']
KWTA, Recurrent = _blocks['KWTA'], _blocks['Recurrent']

__all__ = ['Input', 'Flatten', 'Average', 'Dense', 'Conv', 'Pool', 'KWTA', 'Recurrent']
