"""Resonate-and-fire blocks (``src/lava/lib/dl/slayer/block/rf.py``). The synapses are complex
(a real and an imaginary one, ``synapse.complex``).  As in the reference, the recurrent and
winner-takes-all blocks of a complex family fail on their first call: the walk over time treats
the synapse output as one tensor."""

from ._family import make_family
from .. import synapse
from ..neuron import rf

_blocks = make_family(rf.Neuron, synapse=synapse.complex)
Input, Flatten, Average = _blocks['Input'], _blocks['Flatten'], _blocks['Average']
Dense, Conv, Pool = _blocks['Dense'], _blocks['Conv'], _blocks['Pool']
KWTA, Recurrent = _blocks['KWTA'], _blocks['Recurrent']

__all__ = ['Input', 'Flatten', 'Average', 'Dense', 'Conv', 'Pool', 'KWTA', 'Recurrent']
