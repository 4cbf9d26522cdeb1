"""CUBA-LIF blocks (``src/lava/lib/dl/slayer/block/cuba.py``); 8-bit quantisation ready."""

from . import base
from ._family import make_blocks
from .. import synapse
from ..axon import Delay
from ..neuron import cuba

Dense, Conv, Pool, Flatten = make_blocks(cuba.Neuron)


class Recurrent(base.AbstractRecurrent):
    """Dense recurrent CUBA block (``block/cuba.py:166-174`` of the reference): both
    synapses carry the neuron's 8-bit quantiser."""
    __doc__ = (__doc__ or '') + (base.AbstractRecurrent.__doc__ or '')

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.neuron = cuba.Neuron(**self.neuron_params)
        delay = kwargs.get('delay', args[6] if len(args) > 6 else False)
        self.delay = Delay(max_delay=62) if delay is True else None
        self.input_synapse = synapse.Dense(**self.synapse_params)
        self.recurrent_synapse = synapse.Dense(**self.recurrent_params)
        self.input_synapse.pre_hook_fx = self.neuron.quantize_8bit
        self.recurrent_synapse.pre_hook_fx = self.neuron.quantize_8bit
        del self.synapse_params, self.recurrent_params


__all__ = ['Dense', 'Conv', 'Pool', 'Flatten', 'Recurrent']
