"""Builds the concrete blocks of one neuron family (``block/cuba.py:11-158`` and
its siblings are the same code with a different neuron class)."""

from . import base
from .. import synapse
from ..axon import Delay


def make_blocks(neuron_class, default_delay_shift=True):
    class _Family:
        """Creates the neuron, the optional learnable delay, and hooks the neuron's
        8-bit quantiser into the synapse unless the caller named a pre-hook."""

        def _attach(self, synapse_class, kwargs):
            self.neuron = neuron_class(**self.neuron_params)
            self.delay = Delay(max_delay=62) if kwargs.get('delay', False) is True else None
            self.synapse = synapse_class(**self.synapse_params)
            if 'pre_hook_fx' not in kwargs:
                self.synapse.pre_hook_fx = self.neuron.quantize_8bit
            if 'delay_shift' not in kwargs:
                self.delay_shift = default_delay_shift
            del self.neuron_params, self.synapse_params

    class Dense(_Family, base.AbstractDense):
        __doc__ = base.AbstractDense.__doc__

        def __init__(self, *args, **kwargs):
            super().__init__(*args, **kwargs)
            self._attach(synapse.Dense, kwargs)

    class Conv(_Family, base.AbstractConv):
        __doc__ = base.AbstractConv.__doc__

        def __init__(self, *args, **kwargs):
            super().__init__(*args, **kwargs)
            self._attach(synapse.Conv, kwargs)

    class Pool(_Family, base.AbstractPool):
        __doc__ = base.AbstractPool.__doc__

        def __init__(self, *args, **kwargs):
            super().__init__(*args, **kwargs)
            self._attach(synapse.Pool, kwargs)

    class Flatten(base.AbstractFlatten):
        __doc__ = base.AbstractFlatten.__doc__

    return Dense, Conv, Pool, Flatten
