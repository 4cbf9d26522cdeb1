"""Builds the concrete blocks of one neuron family (``block/cuba.py:11-177`` and its siblings
are the same code with a different neuron class and, for the resonators, the complex synapses)."""

from . import base
from .. import synapse as real_synapse
from ..axon import Delay


def make_blocks(neuron_class, default_delay_shift=True, synapse=real_synapse):
    """Returns ``(Dense, Conv, Pool, Flatten)``; ``make_family`` returns every block."""
    fam = make_family(neuron_class, default_delay_shift, synapse)
    return fam['Dense'], fam['Conv'], fam['Pool'], fam['Flatten']


def make_family(neuron_class, default_delay_shift=True, synapse=real_synapse):
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

    class Input(base.AbstractInput):
        __doc__ = base.AbstractInput.__doc__

        def __init__(self, *args, **kwargs):
            super().__init__(*args, **kwargs)
            if self.neuron_params is not None:
                self.neuron = neuron_class(**self.neuron_params)
                self.pre_hook_fx = self.neuron.quantize_8bit
            del self.neuron_params

    class Flatten(base.AbstractFlatten):
        __doc__ = base.AbstractFlatten.__doc__

    class Average(base.AbstractAverage):
        __doc__ = base.AbstractAverage.__doc__

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

    class KWTA(base.AbstractKWTA):
        __doc__ = base.AbstractKWTA.__doc__

        def __init__(self, *args, **kwargs):
            super().__init__(*args, **kwargs)
            self.neuron = neuron_class(**self.neuron_params)
            self.synapse = synapse.Dense(**self.synapse_params)
            if 'pre_hook_fx' not in kwargs:
                self.synapse.pre_hook_fx = self.neuron.quantize_8bit
            del self.neuron_params, self.synapse_params

    class Recurrent(base.AbstractRecurrent):
        __doc__ = base.AbstractRecurrent.__doc__

        def __init__(self, *args, **kwargs):
            super().__init__(*args, **kwargs)
            self.neuron = neuron_class(**self.neuron_params)
            delay = kwargs.get('delay', args[6] if len(args) > 6 else False)
            self.delay = Delay(max_delay=62) if delay is True else None
            self.input_synapse = synapse.Dense(**self.synapse_params)
            self.recurrent_synapse = synapse.Dense(**self.recurrent_params)
            self.input_synapse.pre_hook_fx = self.neuron.quantize_8bit
            self.recurrent_synapse.pre_hook_fx = self.neuron.quantize_8bit
            del self.neuron_params, self.synapse_params, self.recurrent_params

    return dict(Input=Input, Flatten=Flatten, Average=Average, Dense=Dense, Conv=Conv, Pool=Pool, KWTA=KWTA,
                Recurrent=Recurrent)
