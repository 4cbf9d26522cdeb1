"""Sigma-delta blocks (``src/lava/lib/dl/slayer/block/sigma_delta.py``): the
synapse + neuron blocks with the sigma-delta neuron (no inter-layer step delay
unless asked for, ``sigma_delta.py:24-29``) and the delta-encoding input block."""

import torch

from . import base
from ._family import make_blocks
from .. import synapse
from ..neuron import sigma_delta

Dense, Conv, Pool, Flatten = make_blocks(sigma_delta.Neuron, default_delay_shift=False)


class Input(torch.nn.Module):
    """Input block (``sigma_delta.py:45-73`` over ``base.py:42-137``): an optional
    affine transform of the input, quantised to the 8-bit weight grid, followed by
    the neuron's delta encoder.

    Parameters
    ----------
    neuron_params : dict or None
        sigma-delta neuron parameters; ``None`` passes the input through.
    weight, bias : float or None
        learnable scale and shift of the input.
    delay_shift, count_log : bool
        kept for signature compatibility (the reference's input block ignores them).
    """

    def __init__(self, neuron_params=None, weight=None, bias=None, delay_shift=False, count_log=False):
        super().__init__()
        self.neuron = None if neuron_params is None else sigma_delta.Neuron(**neuron_params)
        self.synapse_params = None
        self.count_log = count_log
        self.delay = None
        self.delay_shift = delay_shift
        for name, value in (('weight', weight), ('bias', bias)):
            if value is not None:
                self.register_parameter(name, torch.nn.Parameter(torch.FloatTensor([value]), requires_grad=True))
            else:
                setattr(self, name, None)
        self.input_shape = None
        self.pre_hook_fx = (lambda x: x) if self.neuron is None else self.neuron.quantize_8bit

    def forward(self, x):
        if self.neuron is not None:
            z = self.pre_hook_fx(x)
            if self.weight is not None:
                z = z * self.pre_hook_fx(self.weight)
            if self.bias is not None:
                z = z + self.pre_hook_fx(self.bias)
            x = self.neuron.delta(z)
            if self.input_shape is None:
                self.input_shape = self.neuron.delta.shape
                self.neuron.sigma.shape = self.neuron.delta.shape
                self.neuron.shape = self.neuron.delta.shape
        elif self.input_shape is None:
            self.input_shape = x.shape[1:-1]
        return x

    @property
    def shape(self):
        return self.input_shape


class Average(base.AbstractAverage):
    __doc__ = base.AbstractAverage.__doc__


class Output(torch.nn.Module):
    """Output block (``sigma_delta.py:168-220``): a dense synapse on the neuron's weight grid
    followed by the neuron's sigma decoder, so that the network returns the accumulated signal
    instead of its changes.

    Parameters
    ----------
    neuron_params : dict
    in_neurons, out_neurons : int
    weight_scale : int
    weight_norm, count_log : bool
    """

    def __init__(self, neuron_params, in_neurons, out_neurons, weight_scale=1, weight_norm=False, count_log=False):
        super().__init__()
        self.neuron = sigma_delta.Neuron(**neuron_params)
        self.delay = None
        self.synapse = synapse.Dense(in_neurons, out_neurons, weight_scale=weight_scale, weight_norm=weight_norm,
                                     pre_hook_fx=self.neuron.quantize_8bit)
        self.count_log = count_log

    def forward(self, x):
        x = self.neuron.sigma(self.synapse(x))
        if self.count_log is True:
            return x, torch.mean((x > 0).to(x.dtype))
        return x

    @property
    def shape(self):
        return self.neuron.sigma.shape


__all__ = ['Input', 'Dense', 'Conv', 'Pool', 'Flatten', 'Average', 'Output']
