"""Block scaffolding (``src/lava/lib/dl/slayer/block/base.py``): a block is
``synapse -> neuron -> one-step delay -> optional learnable axonal delay``,
optionally returning the mean event rate of its output."""

import numpy as np
import torch

from ..axon import delay


def step_delay(module, x):
    """One time step of inter-layer communication delay (``block/base.py:15-39``).
    With a persistent-state neuron the spike that falls off the end is kept and
    re-enters at t = 0 of the next call."""
    if not hasattr(module, 'delay_buffer'):
        module.delay_buffer = None
    persistent_state = hasattr(module, 'neuron') and module.neuron.persistent_state is True
    if module.delay_buffer is not None and module.delay_buffer.shape[0] != x.shape[0]:
        module.delay_buffer = None  # batch size changed
    if persistent_state:
        delay_buffer = 0 if module.delay_buffer is None else module.delay_buffer
        module.delay_buffer = x[..., -1]
    x = delay(x, 1)
    if persistent_state:
        x[..., 0] = delay_buffer
    return x


class _Block(torch.nn.Module):
    """Common forward of every synapse + neuron block."""

    def _init_block(self, neuron_params, synapse_params, delay_shift, count_log):
        self.neuron_params = neuron_params
        self.synapse_params = synapse_params
        self.count_log = count_log
        self.neuron = None
        self.synapse = None
        self.delay = None
        self.delay_shift = delay_shift

    def forward(self, x):
        """``NCT`` or ``NCHWT`` input -> spikes (and event rate when ``count_log``)."""
        mask = getattr(self, 'mask', None)
        if mask is not None:
            if self.synapse.complex is True:
                self.synapse.real.weight.data *= mask
                self.synapse.imag.weight.data *= mask
            else:
                self.synapse.weight.data *= mask
        z = self.synapse(x)
        if self.delay_shift is True and getattr(self.neuron, 'fuses_step_delay', False):
            # a bounded axonal delay (at most 62 steps) is written by the neuron kernel as well
            steps = None if self.delay is None else self.delay.fusable_steps
            fuse_axon = steps is not None and 0 <= steps <= 62 and getattr(self.neuron, 'fuses_axon_delay', False)
            x = self._neuron_with_step_delay(z, self.delay if fuse_axon else None)
            if self.delay is not None and not fuse_axon:
                x = self.delay(x)
        else:
            x = self.neuron(z)
            if self.delay_shift is True:
                x = step_delay(self, x)
            if self.delay is not None:
                x = self.delay(x)
        if self.count_log is True:
            return x, torch.mean((x > 0).to(x.dtype))
        return x

    def _neuron_with_step_delay(self, z, axon=None):
        """``step_delay(self, self.neuron(z))`` in one kernel: the neuron writes its
        spikes one step late; the spike carried over between calls of a
        persistent-state neuron enters at t = 0.  With ``axon`` (an ``axon.Delay``)
        the same kernel also applies the per-channel axonal delay."""
        if not hasattr(self, 'delay_buffer'):
            self.delay_buffer = None
        persistent_state = self.neuron.persistent_state is True
        if self.delay_buffer is not None and self.delay_buffer.shape[0] != z.shape[0]:
            self.delay_buffer = None
        head = self.delay_buffer if persistent_state else None
        if axon is None:
            x, last_spike = self.neuron.forward_step_delayed(z, head)
        else:
            x, last_spike = self.neuron.forward_step_delayed(z, head, axon.delay_per_neuron(z), axon.sampling_time,
                                                             axon.grad_scale)
        if persistent_state:
            self.delay_buffer = last_spike
        return x

    @property
    def shape(self):
        return self.neuron.shape


class AbstractInput(torch.nn.Module):
    """Input block (``block/base.py:42-137``): an optional learnable affine transform of the input,
    both factors passed through the neuron's weight quantiser, then the neuron and the one-step delay.

    Parameters
    ----------
    neuron_params : dict or None
        ``None`` passes the input through (only the delay applies).
    weight, bias : float or None
    delay_shift, count_log : bool
    """

    def __init__(self, neuron_params=None, weight=None, bias=None, delay_shift=True, count_log=False):
        super().__init__()
        self.neuron_params = neuron_params
        self.synapse_params = None
        self.count_log = count_log
        self.neuron = None
        self.delay = None
        for name, value in (('weight', weight), ('bias', bias)):
            if value is not None:
                self.register_parameter(name, torch.nn.Parameter(torch.FloatTensor([value]), requires_grad=True))
            else:
                setattr(self, name, None)
        self.input_shape = None
        self.pre_hook_fx = lambda x: x
        self.delay_shift = delay_shift

    def forward(self, x):
        if self.neuron is not None:
            z = self.pre_hook_fx(x)
            if self.weight is not None:
                z = z * self.pre_hook_fx(self.weight)
            if self.bias is not None:
                z = z + self.pre_hook_fx(self.bias)
            x = self.neuron(z)
        if self.delay_shift is True:
            x = step_delay(self, x)
        if self.input_shape is None:
            self.input_shape = self.neuron.shape if self.neuron is not None else x.shape[1:-1]
        if self.count_log is True:
            return x, torch.mean((x > 0).to(x.dtype))
        return x

    @property
    def shape(self):
        return self.neuron.shape if self.neuron is not None else self.input_shape


class AbstractAverage(torch.nn.Module):
    """Population average (``block/base.py:210-259``): the mean over groups of
    ``neurons / num_outputs`` consecutive neurons, per time step."""

    def __init__(self, num_outputs, count_log=False):
        super().__init__()
        self.count_log = count_log
        self.num_outputs = num_outputs

    def forward(self, x):
        N, T = x.shape[0], x.shape[-1]
        mean = torch.mean(x.reshape((N, self.num_outputs, -1, T)), dim=2)
        return (mean, None) if self.count_log is True else mean

    @property
    def shape(self):
        return torch.Size([self.num_outputs, 1, 1])


class AbstractDense(_Block):
    """Dense block; see ``synapse.Dense`` for the synapse arguments.

    Parameters
    ----------
    neuron_params : dict
    in_neurons, out_neurons : int
    weight_scale, weight_norm, pre_hook_fx : synapse options
    delay : bool
        add a learnable axonal delay.
    delay_shift : bool
        apply the one-step inter-layer delay.
    mask : bool tensor or None
        synapse mask.
    count_log : bool
    """

    def __init__(self, neuron_params, in_neurons, out_neurons, weight_scale=1, weight_norm=False,
                 pre_hook_fx=None, delay=False, delay_shift=True, mask=None, count_log=False):
        super().__init__()
        self._init_block(neuron_params, dict(in_neurons=in_neurons, out_neurons=out_neurons,
                                             weight_scale=weight_scale, weight_norm=weight_norm,
                                             pre_hook_fx=pre_hook_fx), delay_shift, count_log)
        if mask is None:
            self.mask = None
        else:
            self.register_buffer('mask', mask.reshape(mask.shape[0], mask.shape[1], 1, 1, 1))


class AbstractConv(_Block):
    """Convolution block; see ``synapse.Conv`` for the synapse arguments."""

    def __init__(self, neuron_params, in_features, out_features, kernel_size, stride=1, padding=0, dilation=1,
                 groups=1, weight_scale=1, weight_norm=False, pre_hook_fx=None, delay=False, delay_shift=True,
                 count_log=False):
        super().__init__()
        self._init_block(neuron_params, dict(in_features=in_features, out_features=out_features,
                                             kernel_size=kernel_size, stride=stride, padding=padding,
                                             dilation=dilation, groups=groups, weight_scale=weight_scale,
                                             weight_norm=weight_norm, pre_hook_fx=pre_hook_fx), delay_shift,
                         count_log)


class AbstractPool(_Block):
    """Sum-pooling block; see ``synapse.Pool`` for the synapse arguments."""

    def __init__(self, neuron_params, kernel_size, stride=None, padding=0, dilation=1, weight_scale=1,
                 weight_norm=False, pre_hook_fx=None, delay=False, delay_shift=True, count_log=False):
        super().__init__()
        if 'norm' in neuron_params.keys():
            neuron_params['norm'] = None
        self._init_block(neuron_params, dict(kernel_size=kernel_size, stride=stride, padding=padding,
                                             dilation=dilation, weight_scale=weight_scale, weight_norm=weight_norm,
                                             pre_hook_fx=pre_hook_fx), delay_shift, count_log)


class AbstractFlatten(torch.nn.Module):
    """Flattens the spatial dimensions: ``NCHWT -> N(CHW)T``."""

    def __init__(self, count_log=False):
        super().__init__()
        self.count_log = count_log
        self.shape = None

    def forward(self, x):
        if self.shape is None:
            self.shape = [int(np.prod(x.shape[1:-1])), 1, 1]
        flat = x.reshape((x.shape[0], -1, x.shape[-1]))
        return (flat, None) if self.count_log is True else flat


class AbstractRecurrent(torch.nn.Module):
    """Dense recurrent block (``block/base.py:1367-1488`` of the reference):
    ``s[t] = neuron(W x[t] + R s[t-1])``, then the one-step delay and the optional
    axonal delay.  The neuron always keeps its state between calls.

    Parameters
    ----------
    neuron_params : dict
    in_neurons, out_neurons : int
    weight_scale, weight_norm, pre_hook_fx : options of both synapses
    delay : bool
        add a learnable axonal delay.
    delay_shift : bool
        apply the one-step inter-layer delay.
    requires_grad : bool
        kept for signature compatibility.
    count_log : bool
    """

    def __init__(self, neuron_params, in_neurons, out_neurons, weight_scale=1, weight_norm=False,
                 pre_hook_fx=None, delay=False, delay_shift=True, requires_grad=True, count_log=False):
        super().__init__()
        self.neuron_params = dict(neuron_params, persistent_state=True)
        self.synapse_params = dict(in_neurons=in_neurons, out_neurons=out_neurons, weight_scale=weight_scale,
                                   weight_norm=weight_norm, pre_hook_fx=pre_hook_fx)
        self.recurrent_params = dict(self.synapse_params, in_neurons=out_neurons)
        self.num_neurons = out_neurons
        self.requires_grad = requires_grad
        self.count_log = count_log
        self.neuron = None
        self.input_synapse = None
        self.recurrent_synapse = None
        self.delay = None
        self.bias = None
        self.persistent_state = True
        self.delay_shift = delay_shift

    def forward(self, x):
        """``NCT`` input -> spikes (and event rate when ``count_log``)."""
        from ..utils import recurrent
        z = self.input_synapse(x)
        if self.bias is not None:
            z = z + self.bias
        # the spike fed back at t = 0 is always zero: the reference stores a zero tensor as its
        # spike state (block/base.py:1471-1478), only the neuron state survives between calls
        x = recurrent.custom_recurrent(z, self.neuron, self.recurrent_synapse)
        if self.delay_shift is True:
            x = delay(x, 1)
        if self.delay is not None:
            x = self.delay(x)
        if self.count_log is True:
            return x, torch.mean((x > 0).to(x.dtype))
        return x

    @property
    def shape(self):
        return self.neuron.shape



class AbstractKWTA(torch.nn.Module):
    """K-winner-takes-all block (``block/base.py:1222-1364``):
    ``s[t] = neuron(W x[t] + R s[t-1] + alpha (N - 2K))`` with the fixed lateral matrix
    ``R = (1 + a) I - 1`` (self excitation ``a``, everybody else inhibits) on the weight grid of
    the neuron.  The walk over time is the recurrent one (``utils.recurrent``).

    Parameters
    ----------
    neuron_params : dict
    in_neurons, out_neurons, num_winners : int
    self_excitation : float
    weight_scale, weight_norm, pre_hook_fx : synapse options
    delay_shift : bool
    requires_grad : bool
        learnable self excitation.
    count_log : bool
    """

    def __init__(self, neuron_params, in_neurons, out_neurons, num_winners, self_excitation=0.5, weight_scale=1,
                 weight_norm=False, pre_hook_fx=None, delay_shift=True, requires_grad=True, count_log=False):
        super().__init__()
        self.neuron_params = dict(neuron_params, persistent_state=True)
        self.synapse_params = dict(in_neurons=in_neurons, out_neurons=out_neurons, weight_scale=weight_scale,
                                   weight_norm=weight_norm, pre_hook_fx=pre_hook_fx)
        self.num_neurons = out_neurons
        self.num_winners = num_winners
        self.requires_grad = requires_grad
        self.register_parameter('self_excitation', torch.nn.Parameter(torch.FloatTensor([self_excitation]),
                                                                      requires_grad=requires_grad))
        self.count_log = count_log
        self.neuron = None
        self.synapse = None
        self.delay = None
        self.bias = None
        self.register_buffer('spike_state', torch.zeros(1, dtype=torch.float))
        self.persistent_state = True
        self.delay_shift = delay_shift

    def clamp(self):
        self.self_excitation.data.clamp_(0, 1)

    def forward(self, x):
        """``NCT`` input -> spikes (and event rate when ``count_log``)."""
        from ..utils import recurrent
        z = self.synapse(x)
        if self.bias is not None:
            z = z + self.bias
        if isinstance(z, (tuple, list)):
            # the reference allocates zeros_like(z) for its output (block/base.py:1323): a complex
            # synapse's (real, imaginary) pair fails there in the same way
            raise TypeError('zeros_like(): argument \'input\' (position 1) must be Tensor, not tuple')
        self.clamp()
        recurrent_weight = (1 + self.self_excitation) * torch.eye(self.num_neurons, device=z.device) - 1
        recurrent_bias = self.neuron.threshold * (self.num_neurons - 2 * self.num_winners) \
            / self.num_neurons / self.neuron.w_scale
        recurrent_bias = torch.FloatTensor([recurrent_bias]).to(z.device)
        if self.neuron.quantize_8bit is not None:
            recurrent_weight = self.neuron.quantize_8bit(recurrent_weight)
            recurrent_bias = self.neuron.quantize_8bit(recurrent_bias)
        # the spike fed back at t = 0 is zero: the reference never stores a spike state
        # (block/base.py:1352), only the neuron state survives between calls
        x = recurrent.recurrent_walk(z + recurrent_bias, self.neuron, recurrent_weight)
        if self.delay_shift is True:
            x = step_delay(self, x)
        if self.count_log is True:
            return x, torch.mean((x > 0).to(x.dtype))
        return x

    @property
    def shape(self):
        return self.neuron.shape
