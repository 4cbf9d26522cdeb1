"""Common neuron scaffolding (``src/lava/lib/dl/slayer/neuron/base.py:107-217``)
plus the shape / state / parameter-range bookkeeping the four neuron models
share (``cuba.py:292-348``, ``alif.py:433-497``, ``rf.py:379-427``,
``adrf.py:472-571``)."""

import numpy as np
import torch

from ..utils import quantize


class Neuron(torch.nn.Module):
    """Abstract neuron: threshold, gradient relaxation and the fixed-point scales.

    Parameters
    ----------
    threshold : float
        neuron threshold (quantised to ``1 / w_scale``).
    tau_grad, scale_grad : float
        relaxation and scale of the spike-function surrogate gradient.
    p_scale, w_scale, s_scale : int
        parameter, weight and state scales of the integer representation.
    norm : callable or None
        factory of a normalisation module applied to the dendrite output.
    dropout : callable or None
        dropout module applied to the spikes.
    persistent_state : bool
        keep the state between calls.
    shared_param : bool
        one parameter set for the whole group (else one per channel).
    requires_grad : bool
        learnable decays.
    complex : bool
        complex-valued neuron (two normalisers).
    """

    def __init__(self, threshold, tau_grad=1, scale_grad=1, p_scale=1, w_scale=1, s_scale=1, norm=None,
                 dropout=None, persistent_state=False, shared_param=True, requires_grad=True, complex=False):
        super().__init__()
        self.num_neurons = None
        self.shape = None
        self.p_scale = p_scale
        self.w_scale = int(w_scale)
        self.s_scale = int(s_scale)
        self._threshold = int(threshold * self.w_scale) / self.w_scale
        self.tau_rho = tau_grad * self._threshold
        self.scale_rho = scale_grad
        self.shared_param = shared_param
        self.persistent_state = persistent_state
        self.requires_grad = requires_grad
        self.debug = False
        if self.s_scale < self.w_scale:
            raise AssertionError(
                'State scale is expected to be greater than weight scale. Found following\n'
                f'state scale = {self.s_scale}\nweight scale = {self.w_scale}\n'
            )
        self.complex = complex
        if norm is not None:
            names = ('real_norm', 'imag_norm') if complex else ('norm',)
            for name in names:
                module = norm()
                if hasattr(module, 'pre_hook_fx'):
                    module.pre_hook_fx = self.quantize_8bit
                setattr(self, name, module)
        elif complex:
            self.norm = None
            self.real_norm = None
            self.imag_norm = None
        else:
            self.norm = None
        self.drop = dropout

    # -- reference-facing properties ---------------------------------------
    @property
    def threshold(self):
        return self._threshold

    def quantize_8bit(self, weight, descale=False):
        """Quantise synaptic weights to the 8-bit Loihi grid (step ``2 / w_scale``).
        Meant to be installed as ``synapse.pre_hook_fx``."""
        q = quantize(weight, step=2 / self.w_scale).clamp(-256 / self.w_scale, 254 / self.w_scale)
        return q * self.w_scale if descale else q

    @property
    def weight_exponent(self):
        return int(np.log2(self.s_scale // self.w_scale) - 6)

    @property
    def v_th_mant(self):
        return int(self.threshold * self.w_scale)

    @property
    def device(self):
        pass

    def clamp(self):
        pass

    # -- shared bookkeeping --------------------------------------------------
    @property
    def _fusable(self):
        """One-pass kernels assume a power-of-two state scale."""
        s = self.s_scale
        return s > 0 and (s & (s - 1)) == 0

    def _add_decay(self, name, value):
        self.register_parameter(
            name, torch.nn.Parameter(torch.FloatTensor([value]), requires_grad=self.requires_grad))

    @staticmethod
    def _range(value, what, jitter):
        """``[min, max]`` of a per-channel parameter: a scalar gets +-``jitter``."""
        if np.isscalar(value):
            return value * (1 - jitter), value * (1 + jitter)
        if len(value) != 2:
            raise AssertionError(f'Expected {what} to be of length 2 i.e. [min, max]. Found {what}={value}.')
        return value[0], value[1]

    @staticmethod
    def _need_scalar(value, what):
        if not np.isscalar(value):
            raise AssertionError(f'Expected {what} to be a scalar when shared_param is True. Found {what}={value}.')

    def _bind_shape(self, input):
        """Fix the neuron shape on first use; returns True exactly then."""
        if self.shape is None:
            self.shape = input.shape[1:-1]
            if len(self.shape) == 0:
                raise AssertionError(
                    f"Expected input to have at least 3 dimensions: [Batch, Spatial dims ..., Time]. "
                    f"It's shape is {input.shape}."
                )
            self.num_neurons = np.prod(self.shape)
            return True
        if input.shape[1:-1] != self.shape:
            raise AssertionError(
                f'Input tensor shape ({input.shape}) does not match with Neuron shape ({self.shape}).'
            )
        return False

    def _uniform(self, lo, hi):
        return lo + (hi - lo) * torch.rand(self.shape[0], dtype=torch.float).to(self.device)

    def _sync_states(self, input, defaults):
        """Bring the state buffers to ``input.shape[:-1]``: re-initialise when the
        batch size changed, broadcast when they are still 1-element."""
        first = next(iter(defaults))
        ref = getattr(self, first)
        dtype, device, lead = ref.dtype, ref.device, input.shape[:-1]
        if ref.shape[0] != input.shape[0]:
            for name, value in defaults.items():
                setattr(self, name, torch.full(lead, float(value), dtype=dtype, device=device))
        elif ref.shape[1:] != self.shape:
            for name in defaults:
                setattr(self, name, getattr(self, name) * torch.ones(lead, dtype=dtype, device=device))

    def _cx(self, param):
        self.clamp()
        val = quantize(param).cpu().data.numpy().astype(int)
        return val[0] if len(val) == 1 else val
