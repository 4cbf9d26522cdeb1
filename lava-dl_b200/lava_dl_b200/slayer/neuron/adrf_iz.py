"""Adaptive resonate-and-fire neuron, Izhikevich style
(``src/lava/lib/dl/slayer/neuron/adrf_iz.py:132-672``): the adaptive resonator
dynamics (spike condition ``imag >= threshold + refractory``, no state reset)
with a plain threshold spike on the imaginary part.

The reference's ``forward`` calls ``self.spike(real, imag, threshold +
refractory)`` with three arguments although ``spike`` takes four
(``adrf_iz.py:669-670``) and raises ``TypeError``; here ``forward`` passes the
two series separately, which is what ``spike`` is written for."""

import torch

from .adrf import neuron_params  # noqa: F401  (same device-parameter translation)
from .rf import ResonatorBase
from .dynamics import adaptive_resonator
from ..spike.spike import Spike
from ..utils import quantize

SCALE_RHO_MULT = 0.1
TAU_RHO_MULT = 100


class Neuron(ResonatorBase):
    """Adaptive RF Izhikevich neuron; parameters as for ``adrf.Neuron``."""

    def __init__(self, threshold, threshold_step, period, decay, threshold_decay, refractory_decay, tau_grad=1,
                 scale_grad=1, scale=1 << 6, norm=None, dropout=None, shared_param=True, persistent_state=False,
                 requires_grad=False, graded_spike=False, log_init=True):
        super().__init__(
            threshold=threshold, tau_grad=tau_grad, scale_grad=scale_grad, p_scale=1 << 12, w_scale=scale,
            s_scale=scale * (1 << 6), norm=norm, dropout=dropout, persistent_state=persistent_state,
            shared_param=shared_param, requires_grad=requires_grad, complex=True)
        self.threshold_step = int(threshold_step * self.w_scale) / self.w_scale
        self.graded_spike = graded_spike
        self.log_init = log_init
        self._init_rotation(period, decay)
        if self.shared_param:
            self._add_decay('threshold_decay', self.p_scale * threshold_decay)
            self._add_decay('refractory_decay', self.p_scale * refractory_decay)
        else:
            self.threshold_decay_min, self.threshold_decay_max = self._range(
                threshold_decay, 'threshold decay', 0.0)
            self.refractory_decay_min, self.refractory_decay_max = self._range(
                refractory_decay, 'refractory decay', 0.0)
            self._add_decay('threshold_decay', self.p_scale * self.threshold_decay_min)
            self._add_decay('refractory_decay', self.p_scale * self.refractory_decay_min)
        for name, value in (('real_state', 0.), ('imag_state', 0.), ('threshold_state', self.threshold),
                            ('refractory_state', 0.)):
            self.register_buffer(name, torch.tensor([value], dtype=torch.float), persistent=False)
        self.clamp()

    @property
    def cx_threshold_decay(self):
        return self._cx(self.threshold_decay)

    @property
    def cx_refractory_decay(self):
        return self._cx(self.refractory_decay)

    @property
    def v_th_step(self):
        return int(self.threshold_step * self.w_scale)

    @property
    def device_params(self):
        return {
            'type': 'ADRF_IZHIKEVICH',
            'sinDecay': self.cx_sin_decay,
            'cosDecay': self.cx_cos_decay,
            'thDecay': self.cx_threshold_decay,
            'refDecay': self.cx_refractory_decay,
            'vThMant': self.v_th_mant,
            'vThStep': self.v_th_step,
            'gradedSpike': self.graded_spike,
        }

    def dynamics(self, input):
        """Returns ``real, imag, threshold, refractory`` series."""
        real_input, imag_input = self._check_pair(input)
        if self._bind_shape(real_input) and not self.shared_param:
            self._sample_rotation()
            self.threshold_decay.data = self.p_scale * self._uniform(
                self.threshold_decay_min, self.threshold_decay_max)
            self.refractory_decay.data = self.p_scale * self._uniform(
                self.refractory_decay_min, self.refractory_decay_max)
            del self.threshold_decay_min, self.threshold_decay_max
            del self.refractory_decay_min, self.refractory_decay_max
        self._sync_states(real_input, {'real_state': 0, 'imag_state': 0, 'threshold_state': self.threshold,
                                       'refractory_state': 0})
        if self.requires_grad:
            self.clamp()
        real_input, imag_input = self._normalise(real_input, imag_input)
        real, imag, threshold, refractory = adaptive_resonator.dynamics(
            real_input, imag_input, quantize(self.sin_decay), quantize(self.cos_decay),
            quantize(self.refractory_decay), quantize(self.threshold_decay), self.real_state, self.imag_state,
            self.refractory_state, self.threshold_state, self.threshold_step, self.threshold, self.s_scale,
            debug=self.debug)
        if self.persistent_state:
            with torch.no_grad():
                self.real_state = real[..., -1].clone()
                self.imag_state = imag[..., -1].clone()
                self.threshold_state = threshold[..., -1].clone()
                self.refractory_state = refractory[..., -1].clone()
        return real, imag, threshold, refractory

    def spike(self, real, imag, threshold, refractory):
        """Spikes where ``imag >= threshold + refractory``."""
        _ = real.shape
        spike = Spike.apply(
            imag, threshold + refractory, self.tau_rho * TAU_RHO_MULT, self.scale_rho * SCALE_RHO_MULT,
            self.graded_spike, self.imag_state, 1)
        if self.persistent_state:
            with torch.no_grad():
                self.refractory_state = adaptive_resonator.persistent_ref_state(
                    self.refractory_state, spike[..., -1], self.threshold_state).detach().clone()
                self.threshold_state = adaptive_resonator.persistent_th_state(
                    self.threshold_state, spike[..., -1], self.threshold_step).detach().clone()
        if self.drop is not None:
            spike = self.drop(spike)
        return spike

    def forward(self, input):
        """Spike response to the complex input tuple ``(real_input, imag_input)``."""
        real, imag, threshold, refractory = self.dynamics(input)
        return self.spike(real, imag, threshold, refractory)
