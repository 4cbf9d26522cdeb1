"""Adaptive resonate-and-fire neuron
(``src/lava/lib/dl/slayer/neuron/adrf.py:132-677``)."""

import numpy as np
import torch

from .rf import ResonatorBase, _FusedForward
from .dynamics import resonator, adaptive_phase_th
from ..spike import complex
from ..utils import quantize
from ... import _ops

SCALE_RHO_MULT = 0.1
TAU_RHO_MULT = 100


def neuron_params(device_params, scale=1 << 6, p_scale=1 << 12):
    """Translate Loihi device parameters to constructor arguments."""
    sin_decay = device_params['sinDecay'] / p_scale
    cos_decay = device_params['cosDecay'] / p_scale
    decay = 1 - np.sqrt(sin_decay ** 2 + cos_decay ** 2)
    frequency = np.arctan2(sin_decay, cos_decay) / 2 / np.pi
    return {
        'threshold': device_params['vThMant'] / scale,
        'threshold_step': device_params['vThMant'] / scale,
        'period': 1 / frequency,
        'decay': decay,
        'threshold_decay': device_params['thDecay'] / p_scale,
        'refractory_decay': device_params['refDecay'] / p_scale,
    }


class _FusedDynamics(torch.autograd.Function):
    """real, imag, threshold, refractory in one pass; backward is the
    resonator's reverse rotation scan."""

    @staticmethod
    def forward(ctx, real_input, imag_input, sin_decay, cos_decay, ref_decay, th_decay, real_state, imag_state,
                ref_state, th_state, th_step, th0, w_scale):
        ad = dict(ref_decay=ref_decay, th_decay=th_decay, ref_state=ref_state, th_state=th_state,
                  th_step=th_step, th0=th0)
        (real, imag, threshold, refractory), _ = _ops.rf_fwd(
            real_input, imag_input, sin_decay, cos_decay, real_state, imag_state, 0.0, w_scale, adaptive=ad,
            dynamics_mode=True)
        ctx.save_for_backward(real, imag, sin_decay, cos_decay)
        ctx.mark_non_differentiable(threshold, refractory)
        return real, imag, threshold, refractory

    @staticmethod
    def backward(ctx, grad_real, grad_imag, *_):
        real, imag, sin_decay, cos_decay = ctx.saved_tensors
        need = ctx.needs_input_grad[2] or ctx.needs_input_grad[3]
        gre, gim, gsin, gcos = _ops.res_bwd(grad_real, grad_imag, real, imag, sin_decay, cos_decay, need)
        resonator._raise_on_nan(grad_sin_decay=gsin, grad_cos_decay=gcos)
        return (gre, gim, gsin, gcos) + (None,) * 9


class Neuron(ResonatorBase):
    """Adaptive resonate-and-fire neuron: resonator state, adaptive threshold and
    refractory trace; a spike is emitted where ``real >= threshold +
    refractory`` while the imaginary part crosses zero upwards.

    Parameters
    ----------
    threshold, threshold_step : float
    period, decay : float or (min, max)
    threshold_decay, refractory_decay : float or (min, max)
    tau_grad, scale_grad, scale, norm, dropout, shared_param, persistent_state,
    requires_grad, graded_spike, log_init : as for the RF neuron.
    """

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
            'type': 'ADRF_PHASE',
            'sinDecay': self.cx_sin_decay,
            'cosDecay': self.cx_cos_decay,
            'thDecay': self.cx_threshold_decay,
            'refDecay': self.cx_refractory_decay,
            'vThMant': self.v_th_mant,
            'vThStep': self.v_th_step,
            'gradedSpike': self.graded_spike,
        }

    # ------------------------------------------------------------------
    def _prepare(self, input):
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
        return self._normalise(real_input, imag_input)

    def dynamics(self, input):
        """Returns ``real, imag, threshold, refractory`` series."""
        real_input, imag_input = self._prepare(input)
        sd, cd = quantize(self.sin_decay), quantize(self.cos_decay)
        rd, td = quantize(self.refractory_decay), quantize(self.threshold_decay)
        if self._fusable:
            real, imag, threshold, refractory = _FusedDynamics.apply(
                real_input, imag_input, sd, cd, rd, td, self.real_state, self.imag_state, self.refractory_state,
                self.threshold_state, self.threshold_step, self.threshold, self.s_scale)
        else:
            real, imag = resonator.dynamics(real_input, imag_input, sd, cd, self.real_state, self.imag_state,
                                            self.s_scale, debug=self.debug)
            threshold, refractory = adaptive_phase_th.dynamics(
                real, imag, self.imag_state, self.refractory_state, rd, self.threshold_state, td,
                self.threshold_step, self.threshold, self.s_scale, debug=self.debug)
        if self.persistent_state:
            with torch.no_grad():
                self.real_state = real[..., -1].clone()
                self.threshold_state = threshold[..., -1].clone()
                self.refractory_state = refractory[..., -1].clone()
        return real, imag, threshold, refractory

    def _carry_spike(self, last_spike):
        self.refractory_state = adaptive_phase_th.persistent_ref_state(
            self.refractory_state, last_spike, self.threshold_state).detach().clone()
        self.threshold_state = adaptive_phase_th.persistent_th_state(
            self.threshold_state, last_spike, self.threshold_step).detach().clone()

    def spike(self, real, imag, threshold, refractory):
        """Spikes from the four state series."""
        spike = complex.Spike.apply(
            real, imag, threshold + refractory, self.tau_rho * TAU_RHO_MULT, self.scale_rho * SCALE_RHO_MULT,
            self.graded_spike, self.imag_state, 1)
        if self.persistent_state:
            with torch.no_grad():
                self.imag_state = imag[..., -1].clone()
                self._carry_spike(spike[..., -1])
        if self.drop is not None:
            spike = self.drop(spike)
        return spike

    def forward(self, input):
        """Spike response to the complex input tuple ``(real_input, imag_input)``."""
        if not self._fusable:
            real, imag, threshold, refractory = self.dynamics(input)
            return self.spike(real, imag, threshold, refractory)
        spike, _ = self._fused_forward(input, 0, None)
        if self.drop is not None:
            spike = self.drop(spike)
        return spike

    @property
    def fuses_step_delay(self):
        """True when ``forward_step_delayed`` can write the spikes one step late inside the kernel."""
        return self._fusable and self.graded_spike is not True and self.drop is None

    fuses_axon_delay = False   # a block's axonal delay stays a separate shift for this neuron

    def forward_step_delayed(self, input, delay_head=None):
        """``forward`` with the blocks' one-step delay folded in: ``(delayed_spike, last_spike)``."""
        return self._fused_forward(input, 1, delay_head)

    def _fused_forward(self, input, spike_delay, delay_head):
        real_input, imag_input = self._prepare(input)
        spike, final_re, final_im, final_s, final_th, final_ref = _FusedForward.apply(
            real_input, imag_input, quantize(self.sin_decay), quantize(self.cos_decay), self.real_state,
            self.imag_state, self.threshold, self.s_scale, self.tau_rho * TAU_RHO_MULT,
            self.scale_rho * SCALE_RHO_MULT, self.graded_spike is True, quantize(self.refractory_decay),
            quantize(self.threshold_decay), self.refractory_state, self.threshold_state, self.threshold_step,
            self.threshold, spike_delay, delay_head)
        if self.persistent_state:
            with torch.no_grad():
                self.real_state = final_re
                self.imag_state = final_im
                self.threshold_state = final_th
                self.refractory_state = final_ref
                self._carry_spike(final_s)
        return spike, final_s
