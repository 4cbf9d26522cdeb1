"""Resonate-and-fire neuron (``src/lava/lib/dl/slayer/neuron/rf.py:114-500``)."""

import numpy as np
import torch

from . import base
from .dynamics import resonator
from ..spike import complex
from ..utils import quantize
from ... import _ops

SCALE_RHO_MULT = 10
TAU_RHO_MULT = 0.5


def neuron_params(device_params, scale=1 << 6, p_scale=1 << 12):
    """Translate Loihi device parameters to constructor arguments."""
    sin_decay = device_params['sinDecay'] / p_scale
    cos_decay = device_params['cosDecay'] / p_scale
    decay = 1 - np.sqrt(sin_decay ** 2 + cos_decay ** 2)
    frequency = np.arctan2(sin_decay, cos_decay) / 2 / np.pi
    return {
        'threshold': device_params['vThMant'] / scale,
        'period': 1 / frequency,
        'decay': decay,
    }


class _FusedForward(torch.autograd.Function):
    """Resonator + phase-threshold spike in one pass each way.  The adaptive
    neuron additionally passes its threshold / refractory decays and states
    (``ref_decay`` is None for the plain RF neuron)."""

    @staticmethod
    def forward(ctx, real_input, imag_input, sin_decay, cos_decay, real_state, imag_state, threshold, w_scale,
                tau_rho, scale_rho, graded, ref_decay=None, th_decay=None, ref_state=None, th_state=None,
                th_step=0.0, th0=0.0, spike_delay=0, delay_head=None):
        ad = None
        if ref_decay is not None:
            ad = dict(ref_decay=ref_decay, th_decay=th_decay, ref_state=ref_state, th_state=th_state,
                      th_step=th_step, th0=th0)
        # the state series are what the backward pass reads: with nothing to differentiate
        # (inference) only the spikes are written
        lean = not graded and not any(ctx.needs_input_grad)
        # adaptive neuron, sin / cos not learnt: the backward pass reads re only through
        # re - (threshold + refractory), so that one series replaces two
        margin = ad is not None and not lean and not (ctx.needs_input_grad[2] or ctx.needs_input_grad[3])
        outs, fin = _ops.rf_fwd(real_input, imag_input, sin_decay, cos_decay, real_state, imag_state, threshold,
                                w_scale, graded=graded, spike_scale=1.0, adaptive=ad, spike_delay=spike_delay,
                                delay_head=delay_head, spikes_only=lean, margin=margin)
        spike, real, imag = outs[:3]
        if lean:
            ctx.threshold = threshold
        elif margin:
            ctx.save_for_backward(real, imag, sin_decay, cos_decay)
            ctx.threshold = 0.0
        elif ad is None:
            ctx.save_for_backward(real, imag, sin_decay, cos_decay)
            ctx.threshold = threshold
        else:
            ctx.save_for_backward(real, imag, sin_decay, cos_decay, outs[3])
            ctx.threshold = None
        ctx.consts = (tau_rho, scale_rho, graded, spike_delay)
        extras = [fin['final_re'], fin['final_im'], fin['final_s']]
        if ad is not None:
            extras += [fin['final_th'], fin['final_ref']]
        ctx.mark_non_differentiable(*extras)
        return (spike,) + tuple(extras)

    @staticmethod
    def backward(ctx, grad_spike, *_):
        real, imag, sin_decay, cos_decay = ctx.saved_tensors[:4]
        threshold = ctx.saved_tensors[4] if ctx.threshold is None else ctx.threshold
        tau_rho, scale_rho, graded, spike_delay = ctx.consts
        need = ctx.needs_input_grad[2] or ctx.needs_input_grad[3]
        gre, gim, gsin, gcos = _ops.rf_bwd(grad_spike, real, imag, threshold, sin_decay, cos_decay, tau_rho,
                                           scale_rho, graded, need, spike_delay=spike_delay)
        resonator._raise_on_nan(grad_sin_decay=gsin, grad_cos_decay=gcos)
        return (gre, gim, gsin, gcos) + (None,) * 15


class ResonatorBase(base.Neuron):
    """Parameters and helpers common to the resonate-and-fire family: the
    rotation is stored as ``sin_decay = 4096 (1 - decay) sin(2 pi / period)``
    and ``cos_decay`` likewise."""

    def _init_rotation(self, period, decay):
        if self.shared_param:
            self._need_scalar(decay, 'decay')
            self._need_scalar(period, 'period')
            if period < 4:
                raise AssertionError(f'Neuron period less than 4 does not make sense. Found period={period}.')
            self._add_decay('sin_decay', self.p_scale * np.sin(2 * np.pi / period) * (1 - decay))
            self._add_decay('cos_decay', self.p_scale * np.cos(2 * np.pi / period) * (1 - decay))
        else:
            self.period_min, self.period_max = self._range(period, 'period', 0.01)
            if min(self.period_min, self.period_max) < 4 * (0.99 if np.isscalar(period) else 1):
                raise AssertionError(f'Neuron period less than 4 does not make sense. Found period={period}.')
            self.decay_min, self.decay_max = self._range(decay, 'decay', 0.01)
            self._add_decay('sin_decay', 0)
            self._add_decay('cos_decay', 0)

    def _sample_rotation(self):
        if self.log_init is False:
            frequency = self._uniform(1 / self.period_max, 1 / self.period_min)
        else:
            frequency = torch.logspace(
                -np.log10(self.period_max), -np.log10(self.period_min), steps=self.shape[0]).to(self.device)
        decay = self._uniform(self.decay_min, self.decay_max)
        self.sin_decay.data = self.p_scale * torch.sin(2 * np.pi * frequency) * (1 - decay)
        self.cos_decay.data = self.p_scale * torch.cos(2 * np.pi * frequency) * (1 - decay)
        del self.period_min, self.period_max, self.decay_min, self.decay_max

    def clamp(self):
        """Keep (sin, cos) inside the unit circle's first quadrant."""
        with torch.no_grad():
            gain = torch.sqrt(self.sin_decay ** 2 + self.cos_decay ** 2)
            clamped_gain = gain.clamp(0, self.p_scale - 1)
            self.sin_decay.data *= clamped_gain / gain
            self.cos_decay.data *= clamped_gain / gain
            self.sin_decay.data.clamp_(1)  # 0 would mean no oscillation
            self.cos_decay.data.clamp_(0)

    @property
    def decay(self):
        """Decay per step."""
        self.clamp()
        s = quantize(self.sin_decay).cpu().data.numpy() / self.p_scale
        c = quantize(self.cos_decay).cpu().data.numpy() / self.p_scale
        return 1 - np.sqrt(s ** 2 + c ** 2)

    @property
    def lam(self):
        return -np.log(1 - self.decay)

    @property
    def frequency(self):
        self.clamp()
        return np.arctan2(quantize(self.sin_decay).cpu().data.numpy(),
                          quantize(self.cos_decay).cpu().data.numpy()) / 2 / np.pi

    @property
    def period(self):
        return 1 / self.frequency

    @property
    def device(self):
        return self.sin_decay.device

    @property
    def cx_sin_decay(self):
        return self._cx(self.sin_decay)

    @property
    def cx_cos_decay(self):
        return self._cx(self.cos_decay)

    @property
    def scale(self):
        return self.w_scale

    def _check_pair(self, input):
        real_input, imag_input = input
        if real_input.shape != imag_input.shape:
            raise AssertionError(
                f'Real input tensor shape ({real_input.shape}) does not match with imaginary input shape '
                f'({imag_input.shape}).'
            )
        return real_input, imag_input

    def _normalise(self, real_input, imag_input):
        if self.real_norm is not None:
            real_input = self.real_norm(real_input)
        if self.imag_norm is not None:
            imag_input = self.imag_norm(imag_input)
        return real_input, imag_input


class Neuron(ResonatorBase):
    """Resonate-and-fire neuron with phase threshold.

    .. math::
        \\mathfrak{Re}(z[t]) &= (1-\\alpha)(\\cos\\phi\\ \\mathfrak{Re}(z[t-1])
            - \\sin\\phi\\ \\mathfrak{Im}(z[t-1])) + \\mathfrak{Re}(x[t]) + \\text{real bias}\\

        \\mathfrak{Im}(z[t]) &= (1-\\alpha)(\\sin\\phi\\ \\mathfrak{Re}(z[t-1])
            + \\cos\\phi\\ \\mathfrak{Im}(z[t-1])) + \\mathfrak{Im}(x[t]) + \\text{imag bias} \\

        s[t] &= |z[t]| \\geq \\vartheta \\text{ and } \\arg(z[t]) = 0

    Parameters
    ----------
    threshold : float
    period : float or (min, max)
        oscillation period, at least 4 steps.
    decay : float or (min, max)
    tau_grad, scale_grad, scale, norm, dropout, shared_param, persistent_state,
    requires_grad, graded_spike : as for the CUBA neuron.
    log_init : bool
        per-channel frequencies log-spaced (True) or uniform (False).
    """

    def __init__(self, threshold, period, decay, tau_grad=1, scale_grad=1, scale=1 << 6, norm=None,
                 dropout=None, shared_param=True, persistent_state=False, requires_grad=False,
                 graded_spike=False, log_init=True):
        super().__init__(
            threshold=threshold, tau_grad=tau_grad, scale_grad=scale_grad, p_scale=1 << 12, w_scale=scale,
            s_scale=scale * (1 << 6), norm=norm, dropout=dropout, persistent_state=persistent_state,
            shared_param=shared_param, requires_grad=requires_grad, complex=True)
        self.graded_spike = graded_spike
        self.log_init = log_init
        self._init_rotation(period, decay)
        self.register_buffer('real_state', torch.zeros(1, dtype=torch.float), persistent=False)
        self.register_buffer('imag_state', torch.zeros(1, dtype=torch.float), persistent=False)
        self.clamp()

    @property
    def device_params(self):
        return {
            'type': 'RF_PHASE',
            'sinDecay': self.cx_sin_decay,
            'cosDecay': self.cx_cos_decay,
            'vThMant': self.v_th_mant,
            'gradedSpike': self.graded_spike,
        }

    def _prepare(self, input):
        real_input, imag_input = self._check_pair(input)
        if self._bind_shape(real_input) and not self.shared_param:
            self._sample_rotation()
        self._sync_states(real_input, {'real_state': 0, 'imag_state': 0})
        if self.requires_grad:
            self.clamp()
        return self._normalise(real_input, imag_input)

    def dynamics(self, input):
        """``(real, imag)`` response to the complex input tuple."""
        real_input, imag_input = self._prepare(input)
        real, imag = resonator.dynamics(
            real_input, imag_input, quantize(self.sin_decay), quantize(self.cos_decay), self.real_state,
            self.imag_state, self.s_scale, debug=self.debug)
        if self.persistent_state:
            with torch.no_grad():
                self.real_state = real[..., -1].clone()
        return real, imag

    def spike(self, real, imag):
        """Spikes where the state crosses the positive real axis above threshold."""
        spike = complex.Spike.apply(
            real, imag, self.threshold, self.tau_rho * TAU_RHO_MULT, self.scale_rho * SCALE_RHO_MULT,
            self.graded_spike, self.imag_state, 1)
        if self.persistent_state:
            with torch.no_grad():
                self.imag_state = imag[..., -1].clone()
        if self.drop is not None:
            spike = self.drop(spike)
        return spike

    def forward(self, input):
        """Spike response to the complex input tuple ``(real_input, imag_input)``."""
        if not self._fusable:
            real, imag = self.dynamics(input)
            return self.spike(real, imag)
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
        spike, final_re, final_im, final_s = _FusedForward.apply(
            real_input, imag_input, quantize(self.sin_decay), quantize(self.cos_decay), self.real_state,
            self.imag_state, self.threshold, self.s_scale, self.tau_rho * TAU_RHO_MULT,
            self.scale_rho * SCALE_RHO_MULT, self.graded_spike is True, None, None, None, None, 0.0, 0.0,
            spike_delay, delay_head)
        if self.persistent_state:
            with torch.no_grad():
                self.real_state = final_re
                self.imag_state = final_im
        return spike, final_s
