"""Adaptive leaky integrate-and-fire neuron
(``src/lava/lib/dl/slayer/neuron/alif.py:126-610``)."""

import torch

from . import base
from .cuba import chain_backward
from .dynamics import leaky_integrator, adaptive_threshold
from ..spike.spike import Spike
from ..utils import quantize
from ... import _ops

SCALE_RHO_MULT = 0.1
TAU_RHO_MULT = 100


def neuron_params(device_params, scale=1 << 6, p_scale=1 << 12):
    """Translate Loihi device parameters to constructor arguments."""
    return {
        'threshold': device_params['vThMant'] / scale,
        'threshold_step': device_params['vThMant'] / scale,
        'current_decay': device_params['iDecay'] / p_scale,
        'voltage_decay': device_params['vDecay'] / p_scale,
        'threshold_decay': device_params['thDecay'] / p_scale,
        'refractory_decay': device_params['refDecay'] / p_scale,
    }


class _FusedDynamics(torch.autograd.Function):
    """current, voltage, threshold, refractory in one pass."""

    @staticmethod
    def forward(ctx, input, cdecay, vdecay, ref_decay, th_decay, cstate, vstate, ref_state, th_state, th_step,
                th0, w_scale):
        (current, voltage, threshold, refractory), _ = _ops.alif_fwd(
            input, cdecay, vdecay, ref_decay, th_decay, cstate, vstate, ref_state, th_state, th_step, th0,
            w_scale, dynamics_mode=True)
        ctx.save_for_backward(current, voltage, cdecay, vdecay)
        ctx.mark_non_differentiable(threshold, refractory)
        ctx.set_materialize_grads(False)
        return current, voltage, threshold, refractory

    @staticmethod
    def backward(ctx, grad_current, grad_voltage, *_):
        current, voltage, cdecay, vdecay = ctx.saved_tensors
        return chain_backward(ctx, grad_current, grad_voltage, current, voltage, cdecay, vdecay) + (None,) * 9


class _FusedForward(torch.autograd.Function):
    """spike in one pass each way (decays not learnable on this path)."""

    @staticmethod
    def forward(ctx, input, cdecay, vdecay, ref_decay, th_decay, cstate, vstate, ref_state, th_state, th_step,
                th0, w_scale, tau_rho, scale_rho, graded, spike_delay=0, delay_head=None):
        # the voltage and threshold series are what the backward pass reads: with nothing to
        # differentiate (inference) they are not written, three quarters of the kernel's stores
        lean = not graded and not any(ctx.needs_input_grad)
        # otherwise one series: the spike's surrogate gradient reads voltage - (threshold + refractory)
        # and, the decays not being learnt on this path, the reverse scans read nothing else
        (spike, margin, _), fin = _ops.alif_fwd(
            input, cdecay, vdecay, ref_decay, th_decay, cstate, vstate, ref_state, th_state, th_step, th0,
            w_scale, dynamics_mode=False, graded=graded, spike_scale=1.0, spike_delay=spike_delay,
            delay_head=delay_head, spikes_only=lean, margin=not lean)
        if not lean:
            ctx.save_for_backward(margin, cdecay, vdecay)
        ctx.consts = (tau_rho, scale_rho, graded, spike_delay)
        extras = (fin['final_c'], fin['final_v'], fin['final_th'], fin['final_ref'], fin['final_s'])
        ctx.mark_non_differentiable(*extras)
        return (spike,) + extras

    @staticmethod
    def backward(ctx, grad_spike, *_):
        margin, cdecay, vdecay = ctx.saved_tensors
        tau_rho, scale_rho, graded, spike_delay = ctx.consts
        g_in, _, _ = _ops.cuba_bwd(grad_spike, margin, 0.0, None, cdecay, vdecay, tau_rho, scale_rho, graded,
                                   False, spike_delay=spike_delay)
        return (g_in,) + (None,) * 16


class Neuron(base.Neuron):
    """Adaptive LIF neuron: CUBA integration, adaptive threshold and refractory
    trace; a spike is emitted where ``voltage >= threshold + refractory``.

    .. math::
        u[t] &= (1-\\alpha_u)\\,u[t-1] + x[t] \\

        v[t] &= (1-\\alpha_v)\\,v[t-1] + u[t] + \\text{bias} \\

        \\vartheta[t] &= (1-\\alpha_{\\vartheta})\\,(\\vartheta[t-1] - \\vartheta_0) + \\vartheta_0 \\

        r[t] &= (1-\\alpha_r)\\,r[t-1] \\

        s[t] &= (v[t] - r[t]) \\geq \\vartheta[t] \\

        r[t] &= r[t] + 2\\,s[t]\\,\\vartheta[t] \\

        \\vartheta[t] &= \\vartheta[t] + s[t]\\,\\vartheta_{\\text{step}}

    Parameters
    ----------
    threshold, threshold_step : float
    current_decay, voltage_decay, threshold_decay, refractory_decay : float or (min, max)
    tau_grad, scale_grad, scale, norm, dropout, shared_param, persistent_state,
    requires_grad, graded_spike : as for the CUBA neuron.
    """

    _decays = ('current', 'voltage', 'threshold', 'refractory')

    def __init__(self, threshold, threshold_step, current_decay, voltage_decay, threshold_decay,
                 refractory_decay, tau_grad=1, scale_grad=1, scale=1 << 6, norm=None, dropout=None,
                 shared_param=True, persistent_state=False, requires_grad=False, graded_spike=False):
        super().__init__(
            threshold=threshold, tau_grad=tau_grad, scale_grad=scale_grad, p_scale=1 << 12, w_scale=scale,
            s_scale=scale * (1 << 6), norm=norm, dropout=dropout, persistent_state=persistent_state,
            shared_param=shared_param, requires_grad=requires_grad)
        self.threshold_step = int(threshold_step * self.w_scale) / self.w_scale
        self.graded_spike = graded_spike

        given = dict(current=current_decay, voltage=voltage_decay, threshold=threshold_decay,
                     refractory=refractory_decay)
        if self.shared_param:
            self._need_scalar(current_decay, 'current decay')
            self._need_scalar(voltage_decay, 'voltage decay')
            for kind in self._decays:
                self._add_decay(f'{kind}_decay', self.p_scale * given[kind])
        else:
            for kind in self._decays:
                jitter = 0.01 if kind in ('current', 'voltage') else 0.0
                lo, hi = self._range(given[kind], f'{kind} decay', jitter)
                setattr(self, f'{kind}_decay_min', lo)
                setattr(self, f'{kind}_decay_max', hi)
                self._add_decay(f'{kind}_decay', self.p_scale * lo)
        for name, value in (('current_state', 0.), ('voltage_state', 0.), ('threshold_state', self.threshold),
                            ('refractory_state', 0.)):
            self.register_buffer(name, torch.tensor([value], dtype=torch.float), persistent=False)
        self.clamp()

    def clamp(self):
        """Keep the current and voltage decays inside ``[0, p_scale]``."""
        with torch.no_grad():
            self.current_decay.data.clamp_(0, self.p_scale)
            self.voltage_decay.data.clamp_(0, self.p_scale)

    @property
    def device(self):
        return self.current_decay.device

    @property
    def cx_current_decay(self):
        return self._cx(self.current_decay)

    @property
    def cx_voltage_decay(self):
        return self._cx(self.voltage_decay)

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
    def ref_delay(self):
        return 1

    @property
    def scale(self):
        return self.w_scale

    @property
    def device_params(self):
        return {
            'type': 'ALIF',
            'iDecay': self.cx_current_decay,
            'vDecay': self.cx_voltage_decay,
            'thDecay': self.cx_threshold_decay,
            'refDecay': self.cx_refractory_decay,
            'vThMant': self.v_th_mant,
            'vThStep': self.v_th_step,
            'refDelay': self.ref_delay,
            'gradedSpike': self.graded_spike,
        }

    # ------------------------------------------------------------------
    def _prepare(self, input):
        if self._bind_shape(input) and not self.shared_param:
            for kind in self._decays:
                lo, hi = getattr(self, f'{kind}_decay_min'), getattr(self, f'{kind}_decay_max')
                getattr(self, f'{kind}_decay').data = self.p_scale * self._uniform(lo, hi)
                delattr(self, f'{kind}_decay_min')
                delattr(self, f'{kind}_decay_max')
        self._sync_states(input, {'current_state': 0, 'voltage_state': 0, 'threshold_state': self.threshold,
                                  'refractory_state': 0})
        if self.requires_grad:
            self.clamp()

    def _quantised_decays(self):
        return (quantize(self.current_decay), quantize(self.voltage_decay), quantize(self.refractory_decay),
                quantize(self.threshold_decay))

    def dynamics(self, input):
        """Returns ``current, voltage, threshold, refractory`` series."""
        self._prepare(input)
        if self.norm is not None:
            input = self.norm(input)
        cd, vd, rd, td = self._quantised_decays()
        if self._fusable:
            current, voltage, threshold, refractory = _FusedDynamics.apply(
                input, cd, vd, rd, td, self.current_state, self.voltage_state, self.refractory_state,
                self.threshold_state, self.threshold_step, self.threshold, self.s_scale)
        else:
            current = leaky_integrator.dynamics(input, cd, self.current_state.contiguous(), self.s_scale,
                                                debug=self.debug)
            voltage = leaky_integrator.dynamics(current, vd, self.voltage_state.contiguous(), self.s_scale,
                                                debug=self.debug)
            threshold, refractory = adaptive_threshold.dynamics(
                voltage, self.refractory_state.contiguous(), rd, self.threshold_state.contiguous(), td,
                self.threshold_step, self.threshold, self.s_scale, debug=self.debug)
        if self.persistent_state:
            with torch.no_grad():
                self.current_state = current[..., -1].clone()
                self.voltage_state = voltage[..., -1].clone()
                self.threshold_state = threshold[..., -1].clone()
                self.refractory_state = refractory[..., -1].clone()
        return current, voltage, threshold, refractory

    def _carry_spike(self, last_spike):
        self.refractory_state = adaptive_threshold.persistent_ref_state(
            self.refractory_state, last_spike, self.threshold_state).detach().clone()
        self.threshold_state = adaptive_threshold.persistent_th_state(
            self.threshold_state, last_spike, self.threshold_step).detach().clone()

    def spike(self, voltage, threshold, refractory):
        """Spikes where ``voltage >= threshold + refractory``."""
        spike = Spike.apply(
            voltage, threshold + refractory, self.tau_rho * TAU_RHO_MULT, self.scale_rho * SCALE_RHO_MULT,
            self.graded_spike, self.voltage_state, 1)
        if self.persistent_state:
            with torch.no_grad():
                self._carry_spike(spike[..., -1])
        if self.drop is not None:
            spike = self.drop(spike)
        return spike

    def _learnable_decays(self):
        return self.requires_grad and any(getattr(self, f'{k}_decay').requires_grad for k in self._decays)

    def forward(self, input):
        """Spike response to ``input`` (``[batch, ..., time]``)."""
        if not self._fusable or self._learnable_decays():
            _, voltage, threshold, refractory = self.dynamics(input)
            return self.spike(voltage, threshold, refractory)
        spike, _ = self._fused_forward(input, 0, None)
        if self.drop is not None:
            spike = self.drop(spike)
        return spike

    @property
    def fuses_step_delay(self):
        """True when ``forward_step_delayed`` can write the spikes one step late inside the kernel
        (binary spikes, one-pass forward, no dropout)."""
        return self._fusable and not self._learnable_decays() and self.graded_spike is not True \
            and self.drop is None

    fuses_axon_delay = False   # a block's axonal delay stays a separate shift for this neuron

    def forward_step_delayed(self, input, delay_head=None):
        """``forward`` with the blocks' one-step delay folded in: ``(delayed_spike, last_spike)`` with
        ``delayed_spike[..., t] = spike[..., t - 1]`` and ``delayed_spike[..., 0] = delay_head`` (0 when
        ``None``); ``last_spike`` is the undelayed spike of the last time bin."""
        return self._fused_forward(input, 1, delay_head)

    def _fused_forward(self, input, spike_delay, delay_head):
        self._prepare(input)
        if self.norm is not None:
            input = self.norm(input)
        cd, vd, rd, td = self._quantised_decays()
        spike, final_c, final_v, final_th, final_ref, final_s = _FusedForward.apply(
            input, cd, vd, rd, td, self.current_state, self.voltage_state, self.refractory_state,
            self.threshold_state, self.threshold_step, self.threshold, self.s_scale,
            self.tau_rho * TAU_RHO_MULT, self.scale_rho * SCALE_RHO_MULT, self.graded_spike is True,
            spike_delay, delay_head)
        if self.persistent_state:
            with torch.no_grad():
                self.current_state = final_c
                self.voltage_state = final_v
                self.threshold_state = final_th
                self.refractory_state = final_ref
                self._carry_spike(final_s)
        return spike, final_s
