"""CUBA leaky integrate-and-fire neuron
(``src/lava/lib/dl/slayer/neuron/cuba.py:108-440``)."""

import torch

from . import base
from .dynamics import leaky_integrator
from ..spike.spike import Spike
from ..utils import quantize
from ... import _ops
from ..axon.delay import delay_gradient

# heuristic multipliers so that scale_grad = tau_grad = 1 is a good start
SCALE_RHO_MULT = 0.1
TAU_RHO_MULT = 100


def neuron_params(device_params, scale=1 << 6, p_scale=1 << 12):
    """Translate Loihi device parameters to constructor arguments."""
    return {
        'threshold': device_params['vThMant'] / scale,
        'current_decay': device_params['iDecay'] / p_scale,
        'voltage_decay': device_params['vDecay'] / p_scale,
    }


def chain_backward(ctx, grad_current, grad_voltage, current, voltage, cdecay, vdecay):
    """Backward of voltage = LI(current), current = LI(x) for gradients arriving
    at either series: returns (grad_x, grad_cdecay, grad_vdecay)."""
    g_vdecay = None
    g_cur = grad_current
    if grad_voltage is not None:
        g_from_v, g_vdecay = _ops.li_bwd(grad_voltage, voltage, vdecay, ctx.needs_input_grad[2])
        g_cur = g_from_v if g_cur is None else g_cur + g_from_v
    elif ctx.needs_input_grad[2]:
        g_vdecay = torch.zeros_like(vdecay)
    if g_cur is None:
        g_cdecay = torch.zeros_like(cdecay) if ctx.needs_input_grad[1] else None
        return torch.zeros_like(current), g_cdecay, g_vdecay
    g_in, g_cdecay = _ops.li_bwd(g_cur, current, cdecay, ctx.needs_input_grad[1])
    return g_in, g_cdecay, g_vdecay


class _FusedDynamics(torch.autograd.Function):
    """current, voltage = LI(LI(x)) in one pass; backward = two reverse scans."""

    @staticmethod
    def forward(ctx, input, cdecay, vdecay, cstate, vstate, threshold, w_scale):
        r = _ops.cuba_fwd(input, cdecay, vdecay, cstate, vstate, threshold, w_scale,
                          want_current=True, want_spike=False)
        ctx.save_for_backward(r['current'], r['voltage'], cdecay, vdecay)
        ctx.set_materialize_grads(False)
        return r['current'], r['voltage']

    @staticmethod
    def backward(ctx, grad_current, grad_voltage):
        current, voltage, cdecay, vdecay = ctx.saved_tensors
        return chain_backward(ctx, grad_current, grad_voltage, current, voltage, cdecay, vdecay) + (None,) * 4


class _FusedForward(torch.autograd.Function):
    """spike = Spike(LI(LI(x))) in one pass each way.  Also returns the voltage
    series and the last-bin current / voltage / spike for state hand-over."""

    @staticmethod
    def forward(ctx, input, cdecay, vdecay, cstate, vstate, threshold, w_scale, tau_rho, scale_rho, graded,
                spike_delay=0, delay_head=None, axon_delay=None, axon_ts=1, axon_grad_scale=1):
        need_dgrad = ctx.needs_input_grad[1] or ctx.needs_input_grad[2]
        ctx.set_materialize_grads(False)   # no zero tensors for the outputs nobody differentiates
        # the voltage series is what the backward pass reads: with nothing to differentiate (inference)
        # it is not written at all, a third of the kernel's traffic
        need_voltage = graded or any(ctx.needs_input_grad)
        r = _ops.cuba_fwd(input, cdecay, vdecay, cstate, vstate, threshold, w_scale,
                          want_current=need_dgrad, want_spike=True, graded=graded, spike_scale=1.0,
                          spike_delay=spike_delay, delay_head=delay_head,
                          axon_delay=None if axon_delay is None else axon_delay.data, axon_delay_ts=axon_ts,
                          want_voltage=need_voltage)
        if not need_voltage:
            ctx.mark_non_differentiable(r['final_c'], r['final_v'], r['final_s'])
            return r['spike'], None, r['final_c'], r['final_v'], r['final_s']
        saved = [r['voltage'], cdecay, vdecay]
        if need_dgrad:
            saved.append(r['current'])
        if axon_delay is not None:
            saved += [axon_delay.data, r['spike']]
        ctx.save_for_backward(*saved)
        ctx.consts = (threshold, tau_rho, scale_rho, graded, need_dgrad, spike_delay, axon_delay is not None, axon_ts,
                      axon_grad_scale, ctx.needs_input_grad[12] if axon_delay is not None else False)
        ctx.mark_non_differentiable(r['voltage'], r['final_c'], r['final_v'], r['final_s'])
        return r['spike'], r['voltage'], r['final_c'], r['final_v'], r['final_s']

    @staticmethod
    def backward(ctx, grad_spike, *_):
        (threshold, tau_rho, scale_rho, graded, need_dgrad, spike_delay, has_axon, axon_ts, axon_grad_scale,
         need_axon_grad) = ctx.consts
        if grad_spike is None:
            return (None,) * 15
        voltage, cdecay, vdecay = ctx.saved_tensors[:3]
        current = ctx.saved_tensors[3] if need_dgrad else None
        g_axon = None
        if has_axon:
            # the axonal delay is undone here as a separate shift (the forward folded it into the store);
            # its own gradient is the finite difference of the delayed output (axon/delay.py:205-216)
            axon_delay, delayed = ctx.saved_tensors[-2:]
            grad_spike = _ops._c(grad_spike)
            if need_axon_grad:
                g_axon = delay_gradient(delayed, grad_spike, axon_ts) * axon_grad_scale
            grad_spike = _ops.shift(grad_spike, -axon_delay, axon_ts)
        g_in, g_cdecay, g_vdecay = _ops.cuba_bwd(
            grad_spike, voltage, threshold, current, cdecay, vdecay, tau_rho, scale_rho, graded, need_dgrad,
            spike_delay=spike_delay)
        return (g_in, g_cdecay, g_vdecay) + (None,) * 9 + (g_axon, None, None)


class Neuron(base.Neuron):
    """Loihi CUBA neuron.

    .. math::
        u[t] &= (1 - \\alpha_u)\\,u[t-1] + x[t] \\

        v[t] &= (1 - \\alpha_v)\\,v[t-1] + u[t] + \\text{bias} \\

        s[t] &= v[t] \\geq \\vartheta \\

        v[t] &= v[t]\\,(1-s[t])

    Parameters
    ----------
    threshold : float
    current_decay, voltage_decay : float or (min, max)
        decay rates; a pair gives the sampling range when ``shared_param`` is False.
    tau_grad, scale_grad : float
    scale : int
        quantisation scale (default ``1 << 6``); states are scaled by ``scale * 64``.
    norm, dropout : callables or None
    shared_param, persistent_state, requires_grad, graded_spike : bool
    """

    def __init__(self, threshold, current_decay, voltage_decay, tau_grad=1, scale_grad=1, scale=1 << 6,
                 norm=None, dropout=None, shared_param=True, persistent_state=False, requires_grad=False,
                 graded_spike=False):
        super().__init__(
            threshold=threshold, tau_grad=tau_grad, scale_grad=scale_grad, p_scale=1 << 12, w_scale=scale,
            s_scale=scale * (1 << 6), norm=norm, dropout=dropout, persistent_state=persistent_state,
            shared_param=shared_param, requires_grad=requires_grad)
        self.graded_spike = graded_spike
        # SLAYER spikes at v >= vth, Loihi at v > vth: the epsilon aligns them
        self.threshold_eps = 0.01 / self.s_scale

        if self.shared_param:
            self._need_scalar(current_decay, 'current decay')
            self._need_scalar(voltage_decay, 'voltage decay')
            init_c, init_v = current_decay, voltage_decay
        else:
            self.current_decay_min, self.current_decay_max = self._range(current_decay, 'current decay', 0.01)
            self.voltage_decay_min, self.voltage_decay_max = self._range(voltage_decay, 'voltage decay', 0.01)
            init_c, init_v = self.current_decay_min, self.voltage_decay_min
        self._add_decay('current_decay', self.p_scale * init_c)
        self._add_decay('voltage_decay', self.p_scale * init_v)
        self.register_buffer('current_state', torch.zeros(1, dtype=torch.float), persistent=False)
        self.register_buffer('voltage_state', torch.zeros(1, dtype=torch.float), persistent=False)
        self.clamp()

    def clamp(self):
        """Keep the decays inside ``[0, p_scale]``."""
        with torch.no_grad():
            self.current_decay.data.clamp_(0, self.p_scale)
            self.voltage_decay.data.clamp_(0, self.p_scale)

    @property
    def device(self):
        return self.current_decay.device

    @property
    def cx_current_decay(self):
        """Compartment current decay as configured on Loihi."""
        return self._cx(self.current_decay)

    @property
    def cx_voltage_decay(self):
        """Compartment voltage decay as configured on Loihi."""
        return self._cx(self.voltage_decay)

    @property
    def ref_delay(self):
        return 1

    @property
    def scale(self):
        return self.w_scale

    @property
    def device_params(self):
        return {
            'type': 'CUBA',
            'iDecay': self.cx_current_decay,
            'vDecay': self.cx_voltage_decay,
            'vThMant': self.v_th_mant,
            'refDelay': self.ref_delay,
            'gradedSpike': self.graded_spike,
        }

    # ------------------------------------------------------------------
    def _prepare(self, input):
        if self._bind_shape(input) and not self.shared_param:
            self.current_decay.data = self.p_scale * self._uniform(self.current_decay_min, self.current_decay_max)
            self.voltage_decay.data = self.p_scale * self._uniform(self.voltage_decay_min, self.voltage_decay_max)
            del self.current_decay_min, self.current_decay_max
            del self.voltage_decay_min, self.voltage_decay_max
        self._sync_states(input, {'current_state': 0, 'voltage_state': 0})
        if self.requires_grad:
            self.clamp()

    def dynamics(self, input):
        """Current and voltage response (reset applied, no spike extraction).

        Returns
        -------
        current, voltage : torch tensors
        """
        self._prepare(input)
        threshold = self.threshold + self.threshold_eps
        if self.norm is None and self._fusable:
            current, voltage = _FusedDynamics.apply(
                input, quantize(self.current_decay), quantize(self.voltage_decay),
                self.current_state, self.voltage_state, threshold, self.s_scale)
        else:
            current = leaky_integrator.dynamics(
                input, quantize(self.current_decay), self.current_state.contiguous(), self.s_scale,
                debug=self.debug)
            if self.norm is not None:
                current = self.norm(current)
            voltage = leaky_integrator.dynamics(
                current, quantize(self.voltage_decay), self.voltage_state.contiguous(), self.s_scale,
                threshold, debug=self.debug)
        if self.persistent_state:
            with torch.no_grad():
                self.current_state = current[..., -1].clone()
                self.voltage_state = voltage[..., -1].clone()
        return current, voltage

    def spike(self, voltage):
        """Spikes of a voltage series that already carries the reset dynamics."""
        spike = Spike.apply(
            voltage, self.threshold + self.threshold_eps, self.tau_rho * TAU_RHO_MULT,
            self.scale_rho * SCALE_RHO_MULT, self.graded_spike, self.voltage_state, 1)
        if self.persistent_state:
            with torch.no_grad():
                self.voltage_state = leaky_integrator.persistent_state(
                    self.voltage_state, spike[..., -1]).detach().clone()
        if self.drop is not None:
            spike = self.drop(spike)
        return spike

    def forward(self, input):
        """Spike response to ``input`` (``[batch, ..., time]``)."""
        if self.norm is not None or not self._fusable:
            _, voltage = self.dynamics(input)
            return self.spike(voltage)
        spike, _ = self._fused_forward(input, 0, None)
        if self.drop is not None:
            spike = self.drop(spike)
        return spike

    def forward_packed(self, input, want_voltage=False):
        """Inference-only ``forward`` with the spikes as bits (no counterpart in lava-dl).

        Returns an int32 tensor ``input.shape[:-1] + (ceil(T / 32),)``: bit ``i`` of word ``w``
        is the spike at step ``32 w + i``; ``slayer.utils.unpack_spikes(bits, T)`` restores what
        ``forward`` returns.  The fp32 spike tensor is never written, so the pass moves a third of
        the bytes and its result is 32 times smaller to copy to the host.  No gradient, binary
        spikes, no normalisation or dropout; persistent state is kept as ``forward`` keeps it.
        With ``want_voltage`` the voltage series is returned as well: ``(bits, voltage)``."""
        if self.norm is not None or not self._fusable or self.graded_spike is True or self.drop is not None:
            raise NotImplementedError('forward_packed needs binary spikes and no normalisation or dropout')
        self._prepare(input)
        with torch.no_grad():
            r = _ops.cuba_fwd_packed(input, quantize(self.current_decay), quantize(self.voltage_decay),
                                     self.current_state, self.voltage_state,
                                     self.threshold + self.threshold_eps, self.s_scale, want_voltage=want_voltage)
            if self.persistent_state:
                self.current_state = r['final_c']
                self.voltage_state = leaky_integrator.persistent_state(r['final_v'], r['final_s'])
        return (r['spike_bits'], r['voltage']) if want_voltage else r['spike_bits']

    @property
    def fuses_step_delay(self):
        """True when ``forward_step_delayed`` can write the spikes one step late
        inside the kernel (binary spikes, no normalisation, no dropout)."""
        return self.norm is None and self._fusable and self.graded_spike is not True and self.drop is None

    fuses_axon_delay = True   # a bounded axonal delay of the block rides on the same store

    def forward_step_delayed(self, input, delay_head=None, axon_delay=None, axon_ts=1, axon_grad_scale=1):
        """``forward`` with the blocks' one-step delay folded in: returns
        ``(delayed_spike, last_spike)`` where ``delayed_spike[..., t] = spike[..., t - 1]``,
        ``delayed_spike[..., 0] = delay_head`` (0 when ``None``), and ``last_spike``
        is the undelayed spike of the last time bin.  ``axon_delay`` (one value per
        neuron, at most 62 steps) delays every neuron's train further, as
        ``axon.Delay`` does after the step delay; it receives ``axon.Delay``'s gradient."""
        return self._fused_forward(input, 1, delay_head, axon_delay, axon_ts, axon_grad_scale)

    def _fused_forward(self, input, spike_delay, delay_head, axon_delay=None, axon_ts=1, axon_grad_scale=1):
        self._prepare(input)
        spike, _, final_c, final_v, final_s = _FusedForward.apply(
            input, quantize(self.current_decay), quantize(self.voltage_decay),
            self.current_state, self.voltage_state, self.threshold + self.threshold_eps, self.s_scale,
            self.tau_rho * TAU_RHO_MULT, self.scale_rho * SCALE_RHO_MULT, self.graded_spike is True,
            spike_delay, delay_head, axon_delay, axon_ts, axon_grad_scale)
        if self.persistent_state:
            with torch.no_grad():
                self.current_state = final_c
                self.voltage_state = leaky_integrator.persistent_state(final_v, final_s)
        return spike, final_s
