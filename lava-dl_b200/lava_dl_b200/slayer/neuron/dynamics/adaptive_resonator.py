"""Adaptive resonator dynamics
(``src/lava/lib/dl/slayer/neuron/dynamics/adaptive_resonator.py:49-525``)."""

import torch

from .... import _ops
from . import _debug
from .resonator import _raise_on_nan


def dynamics(real_input, imag_input, sin_decay, cos_decay, ref_decay, th_decay, real_state, imag_state, ref_state,
             th_state, th_scale, th0, w_scale, debug=False):
    """Resonator plus adaptive threshold / refractory traces in one recurrence;
    the spike condition is ``imag >= threshold + refractory`` and the resonator
    state is not reset.  Returns ``(real, imag, threshold, refractory)``;
    gradients flow to the inputs and to ``sin_decay`` / ``cos_decay``.

    ``debug=True`` does not run a second implementation (there is none to compare with): it checks that the
    scaled states are integers below 2^30 in magnitude and that the device status word is clean.
    """
    out = _AdResDynamics.apply(
        real_input, imag_input, sin_decay, cos_decay, ref_decay, th_decay, real_state, imag_state, ref_state,
        th_state, th_scale, th0, w_scale)
    if debug:
        _debug.check_quantised(w_scale, real=out[0], imag=out[1], threshold=out[2], refractory=out[3])
    return out


def persistent_ref_state(ref_state, spike, th_state):
    """Refractory state to carry over when the last time bin spiked."""
    spike = (spike > 0).to(ref_state.dtype)
    return ref_state + 2 * spike * th_state


def persistent_th_state(th_state, spike, th_step):
    """Threshold state to carry over when the last time bin spiked."""
    spike = (spike > 0).to(th_state.dtype)
    return th_state + spike * th_step


class _AdResDynamics(torch.autograd.Function):
    @staticmethod
    def forward(ctx, real_input, imag_input, sin_decay, cos_decay, ref_decay, th_decay, real_state, imag_state,
                ref_state, th_state, th_scale, th0, w_scale):
        real, imag, threshold, refractory = _ops.adres_fwd(
            real_input, imag_input, sin_decay, cos_decay, ref_decay, th_decay, real_state, imag_state, ref_state,
            th_state, th_scale, th0, w_scale)
        ctx.save_for_backward(real, imag, sin_decay, cos_decay)
        ctx.mark_non_differentiable(threshold, refractory)
        return real, imag, threshold, refractory

    @staticmethod
    def backward(ctx, grad_real, grad_imag, grad_threshold, grad_refractory):
        real, imag, sin_decay, cos_decay = ctx.saved_tensors
        need = ctx.needs_input_grad[2] or ctx.needs_input_grad[3]
        gre, gim, gsin, gcos = _ops.res_bwd(grad_real, grad_imag, real, imag, sin_decay, cos_decay, need)
        _raise_on_nan(grad_sin_decay=gsin, grad_cos_decay=gcos)
        return (gre, gim, gsin, gcos) + (None,) * 9
