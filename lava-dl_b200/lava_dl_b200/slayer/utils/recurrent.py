"""Recurrent walk over time (``src/lava/lib/dl/slayer/utils/recurrent.py``).

The reference loops over the time axis in Python, calling the neuron with one
time step at a time.  Here the whole walk is one kernel launch each way
(``sb_cuba_recurrent_fwd`` / ``sb_cuba_recurrent_bwd``); only the gradient of
the recurrent matrix, a plain matrix product, is left to the GEMM library, as
in the reference (``recurrent.py:101-110``)."""

import torch

from ... import _ops
from .quantize import quantize


class _CubaRecurrent(torch.autograd.Function):
    @staticmethod
    def forward(ctx, z, rec, cdecay, vdecay, cstate, vstate, threshold, w_scale, tau_rho, scale_rho, graded):
        r = _ops.cuba_recurrent_fwd(z, rec, cdecay, vdecay, cstate, vstate, threshold, w_scale, graded=graded)
        ctx.save_for_backward(r['voltage'], r['spike'], rec)
        ctx.consts = (threshold, tau_rho, scale_rho, graded)
        ctx.mark_non_differentiable(r['final_c'], r['final_v'], r['final_s'])
        return r['spike'], r['final_c'], r['final_v'], r['final_s']

    @staticmethod
    def backward(ctx, grad_spike, *_):
        voltage, spike, rec = ctx.saved_tensors
        threshold, tau_rho, scale_rho, graded = ctx.consts
        grad_z = _ops.cuba_recurrent_bwd(grad_spike, voltage, rec, threshold, tau_rho, scale_rho, graded)
        grad_rec = None
        if ctx.needs_input_grad[1]:
            C = voltage.shape[1]
            go = grad_z[..., 1:].transpose(0, 1).reshape(C, -1)
            si = spike[..., :-1].transpose(1, 2).reshape(-1, C)
            grad_rec = torch.matmul(go, si)
        # a neuron call with a single time step has no decay gradient (leaky_integrator.py:234-259)
        return (grad_z, grad_rec) + (None,) * 9


def custom_recurrent(z, neuron, recurrent_synapse):
    """``s[t] = neuron(z[t] + R s[t-1])`` for ``z`` of shape ``[batch, neurons, time]``.
    ``neuron`` keeps its state across calls (``persistent_state``), as the recurrent
    blocks require (``block/base.py:1455-1456``)."""
    from ..neuron import cuba   # the neuron package imports this one
    from ..neuron.dynamics import leaky_integrator
    if not isinstance(neuron, cuba.Neuron) or neuron.norm is not None or neuron.drop is not None:
        raise NotImplementedError('the recurrent kernel covers the CUBA neuron without normalisation or dropout')
    if z.dim() != 3:
        raise ValueError(f'recurrent input must be [batch, neurons, time], got {tuple(z.shape)}')
    mat_shape = recurrent_synapse.weight.shape[:2]
    rec = recurrent_synapse.weight.reshape(mat_shape)
    if recurrent_synapse.pre_hook_fx is not None:
        rec = recurrent_synapse.pre_hook_fx(rec)
    neuron._prepare(z)
    if not neuron._fusable:
        raise NotImplementedError('the recurrent kernel needs a power-of-two weight scale')
    spike, final_c, final_v, final_s = _CubaRecurrent.apply(
        z, rec, quantize(neuron.current_decay), quantize(neuron.voltage_decay),
        neuron.current_state, neuron.voltage_state, neuron.threshold + neuron.threshold_eps, neuron.s_scale,
        neuron.tau_rho * cuba.TAU_RHO_MULT, neuron.scale_rho * cuba.SCALE_RHO_MULT, neuron.graded_spike is True)
    if neuron.persistent_state:
        with torch.no_grad():
            neuron.current_state = final_c
            neuron.voltage_state = leaky_integrator.persistent_state(final_v, final_s)
    return spike
