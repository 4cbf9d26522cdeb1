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
        ctx.decay_shapes = (cdecay.shape, vdecay.shape)
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
        # a neuron call with a single time step has a decay gradient of exactly zero
        # (leaky_integrator.py:234-259): learnable decays get zeros, as the reference's walk leaves them
        zeros = [torch.zeros(shape, device=voltage.device) if ctx.needs_input_grad[2 + i] else None
                 for i, shape in enumerate(ctx.decay_shapes)]
        return (grad_z, grad_rec, zeros[0], zeros[1]) + (None,) * 7


class _StepwiseRecurrent(torch.autograd.Function):
    """The reference's own walk (``utils/recurrent.py:45-112``): one neuron call with a single time
    step per step, feedback ``s[t-1] R^T`` in front of it, and for the gradient the reverse walk in
    which only ``R`` couples the steps.  Any neuron works, at the price of a dozen launches per
    step; it is what runs when the one-launch kernel does not take the case."""

    @staticmethod
    def forward(ctx, z, neuron, recurrent_mat):
        z = z.detach().requires_grad_()
        x = torch.zeros_like(z)
        recurrent_mat_T = recurrent_mat.transpose(0, 1).clone().detach().to(z.device)
        ctx.dend_sums, ctx.spikes = [], []
        spike = torch.zeros(z.shape[:-1] + (1,), device=z.device)
        for time in range(z.shape[-1]):
            feedback = torch.matmul(spike[..., 0], recurrent_mat_T)
            with torch.enable_grad():
                dend_sum = (z[..., time] + feedback).detach().requires_grad_()
                spike = neuron(torch.unsqueeze(dend_sum, dim=-1))
            ctx.dend_sums.append(dend_sum)
            ctx.spikes.append(spike)
            x[..., time:time + 1] = spike
        ctx.recurrent_mat = recurrent_mat
        ctx.x = x
        return x.detach()

    @staticmethod
    def backward(ctx, grad_x):
        grad_z = torch.zeros_like(grad_x)
        grad_spike = 0
        for time in range(grad_x.shape[-1])[::-1]:
            grad_spike = grad_spike + grad_x[..., time:time + 1]
            torch.autograd.backward(ctx.spikes[time], grad_spike)
            grad_dend_sum = ctx.dend_sums[time].grad
            grad_spike = torch.unsqueeze(torch.matmul(grad_dend_sum, ctx.recurrent_mat), dim=-1)
            grad_z[..., time] = grad_dend_sum
        C = grad_z.shape[1]
        grad_output = grad_z[..., 1:].transpose(0, 1).reshape(C, -1)
        spikes_in = ctx.x[..., :-1].transpose(1, 2).reshape(-1, ctx.x.shape[1])
        return grad_z, None, torch.matmul(grad_output, spikes_in)


def _kernel_takes(z, neuron):
    """The one-launch kernel covers the CUBA neuron (no normalisation, no dropout, power-of-two
    scale) on ``[batch, neurons, time]`` input with at most 1024 neurons."""
    from ..neuron import cuba   # the neuron package imports this one
    return (isinstance(neuron, cuba.Neuron) and neuron.norm is None and neuron.drop is None
            and z.dim() == 3 and z.shape[1] <= 1024 and z.is_cuda)


def recurrent_walk(z, neuron, rec):
    """``s[t] = neuron(z[t] + R s[t-1])`` with the recurrent matrix ``rec`` given as a tensor
    (already hooked / quantised; gradients flow back into whatever it was computed from)."""
    from ..neuron import cuba
    from ..neuron.dynamics import leaky_integrator
    if _kernel_takes(z, neuron):
        neuron._prepare(z)
        if neuron._fusable:
            spike, final_c, final_v, final_s = _CubaRecurrent.apply(
                z, rec, quantize(neuron.current_decay), quantize(neuron.voltage_decay),
                neuron.current_state, neuron.voltage_state, neuron.threshold + neuron.threshold_eps,
                neuron.s_scale, neuron.tau_rho * cuba.TAU_RHO_MULT, neuron.scale_rho * cuba.SCALE_RHO_MULT,
                neuron.graded_spike is True)
            if neuron.persistent_state:
                with torch.no_grad():
                    neuron.current_state = final_c
                    neuron.voltage_state = leaky_integrator.persistent_state(final_v, final_s)
            return spike
    if getattr(neuron, 'complex', False) or isinstance(z, (tuple, list)):
        # the reference's walk indexes z as one tensor (utils/recurrent.py:59-67): a complex
        # neuron's (real, imaginary) input fails there in the same way
        raise AttributeError("'tuple' object has no attribute 'shape'")
    return _StepwiseRecurrent.apply(z, neuron, rec)


def custom_recurrent(z, neuron, recurrent_synapse):
    """``s[t] = neuron(z[t] + R s[t-1])`` for ``z`` of shape ``[batch, neurons, time]``.
    ``neuron`` keeps its state across calls (``persistent_state``), as the recurrent
    blocks require (``block/base.py:1455-1456``).  A CUBA neuron of up to 1024 units runs as one
    kernel launch per direction; every other case walks step by step as the reference does."""
    mat_shape = recurrent_synapse.weight.shape[:2]
    rec = recurrent_synapse.weight.reshape(mat_shape)
    if recurrent_synapse.pre_hook_fx is not None:
        rec = recurrent_synapse.pre_hook_fx(rec)
    return recurrent_walk(z, neuron, rec)
