"""Leaky integrator dynamics
(``src/lava/lib/dl/slayer/neuron/dynamics/leaky_integrator.py:50-259``)."""

import torch

from .... import _ops
from . import _debug


def dynamics(input, decay, state, w_scale, threshold=None, debug=False):
    """Leaky integrator in Loihi fixed-point arithmetic.

    .. math::
        y[t] &= (1 - \\alpha)\\,y[t-1] + x[t] \\

        s[t] &= y[t] \\geq \\vartheta \\

        y[t] &= y[t]\\,(1-s[t])

    Parameters
    ----------
    input : torch tensor
        CUDA tensor, time last.
    decay : torch tensor
        decay (un-scaled integer value, 0..4096), 1 element or one per channel.
    state : torch tensor
        initial state, 1 element or ``input.shape[:-1]``.
    w_scale : int
        scale of the integer representation.
    threshold : float or None
        reset threshold; ``None`` means no reset.
    debug : bool
        no second implementation is run (there is none to compare with): checks that the scaled
        states are integers below 2^30 in magnitude and that the device status word is clean.

    Returns
    -------
    torch tensor
        leaky integrator output.
    """
    output = _LIDynamics.apply(input, decay, state, threshold, w_scale)
    if debug:
        _debug.check_quantised(w_scale, output=output)
    return output


def persistent_state(state, spike):
    """State to carry over when the last time bin spiked: reset to zero there."""
    spike = (spike > 0).to(state.dtype)
    return state * (1 - spike)


class _LIDynamics(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, decay, state, threshold, w_scale):
        output = _ops.li_fwd(input, decay, state, w_scale, threshold)
        ctx.save_for_backward(output, decay)
        return output

    @staticmethod
    def backward(ctx, grad_output):
        output, decay = ctx.saved_tensors
        grad_input, grad_decay = _ops.li_bwd(grad_output, output, decay, ctx.needs_input_grad[1])
        return grad_input, grad_decay, None, None, None
