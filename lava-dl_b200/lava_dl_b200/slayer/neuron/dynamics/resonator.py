"""Resonator dynamics
(``src/lava/lib/dl/slayer/neuron/dynamics/resonator.py:49-467``)."""

import torch

from .... import _ops
from . import _debug


def dynamics(real_input, imag_input, sin_decay, cos_decay, real_state, imag_state, w_scale, threshold=None,
             debug=False):
    """Damped rotation of a complex state in Loihi fixed-point arithmetic.

    .. math::
        \\mathfrak{Re}(z[t]) &= (1-\\alpha)(\\cos\\phi\\ \\mathfrak{Re}(z[t-1])
            - \\sin\\phi\\ \\mathfrak{Im}(z[t-1])) + \\mathfrak{Re}(x[t])\\

        \\mathfrak{Im}(z[t]) &= (1-\\alpha)(\\sin\\phi\\ \\mathfrak{Re}(z[t-1])
            + \\cos\\phi\\ \\mathfrak{Im}(z[t-1])) + \\mathfrak{Im}(x[t])

    ``sin_decay``/``cos_decay`` are the products with ``(1-\\alpha)`` scaled by
    4096.  With a ``threshold`` the Izhikevich reset is applied where the
    imaginary part reaches it.  Returns ``(real, imag)``.

    ``debug=True`` does not run a second implementation (there is none to compare with): it checks that the
    scaled states are integers below 2^30 in magnitude and that the device status word is clean.
    """
    real, imag = _ResDynamics.apply(
        real_input, imag_input, sin_decay, cos_decay, real_state, imag_state, threshold, w_scale)
    if debug:
        _debug.check_quantised(w_scale, real=real, imag=imag)
    return real, imag


def persistent_real_state(real_state, spike):
    """Real state to carry over when the last time bin spiked (reset to zero)."""
    spike = (spike > 0).to(real_state.dtype)
    return real_state * (1 - spike)


def persistent_imag_state(imag_state, spike, threshold, scale):
    """Imaginary state to carry over when the last time bin spiked: one
    quantisation step below the threshold (``resonator.py:152-174``)."""
    spike = (spike > 0).to(imag_state.dtype)
    return spike * (threshold - 1 / scale) + (1 - spike) * imag_state


class _ResDynamics(torch.autograd.Function):
    @staticmethod
    def forward(ctx, real_input, imag_input, sin_decay, cos_decay, real_state, imag_state, threshold, w_scale):
        real, imag = _ops.res_fwd(
            real_input, imag_input, sin_decay, cos_decay, real_state, imag_state, w_scale, threshold)
        ctx.save_for_backward(real, imag, sin_decay, cos_decay)
        return real, imag

    @staticmethod
    def backward(ctx, grad_real, grad_imag):
        real, imag, sin_decay, cos_decay = ctx.saved_tensors
        need = ctx.needs_input_grad[2] or ctx.needs_input_grad[3]
        gre, gim, gsin, gcos = _ops.res_bwd(grad_real, grad_imag, real, imag, sin_decay, cos_decay, need)
        _raise_on_nan(grad_sin_decay=gsin, grad_cos_decay=gcos)
        return gre, gim, gsin, gcos, None, None, None, None


def _raise_on_nan(**tensors):
    # the reference aborts on NaN gradients (resonator.py:424-441); the
    # parameter gradients sum over everything, so checking them is enough
    for name, t in tensors.items():
        if t is not None and bool(torch.isnan(t).any()):
            raise Exception(f'{name} has NaN.')
