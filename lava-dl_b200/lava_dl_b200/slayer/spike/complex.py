"""Phase-threshold (complex) spike with surrogate gradient
(``src/lava/lib/dl/slayer/spike/complex.py:10-167``)."""

import torch

from ... import _ops


class Spike(torch.autograd.Function):
    """Complex spike function with autograd link.

    .. math::
        f_s(z) = \\mathcal{H}(|z| - \\vartheta)\\,\\delta(\\arg(z))

    A spike is emitted where ``real >= threshold`` and the imaginary part
    crosses zero upwards (``imag[t-1] < 0 <= imag[t]``, ``imag[-1] = imag_last``).

    Examples
    --------
    >>> spike = Spike.apply(re, im, th, tau_rho, scale_rho, False, 0, 1)
    """

    derivative = None

    @staticmethod
    def forward(ctx, real, imag, threshold, tau_rho, scale_rho, graded_spike, imag_last, scale):
        graded = graded_spike is True
        spikes = _ops.cspike_fwd(real, imag, threshold, imag_last, graded, scale)
        if torch.is_tensor(threshold):
            ctx.save_for_backward(real, imag, threshold.detach())
            ctx.threshold = None
        else:
            ctx.save_for_backward(real, imag)
            ctx.threshold = threshold
        ctx.consts = (float(tau_rho), float(scale_rho), graded)
        return spikes

    @staticmethod
    def backward(ctx, grad_output):
        real, imag = ctx.saved_tensors[:2]
        threshold = ctx.saved_tensors[2] if ctx.threshold is None else ctx.threshold
        tau_rho, scale_rho, graded = ctx.consts
        grad_real, grad_imag = _ops.cspike_bwd(real, imag, threshold, grad_output, tau_rho, scale_rho, graded)
        return grad_real, grad_imag, None, None, None, None, None, None
