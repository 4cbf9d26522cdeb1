"""Threshold spike with surrogate gradient
(``src/lava/lib/dl/slayer/spike/spike.py:10-126``)."""

import torch

from ... import _ops


class Spike(torch.autograd.Function):
    """Spiking mechanism with autograd link.

    .. math::
        f_s(x) = \\mathcal{H}(x - \\vartheta)

    Forward: ``voltage >= threshold`` as float, or ``(voltage >= threshold) *
    voltage / scale`` when ``graded_spike``.  Backward: relaxed delta function
    ``scale_rho / (2 tau_rho) * exp(-|v - threshold| / tau_rho)`` (binary) or
    ``scale_rho * exp(min(v - threshold, 0) / tau_rho)`` (graded).

    Parameters
    ----------
    voltage : torch tensor
    threshold : float or torch tensor
    tau_rho : float
    scale_rho : float
    graded_spike : bool
    voltage_last : torch tensor
        voltage at t = -1 (accepted for signature compatibility; the forward
        result does not depend on it).
    scale : int

    Examples
    --------
    >>> spike = Spike.apply(v, th, tau_rho, scale_rho, False, 0, 1)
    """

    derivative = None

    @staticmethod
    def forward(ctx, voltage, threshold, tau_rho, scale_rho, graded_spike, voltage_last, scale):
        graded = graded_spike is True
        spikes = _ops.spike_fwd(voltage, threshold, graded, scale)
        if torch.is_tensor(threshold):
            ctx.save_for_backward(voltage, threshold.detach())
            ctx.threshold = None
        else:
            ctx.save_for_backward(voltage)
            ctx.threshold = threshold
        ctx.consts = (float(tau_rho), float(scale_rho), graded)
        return spikes

    @staticmethod
    def backward(ctx, grad_spikes):
        voltage = ctx.saved_tensors[0]
        threshold = ctx.saved_tensors[1] if ctx.threshold is None else ctx.threshold
        tau_rho, scale_rho, graded = ctx.consts
        grad = _ops.spike_bwd(voltage, threshold, grad_spikes, tau_rho, scale_rho, graded)
        return grad, None, None, None, None, None, None
