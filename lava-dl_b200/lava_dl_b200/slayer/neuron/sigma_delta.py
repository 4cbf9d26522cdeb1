"""Sigma-delta neuron (``src/lava/lib/dl/slayer/neuron/sigma_delta.py:13-240``):
sigma decoder -> (normalisation) -> bias -> activation -> delta encoder."""

import math

import torch

from . import base
from ..dendrite import Sigma
from ..axon import Delta
from ... import _ops


class _SdnnRelu(torch.autograd.Function):
    """Sigma -> bias -> ReLU -> delta -> floor as one kernel each way."""

    @staticmethod
    def forward(ctx, input, threshold, bias, sigma_state, pre_state, residual_state, scale, tau_grad, scale_grad):
        need_tgrad = ctx.needs_input_grad[1]
        need_grad = need_tgrad or ctx.needs_input_grad[0]
        r = _ops.sdnn_relu_fwd(input, threshold, bias, sigma_state, pre_state, residual_state, scale,
                               want_act=need_grad, want_delta=need_tgrad)
        if need_grad:
            ctx.save_for_backward(threshold, r['activation'], *([r['delta_input']] if need_tgrad else []))
        ctx.consts = (tau_grad, scale_grad, need_tgrad)
        ctx.mark_non_differentiable(r['final_sigma'], r['final_pre'], r['final_residual'])
        return r['out'], r['final_sigma'], r['final_pre'], r['final_residual']

    @staticmethod
    def backward(ctx, grad_out, *_):
        tau_grad, scale_grad, need_tgrad = ctx.consts
        threshold, activation = ctx.saved_tensors[:2]
        delta_input = ctx.saved_tensors[2] if need_tgrad else None
        gx, gthr = _ops.sdnn_relu_bwd(grad_out, activation, delta_input, threshold, tau_grad, scale_grad, need_tgrad)
        return (gx, gthr) + (None,) * 7


def neuron_params(device_params, scale=1 << 6):
    """Translate device parameters to neuron parameters."""
    return {'threshold': device_params['vThMant'] / scale}


class Neuron(base.Neuron):
    """Sigma-delta wrapper around an activation function.

    Parameters
    ----------
    threshold : float
        delta threshold.
    activation : callable
        activation wrapped by the sigma-delta unit, e.g. ``torch.nn.functional.relu``.
    tau_grad, scale_grad : float
        relaxation and scale of the threshold gradient. Default 1.
    scale : int
        scale of the internal state. Defaults to ``1 << 6``.
    cum_error : bool
        see ``axon.Delta``. Defaults to False.
    norm, dropout : callable or None
    shared_param, persistent_state, requires_grad : bool

    With ``relu``, no normalisation, no dropout and no learnable bias the whole neuron
    runs as one kernel each way (8 bytes per step without gradients, 12 with).
    """

    def __init__(self, threshold, activation, tau_grad=1, scale_grad=1, scale=1 << 6, cum_error=False, norm=None,
                 dropout=None, shared_param=True, persistent_state=False, requires_grad=False):
        super().__init__(threshold=threshold, w_scale=scale, s_scale=scale * (1 << 6), norm=norm, dropout=dropout,
                         persistent_state=persistent_state, shared_param=shared_param, requires_grad=requires_grad)
        self.graded_spike = True
        self.activation = activation
        self.sigma = Sigma(persistent_state=self.persistent_state)
        self.delta = Delta(threshold=self._threshold, scale=self.s_scale, tau_grad=tau_grad, scale_grad=scale_grad,
                           cum_error=cum_error, shared_param=self.shared_param,
                           persistent_state=self.persistent_state, requires_grad=self.requires_grad)
        self.bias_is_set = False
        self.register_parameter('bias', torch.nn.Parameter(torch.FloatTensor([0]), requires_grad=self.requires_grad))

    @property
    def device(self):
        return self.delta.pre_state.device

    @property
    def threshold(self):
        return self.delta.threshold

    @property
    def scale(self):
        return self.w_scale

    @property
    def v_th_mant(self):
        return int(self.delta.threshold.item() * self.w_scale)

    @property
    def device_params(self):
        return {'type': 'SDNN', 'activation': self.activation.__name__, 'vThMant': self.v_th_mant}

    def set_bias(self, bias):
        """Set one bias per neuron."""
        if self.shape is None:
            self.bias.data = bias.to(self.bias.device)
        else:
            self.bias.data = bias.reshape(self.shape).to(self.bias.device)
        self.bias_is_set = True

    def _one_pass(self, input):
        """True when sigma -> bias -> relu -> delta can run as one kernel each way."""
        if self.activation is not torch.nn.functional.relu or self.norm is not None or self.drop is not None:
            return False
        if self.bias_is_set and torch.is_grad_enabled() and self.bias.requires_grad:
            return False    # the fused backward has no bias gradient
        if self.bias_is_set and self.bias.numel() not in (1, math.prod(input.shape[1:-1])):
            return False
        return True

    def forward(self, input):
        """Graded-spike response of the neuron to ``input`` (``[batch, ..., time]``)."""
        if self._one_pass(input):
            self.sigma._check(input)
            self.delta._check(input)
            self.delta.clamp()
            persistent = self.persistent_state is True
            axon, final_sigma, final_pre, final_residual = _SdnnRelu.apply(
                input, self.delta.threshold, self.bias if self.bias_is_set else None,
                self.sigma.pre_state if persistent else None, self.delta.pre_state if persistent else None,
                self.delta.residual_state if persistent else None, self.delta.scale, self.delta.tau_grad,
                self.delta.scale_grad)
            if persistent:
                self.sigma.pre_state = final_sigma.detach()
                self.delta.pre_state = final_pre.detach()
                self.delta.residual_state = final_residual.detach()
        else:
            dend = self.sigma(input)
            if self.norm is not None:
                dend = self.norm(dend)
            if self.bias_is_set:
                dend = dend + torch.unsqueeze(torch.unsqueeze(self.bias, dim=0), dim=-1)
            axon = self.delta(self.activation(dend))
            if self.drop is not None:
                axon = self.drop(axon)
        if self.shape is None:
            if self.sigma.shape != self.delta.shape:
                raise AssertionError(
                    f'The shape of sigma and delta do not match. '
                    f'Found {self.sigma.shape=} and {self.delta.shape=}.'
                )
            self.shape = self.sigma.shape
        return axon
