"""Finite-impulse-response filter modules
(``src/lava/lib/dl/slayer/utils/filter/fir.py:13-100``)."""

import numpy as np
import torch

from .conv import conv
from .... import _ops


class FIR(torch.nn.Module):
    """Non-learnable FIR filter applied along time.

    Parameters
    ----------
    fir_response : array, optional
        impulse response; an exponential ``exp(-t / time_constant)`` of
        ``length`` taps when ``None``.
    time_constant : float
    length : int
    sampling_time : float
    """

    def __init__(self, fir_response=None, time_constant=1, length=20, sampling_time=1):
        super().__init__()
        if fir_response is None:
            fir_response = np.exp(-np.arange(length) / time_constant)
        self.register_buffer('filter', torch.FloatTensor(fir_response))
        self.sampling_time = sampling_time

    def forward(self, input):
        return conv(input, self.filter, self.sampling_time)


class _BankFn(torch.autograd.Function):
    """``out[b, f * C + c, ..., t] = Ts * sum_j h[f, j] * x[b, c, ..., t - j]`` for every filter f of the
    bank, ``h[f, j] = weight[f, K - 1 - j]`` (the reference applies ``conv3d``, a correlation, to the
    input padded with ``K - 1`` zeros on the left).  Each filter is one pass of the temporal filter
    kernel; the input gradient is the sum of the adjoint passes; the weight gradient is one
    dot product per filter and lag."""

    @staticmethod
    def forward(ctx, input, weight, sampling_time):
        ctx.save_for_backward(input, weight)
        ctx.sampling_time = sampling_time
        taps = weight.detach().flip(-1)
        outs = [_ops.fir(input, taps[f], sampling_time, corr=False) for f in range(weight.shape[0])]
        return torch.cat(outs, dim=1)

    @staticmethod
    def backward(ctx, grad_output):
        input, weight = ctx.saved_tensors
        F, K = weight.shape
        C = input.shape[1]
        T = input.shape[-1]
        taps = weight.detach().flip(-1)
        grad_input = grad_weight = None
        if ctx.needs_input_grad[0]:
            for f in range(F):
                g = _ops.fir(grad_output[:, f * C:(f + 1) * C], taps[f], ctx.sampling_time, corr=True)
                grad_input = g if grad_input is None else grad_input + g
        if ctx.needs_input_grad[1]:
            # d out[t] / d weight[f, k] = Ts * x[t - (K - 1 - k)]
            x = input.reshape(input.shape[0], C, -1, T)
            g = grad_output.reshape(input.shape[0], F, C, -1, T)
            grad_weight = torch.zeros_like(weight)
            for lag in range(min(K, T)):
                gw = torch.einsum('bfcnt,bcnt->f', g[..., lag:], x[..., :T - lag])
                grad_weight[:, K - 1 - lag] = gw * ctx.sampling_time
        return grad_input, grad_weight, None


class FIRBank(torch.nn.Conv3d):
    """Bank of learnable FIR filters applied along time
    (``src/lava/lib/dl/slayer/utils/filter/fir.py:57-100``).  It keeps the reference's
    parameter (a ``Conv3d`` weight ``[num_filter, 1, 1, 1, K]`` with the default initialisation, so
    state dicts are interchangeable) and output layout (``[B, num_filter * C, ..., T]``, filter
    major); the arithmetic runs on the temporal filter kernel instead of ``F.conv3d``.

    Parameters
    ----------
    num_filter : int
    filter_length : float
        time length of the filters; ``int(filter_length / sampling_time)`` taps.
    sampling_time : float
    scale : float
        factor applied to the initial weights.
    """

    def __init__(self, num_filter, filter_length, sampling_time=1, scale=1):
        super().__init__(1, num_filter, (1, 1, int(filter_length / sampling_time)), bias=False)
        self.sampling_time = sampling_time
        # the reference pads with filter_length - 1 zeros whatever the sampling time; the output
        # keeps the input's length only when that equals the number of taps minus one
        self.pad_steps = filter_length - 1
        if scale != 1:
            self.weight.data *= scale

    def forward(self, input):
        K = self.weight.shape[-1]
        if self.pad_steps != K - 1:
            raise ValueError(
                f'FIRBank: {K} taps with a left padding of {self.pad_steps} steps change the length of the '
                f'signal (the reference then fails to reshape its output); use sampling_time = 1')
        return _BankFn.apply(input, self.weight.reshape(self.weight.shape[0], K), self.sampling_time)

    @property
    def num_filter(self):
        """Number of filters in the bank."""
        return self.out_channels
