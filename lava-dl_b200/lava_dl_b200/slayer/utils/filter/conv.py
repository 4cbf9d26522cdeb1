"""Causal convolution / correlation in time with one shared filter
(``src/lava/lib/dl/slayer/utils/filter/conv.py:100-223``).

``conv`` and ``corr`` are each other's adjoint, so each one's backward is the
other's forward; like the reference, no filter gradient is produced.
"""

import torch

from .... import _ops


def fwd(input, filter, sampling_time=1):
    """``out[t] = Ts * sum_i filter[i] * input[t - i]``"""
    return _ops.fir(input, filter, sampling_time, corr=False)


def bwd(input, filter, sampling_time=1):
    """``out[t] = Ts * sum_i filter[i] * input[t + i]``"""
    return _ops.fir(input, filter, sampling_time, corr=True)


class _Fir(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, filter, sampling_time, corr):
        ctx.save_for_backward(filter)
        ctx.sampling_time = sampling_time
        ctx.corr = corr
        return _ops.fir(input, filter, sampling_time, corr=corr)

    @staticmethod
    def backward(ctx, grad_output):
        (filter,) = ctx.saved_tensors
        if filter.requires_grad:
            print(('correlation' if ctx.corr else 'convolution') + ' filter gradient is not implemented.')
        grad_input = _ops.fir(grad_output, filter, ctx.sampling_time, corr=not ctx.corr)
        return grad_input, None, None, None


def conv(input, filter, sampling_time=1):
    """Convolution in time; output has the input's shape.

    Examples
    --------
    >>> output = conv(input, filter)
    """
    if input.dim() == 1:
        input = input.reshape(1, -1)
    return _Fir.apply(input, filter.flatten(), sampling_time, False)


def corr(input, filter, sampling_time=1):
    """Correlation in time; output has the input's shape.

    Examples
    --------
    >>> output = corr(input, filter)
    """
    if input.dim() == 1:
        input = input.reshape(1, -1)
    return _Fir.apply(input, filter.flatten(), sampling_time, True)
