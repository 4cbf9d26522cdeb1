"""Axonal delay (``src/lava/lib/dl/slayer/axon/delay.py:12-221``): a shift in
time whose backward is the opposite shift; the learnable form also returns a
finite-difference gradient for the delays."""

import numpy as np
import torch

from .. import utils
from ... import _ops


class _DelayNoGrad(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, delay_val, sampling_time):
        ctx.delay_val = delay_val
        ctx.sampling_time = sampling_time
        return _ops.shift(input, delay_val, sampling_time)

    @staticmethod
    def backward(ctx, grad_output):
        back = -ctx.delay_val
        return _ops.shift(grad_output, back, ctx.sampling_time), None, None


class _DelayLearnable(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, delay_val, grad_scale, sampling_time):
        output = _ops.shift(input, delay_val.data, sampling_time)
        ctx.save_for_backward(output, delay_val.data)
        ctx.grad_scale = grad_scale
        ctx.sampling_time = sampling_time
        return output

    @staticmethod
    def backward(ctx, grad_output):
        output, delay_val = ctx.saved_tensors
        ts = ctx.sampling_time
        # d(output)/d(delay) ~ -(x[k] - x[k-1]) / Ts: a two-tap filter (delay.py:205-216)
        diff_filter = torch.tensor([-1, 1], dtype=grad_output.dtype, device=grad_output.device) / ts
        output_diff = _ops.fir(output, diff_filter, 1, corr=False)
        grad_delay = torch.sum(grad_output * output_diff, [0, -1], keepdim=True).reshape(
            grad_output.shape[1:-1]) * ts
        return _ops.shift(grad_output, -delay_val, ts), grad_delay * ctx.grad_scale, None, None


def delay_gradient(output, grad_output, sampling_time):
    """Finite-difference gradient of a delayed signal with respect to its per-neuron
    delays (delay.py:205-216), for callers that produced ``output`` themselves."""
    diff_filter = torch.tensor([-1, 1], dtype=grad_output.dtype, device=grad_output.device) / sampling_time
    output_diff = _ops.fir(output, diff_filter, 1, corr=False)
    return torch.sum(grad_output * output_diff, [0, -1], keepdim=True).reshape(grad_output.shape[1:-1]) * sampling_time


def delay(input, delay_val=1, sampling_time=1):
    """Delay the signal in time (last dimension).

    Examples
    --------
    >>> x_delayed = delay(x, 2)  # delay x by 2 timesteps
    """
    return _DelayNoGrad.apply(input, delay_val, sampling_time)


class Delay(torch.nn.Module):
    """Learnable per-channel axonal delay.

    Parameters
    ----------
    sampling_time : int
    max_delay : int or None
        upper clamp of the delays.
    grad_scale : float
        multiplier of the delay gradient.
    """

    def __init__(self, sampling_time=1, max_delay=None, grad_scale=1):
        super().__init__()
        self.sampling_time = sampling_time
        self.max_delay = max_delay
        self.grad_scale = grad_scale
        self.register_parameter('delay', torch.nn.Parameter(torch.FloatTensor([0]), requires_grad=True))
        self.init = False
        self.clamp()

    def clamp(self):
        """Clamp delays to ``[0, max_delay]``."""
        if self.init is True:
            if self.max_delay is None:
                self.delay.data.clamp_(0)
            else:
                self.delay.data.clamp_(0, self.max_delay)

    @property
    def shape(self):
        return self.delay.shape if self.init else None

    def delay_per_neuron(self, input):
        """Initialise on first use, clamp, and return one delay per neuron of
        ``input`` (the parameter itself, or expanded over the spatial dimensions)."""
        if self.init is False:
            if input.dim() <= 2:
                raise AssertionError(
                    f"Expected input to have at least 3 dimensions: [Batch, Spatial dims ..., Time]. "
                    f"It's shape is {input.shape}."
                )
            self.delay.data = torch.rand(input.shape[1], dtype=torch.float, device=input.device)
            self.init = True
        self.clamp()
        if self.shape[0] != input.shape[1]:
            raise AssertionError(
                f"Expected input to have same number of channels as delays. "
                f"Expected {self.shape[0]}, found {input.shape[1]}."
            )
        if np.prod(input.shape[1:-1]) == self.shape[0]:
            return self.delay
        tile = list(input.shape[1:-1])
        tile[0] = 1
        return self.delay.reshape(-1, *([1] * (len(tile) - 1))).repeat(tile)

    @property
    def fusable_steps(self):
        """Largest delay in time steps when it is bounded (``max_delay`` set), else ``None``:
        a bounded delay of at most 62 steps can be written by the neuron kernel itself."""
        if self.max_delay is None:
            return None
        return int(self.max_delay / self.sampling_time)

    def forward(self, input):
        delay_val = self.delay_per_neuron(input)
        return _DelayLearnable.apply(input, delay_val, self.grad_scale, self.sampling_time)
