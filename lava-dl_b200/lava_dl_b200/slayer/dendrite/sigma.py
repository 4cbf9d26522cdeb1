"""Sigma decoder (``src/lava/lib/dl/slayer/dendrite/sigma.py:9-77``): a running
sum over time, as one scan kernel each way instead of ``torch.cumsum``."""

import torch

from ... import _ops


class _Sigma(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, state):
        out, final = _ops.sigma_fwd(input, state, want_final=True)
        ctx.mark_non_differentiable(final)
        return out, final

    @staticmethod
    def backward(ctx, grad_output, _):
        return _ops.sigma_bwd(grad_output), None


class Sigma(torch.nn.Module):
    """Sigma decoder: ``output[t] = sum of input up to t`` (plus what the previous
    call left when ``persistent_state``).

    Parameters
    ----------
    persistent_state : bool
        keep the running sum between calls. Defaults to False.
    """

    def __init__(self, persistent_state=False):
        super().__init__()
        self.persistent_state = persistent_state
        self.shape = None
        self.register_buffer('pre_state', torch.zeros(1, dtype=torch.float), persistent=False)

    def _check(self, input):
        if self.shape is None:
            self.shape = input.shape[1:-1]
            if len(self.shape) == 0:
                raise AssertionError(
                    f"Expected input to have at least 3 dimensions: [Batch, Spatial dims ..., Time]. "
                    f"It's shape is {input.shape}."
                )
        elif input.shape[1:-1] != self.shape:
            raise AssertionError(
                f'Input tensor shape ({input.shape}) does not match with Neuron shape ({self.shape}).'
            )
        if self.pre_state.shape[0] != input.shape[0]:
            # batch size changed: the kept state cannot be continued
            self.pre_state = torch.zeros(input.shape[:-1], dtype=self.pre_state.dtype, device=self.pre_state.device)

    def forward(self, input):
        self._check(input)
        output, final = _Sigma.apply(input, self.pre_state if self.persistent_state else None)
        if self.persistent_state is True:
            self.pre_state = final.detach()
        return output

    @property
    def device_params(self):
        """Dictionary of device parameters."""
        return {'type': 'SDNN', 'sigma_output': True}
