"""Delta encoder (``src/lava/lib/dl/slayer/axon/delta.py:10-320``): thresholded
temporal difference with a residual, one scan kernel each way instead of the
reference's Python loop over time."""

import torch

from ... import _ops


class _DeltaUnit(torch.autograd.Function):
    """``delta.py:10-122`` plus the floor quantisation of ``Delta.forward``
    (``delta.py:316``), whose gradient is the identity."""

    @staticmethod
    def forward(ctx, input, threshold, pre_state, residual_state, scale, tau_grad, scale_grad):
        need_tgrad = ctx.needs_input_grad[1]
        out, delta_input, residual = _ops.delta_fwd(input, threshold, pre_state, residual_state, scale,
                                                    want_delta=need_tgrad)
        ctx.save_for_backward(threshold, *([delta_input] if need_tgrad else []))
        ctx.consts = (tau_grad, scale_grad, need_tgrad)
        ctx.mark_non_differentiable(residual)
        return out, residual

    @staticmethod
    def backward(ctx, grad_output, _):
        tau_grad, scale_grad, need_tgrad = ctx.consts
        threshold = ctx.saved_tensors[0]
        delta_input = ctx.saved_tensors[1] if need_tgrad else None
        gx, gthr = _ops.delta_bwd(grad_output, delta_input, threshold, tau_grad, scale_grad, need_tgrad)
        return gx, gthr, None, None, None, None, None


class Delta(torch.nn.Module):
    """Delta differential encoding followed by thresholding; the thresholds are
    learnable, individually or as a group.

    .. math::
        \\Delta x[t] &= x[t] - x[t-1] + r[t-1] \\\\
        y[t] &= \\Delta x[t] \\text{ if } |\\Delta x[t]| \\geq \\vartheta \\text{ else } 0 \\\\
        r[t] &= \\Delta x[t] - y[t]

    Parameters
    ----------
    threshold : float
    scale : int
        quantisation step is ``1 / scale``. Defaults to 64.
    tau_grad, scale_grad : float
        relaxation and scale of the threshold gradient. Default 1.
    cum_error : bool
        cumulative-error thresholding. Not available: the reference's own loop for
        it (``delta.py:30-43``) raises with current PyTorch (``1 - bool tensor``).
    shared_param : bool
        one threshold for the group (else one per channel). Defaults to True.
    persistent_state : bool
        keep ``x[t-1]`` and the residual between calls. Defaults to False.
    requires_grad : bool
        learnable threshold. Defaults to False.
    """

    def __init__(self, threshold, scale=(1 << 6), tau_grad=1, scale_grad=1, cum_error=False, shared_param=True,
                 persistent_state=False, requires_grad=False):
        super().__init__()
        if cum_error:
            raise NotImplementedError(
                'cum_error=True is not implemented: the reference implementation of that mode fails in '
                'PyTorch >= 1.2 (subtraction from a bool tensor, axon/delta.py:41)')
        self.scale = scale
        self.tau_grad = tau_grad
        self.scale_grad = scale_grad
        self.cum_error = cum_error
        self.shared_param = shared_param
        self.persistent_state = persistent_state
        self.requires_grad = requires_grad
        self.shape = None
        for name in ('pre_state', 'residual_state', 'error_state'):
            self.register_buffer(name, torch.zeros(1, dtype=torch.float), persistent=False)
        self.register_parameter('threshold', torch.nn.Parameter(torch.FloatTensor([threshold]),
                                                                requires_grad=self.requires_grad))

    def clamp(self):
        """Clamp the threshold to ``[1 / scale, inf)``."""
        self.threshold.data.clamp_(1 / self.scale)

    @property
    def device(self):
        return self.threshold.device

    def _check(self, input):
        if self.shape is None:
            self.shape = input.shape[1:-1]
            if len(self.shape) == 0:
                raise AssertionError(
                    f"Expected input to have at least 3 dimensions: [Batch, Spatial dims ..., Time]. "
                    f"It's shape is {input.shape}."
                )
            if self.shared_param is False:
                self.threshold.data = self.threshold.data * torch.ones(self.shape[0]).to(self.device)
                self.threshold.data = self.threshold.data.reshape([self.shape[0]] + [1 for _ in self.shape[1:]])
        elif input.shape[1:-1] != self.shape:
            raise AssertionError(
                f'Input tensor shape ({input.shape}) does not match withNeuron shape ({self.shape}).'
            )
        if self.pre_state.shape[0] != input.shape[0]:
            for name in ('pre_state', 'error_state', 'residual_state'):
                old = getattr(self, name)
                setattr(self, name, torch.zeros(input.shape[:-1], dtype=old.dtype, device=old.device))

    def forward(self, input):
        self._check(input)
        self.clamp()
        persistent = self.persistent_state is True
        output, residual = _DeltaUnit.apply(
            input, self.threshold, self.pre_state if persistent else None,
            self.residual_state if persistent else None, self.scale, self.tau_grad, self.scale_grad)
        if persistent:
            self.pre_state = input[..., -1].clone().detach()
            self.residual_state = residual.detach()
        return output
