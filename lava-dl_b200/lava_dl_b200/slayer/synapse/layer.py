"""Dense, convolution and sum-pooling synapses
(``src/lava/lib/dl/slayer/synapse/layer.py:9-508``): ``Conv3d`` with a time
kernel of 1, no bias, and an optional weight pre-hook (the 8-bit quantiser of
the neuron the synapse feeds)."""

import numpy as np
import torch
import torch.nn.functional as F

from ... import _ops


def _hw(value, what, third):
    """int or (h, w) -> (h, w, third)."""
    if isinstance(value, int):
        return (value, value, third)
    if len(value) == 2:
        return (value[0], value[1], third)
    raise Exception(f'{what} can be either int or tuple of size 2. Found {value}')


class GenericLayer(torch.nn.Module):
    """Weight-norm switch, gradient norm and the pre-hook shared by all synapses."""

    def __init__(self):
        super().__init__()
        self.weight_norm_enabled = False
        self.complex = False

    def enable_weight_norm(self):
        self = torch.nn.utils.weight_norm(self, name='weight')
        self.weight_norm_enabled = True

    def disable_weight_norm(self):
        torch.nn.utils.remove_weight_norm(self, name='weight')
        self.weight_norm_enabled = False

    @property
    def grad_norm(self):
        """Norm of the weight gradient per weight; 0 before the first backward."""
        w = self.weight_g if self.weight_norm_enabled else self.weight
        if w.grad is None:
            return 0
        return torch.norm(w.grad).item() / torch.numel(w.grad)

    @property
    def pre_hook_fx(self):
        return self._pre_hook_fx

    @pre_hook_fx.setter
    def pre_hook_fx(self, fx):
        self._pre_hook_fx = fx

    @property
    def shape(self):
        return self.weight.shape

    def _finish_init(self, weight_scale, weight_norm, pre_hook_fx):
        if weight_scale != 1:
            self.weight = torch.nn.Parameter(weight_scale * self.weight)
        self._pre_hook_fx = pre_hook_fx
        if weight_norm is True:
            self.enable_weight_norm()

    def _hooked_weight(self):
        return self.weight if self._pre_hook_fx is None else self._pre_hook_fx(self.weight)


class Dense(torch.nn.Conv3d, GenericLayer):
    """Fully connected synapse: a 1x1x1 convolution over ``NCT`` (or ``NCHWT``) input.

    Parameters
    ----------
    in_neurons : int or (w, h) or (w, h, c)
    out_neurons : int
    weight_scale : int
    weight_norm : bool
    pre_hook_fx : callable or None
    """

    def __init__(self, in_neurons, out_neurons, weight_scale=1, weight_norm=False, pre_hook_fx=None):
        if isinstance(in_neurons, int):
            kernel, in_channels = (1, 1, 1), in_neurons
        elif len(in_neurons) == 2:
            kernel, in_channels = (in_neurons[1], in_neurons[0], 1), 1
        elif len(in_neurons) == 3:
            kernel, in_channels = (in_neurons[1], in_neurons[0], 1), in_neurons[2]
        else:
            raise Exception(f'in_neurons should not be more than 3 dimension. Found {in_neurons}')
        if not isinstance(out_neurons, int):
            raise Exception(f'out_neurons should not be more than 1 dimension. Found {out_neurons}')
        super().__init__(in_channels, out_neurons, kernel, bias=False)
        self._finish_init(weight_scale, weight_norm, pre_hook_fx)

    def forward(self, input):
        weight = self._hooked_weight()
        if input.dim() == 3:
            n, t = input.shape[0], input.shape[-1]
            return F.conv3d(input.reshape(n, -1, 1, 1, t), weight, self.bias, self.stride, self.padding,
                            self.dilation, self.groups).reshape(n, -1, t)
        return F.conv3d(input, weight, self.bias, self.stride, self.padding, self.dilation, self.groups)


class _SpikeConv(torch.autograd.Function):
    """Forward, input gradient and weight gradient through the direct convolution
    kernels (time stays the vector axis, no layout change, fp32 throughout).  Shapes
    the weight-gradient kernel does not take go to ATen's convolution backward."""

    @staticmethod
    def forward(ctx, input, weight, padding):
        ctx.save_for_backward(input, weight)
        ctx.padding = tuple(padding)
        return _ops.conv_fwd(input, weight, padding)

    @staticmethod
    def backward(ctx, grad_output):
        input, weight = ctx.saved_tensors
        grad_output = grad_output.contiguous()
        kh, kw = weight.shape[2], weight.shape[3]
        # the input gradient is the forward kernel on the swapped problem (channels Co -> Ci, flipped
        # padding): it must pass that kernel's own limits, which a wide layer can meet forward only
        flipped = (kh - 1 - ctx.padding[0], kw - 1 - ctx.padding[1], 0)
        own_dgrad = flipped[0] >= 0 and flipped[1] >= 0 and _ops.conv_fwd_supported(
            grad_output, weight.transpose(0, 1), (1, 1, 1), flipped, (1, 1, 1), 1)
        own_wgrad = _ops.conv_wgrad_supported(input, weight, ctx.padding) and grad_output.data_ptr() % 16 == 0
        grad_input = grad_weight = None
        if ctx.needs_input_grad[0] and own_dgrad:
            grad_input = _ops.conv_dgrad(grad_output, weight, ctx.padding)
        if ctx.needs_input_grad[1] and own_wgrad:
            grad_weight = _ops.conv_wgrad(input, grad_output, weight.shape, ctx.padding)
        need = [ctx.needs_input_grad[0] and grad_input is None, ctx.needs_input_grad[1] and grad_weight is None, False]
        if need[0] or need[1]:
            gi, gw, _ = torch.ops.aten.convolution_backward(
                grad_output, input, weight, None, [1, 1, 1], list(ctx.padding), [1, 1, 1], False, [0, 0, 0], 1, need)
            grad_input = gi if need[0] else grad_input
            grad_weight = gw if need[1] else grad_weight
        return grad_input, grad_weight, None


class Conv(torch.nn.Conv3d, GenericLayer):
    """Spatial convolution synapse over ``NCHWT`` input (time kernel 1).
    ``kernel_size``, ``stride``, ``padding``, ``dilation``: int or (height, width)."""

    def __init__(self, in_features, out_features, kernel_size, stride=1, padding=0, dilation=1, groups=1,
                 weight_scale=1, weight_norm=False, pre_hook_fx=None):
        super().__init__(in_features, out_features, _hw(kernel_size, 'kernel_size', 1), _hw(stride, 'stride', 1),
                         _hw(padding, 'padding', 0), _hw(dilation, 'dilation', 1), groups, bias=False)
        self._finish_init(weight_scale, weight_norm, pre_hook_fx)

    def forward(self, input):
        weight = self._hooked_weight()
        if _ops.conv_fwd_supported(input, weight, self.stride, self.padding, self.dilation, self.groups):
            return _SpikeConv.apply(input, weight, self.padding)
        return F.conv3d(input, weight, self.bias, self.stride, self.padding, self.dilation, self.groups)


class _SumPool(torch.autograd.Function):
    """Sum pooling with stride = window through the gather-and-add kernel; the
    (fixed) pooling weights get no gradient."""

    @staticmethod
    def forward(ctx, input, weight):
        ctx.save_for_backward(weight)
        ctx.in_shape = tuple(input.shape)
        return _ops.pool_fwd(input, weight)

    @staticmethod
    def backward(ctx, grad_output):
        (weight,) = ctx.saved_tensors
        return _ops.pool_bwd(grad_output, weight, ctx.in_shape), None


class Pool(torch.nn.Conv3d, GenericLayer):
    """Sum pooling with a fixed all-``weight_scale`` kernel, applied per channel."""

    def __init__(self, kernel_size, stride=None, padding=0, dilation=1, weight_scale=1, weight_norm=False,
                 pre_hook_fx=None):
        kernel = _hw(kernel_size, 'kernel_size', 1)
        stride = kernel if stride is None else _hw(stride, 'stride', 1)
        super().__init__(1, 1, kernel, stride, _hw(padding, 'padding', 0), _hw(dilation, 'dilation', 1),
                         bias=False)
        self.weight = torch.nn.Parameter(
            torch.FloatTensor(weight_scale * np.ones(self.weight.shape)).to(self.weight.device),
            requires_grad=False)
        self._pre_hook_fx = pre_hook_fx
        if weight_norm is True:
            self.enable_weight_norm()

    def _plain_geometry(self):
        return (tuple(self.stride) == tuple(self.kernel_size) and tuple(self.padding) == (0, 0, 0)
                and tuple(self.dilation) == (1, 1, 1) and self.kernel_size[0] * self.kernel_size[1] <= 64)

    def forward(self, input):
        if input.is_cuda and input.dim() == 5 and self._plain_geometry() and not self.weight.requires_grad \
                and not self.weight_norm_enabled:
            return _SumPool.apply(input, self._hooked_weight())
        # the reference pads odd spatial sizes with (size % kernel) zero rows / columns
        # (synapse/layer.py:438-460); kept as is
        for dim in (2, 3):
            rem = input.shape[dim] % self.weight.shape[dim]
            if rem != 0:
                pad_shape = list(input.shape)
                pad_shape[dim] = rem
                input = torch.cat((input, torch.zeros(pad_shape, dtype=input.dtype, device=input.device)), dim)
        n, c, h, w, t = input.shape
        result = F.conv3d(input.reshape(n, 1, c * h, w, t), self._hooked_weight(), self.bias, self.stride,
                          self.padding, self.dilation)
        return result.reshape(result.shape[0], c, -1, result.shape[3], result.shape[4])
