"""Integer shift helpers (``src/lava/lib/dl/slayer/utils/int_utils.py:9-50``).

These are host-side conveniences on torch tensors of any device; the kernels
carry their own copy of the arithmetic.
"""

import torch


def right_shift_to_zero(x, bits):
    """Arithmetic right shift that rounds toward zero (sign-magnitude shift)."""
    if x.dtype not in (torch.int32, torch.int64):
        raise Exception(f'Expected torch.int32 or torch.int64 data, found {x.dtype}.')
    magnitude = torch.abs(x) >> bits
    return torch.where(x < 0, -magnitude, magnitude).to(x.dtype)


class Q2Zero(torch.autograd.Function):
    """Truncation toward zero with a straight-through gradient."""

    @staticmethod
    def forward(ctx, x):
        return torch.trunc(x).to(torch.int32).to(x.dtype)

    @staticmethod
    def backward(ctx, grad_output):
        return grad_output
