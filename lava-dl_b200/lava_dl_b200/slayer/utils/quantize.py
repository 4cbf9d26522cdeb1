"""Parameter quantisation with straight-through gradient
(``src/lava/lib/dl/slayer/utils/quantize.py:11-115``)."""

from enum import IntEnum, unique

import torch


@unique
class MODE(IntEnum):
    """Quantisation mode: ``ROUND`` (0) or ``FLOOR`` (1)."""
    ROUND = 0
    FLOOR = 1


class _StraightThrough(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, step, floor):
        if step == 1:
            # x / 1 and y * 1 are identities in fp32: one kernel instead of three (the neuron classes
            # quantise every decay with step 1 on every call)
            return torch.floor(input) if floor else torch.round(input)
        scaled = input / step
        return (torch.floor(scaled) if floor else torch.round(scaled)) * step

    @staticmethod
    def backward(ctx, grad_output):
        return grad_output, None, None


def quantize(input, step=1, mode=MODE.ROUND):
    """Round (or floor) ``input`` to multiples of ``step``; gradient passes unchanged."""
    if mode == MODE.ROUND:
        return _StraightThrough.apply(input, step, False)
    if mode == MODE.FLOOR:
        return _StraightThrough.apply(input, step, True)
    raise ValueError(f'{mode=} is not recognized.')


def quantize_hook_fx(x, scale=(1 << 6), num_bits=8, descale=False):
    """Synapse pre-hook: quantise weights in steps of ``2 / scale`` and clamp to
    the ``num_bits`` range (optionally returned as integers)."""
    lo = -2 * (1 << num_bits)
    hi = 2 * ((1 << num_bits) - 1)
    q = quantize(x, step=2 / scale).clamp(lo / scale, hi / scale)
    return q * scale if descale else q
