"""Shift along the time axis (``src/lava/lib/dl/slayer/utils/time/shift.py:94-143``).

One kernel launch covers every batch element and both the scalar and the
per-neuron form.  The shift count is ``int(shift / sampling_time)`` (truncation
toward zero), which is what the reference's scalar path and CUDA path compute;
its CPU per-neuron loop divides by ``sampling_time`` twice
(``shift.py:82,87-88``), equal only for ``sampling_time == 1``.
"""

from .... import _ops


def shift(input, shift_val, sampling_time=1):
    """``output[..., t] = input[..., t - shift]`` with zero fill.

    Parameters
    ----------
    input : torch tensor
        CUDA tensor, time last.
    shift_val : torch tensor or float or int
        scalar (same shift everywhere) or a tensor whose element count equals
        the number of neurons ``prod(input.shape[1:-1])``.
    sampling_time : float
        sampling time. Defaults to 1.

    Examples
    --------
    >>> output = shift(input, 7)
    >>> output = shift(torch.rand(1, 10, 100).cuda(), torch.arange(10).cuda())
    """
    return _ops.shift(input, shift_val, sampling_time)
