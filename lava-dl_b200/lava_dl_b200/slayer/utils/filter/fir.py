"""Fixed finite-impulse-response filter module
(``src/lava/lib/dl/slayer/utils/filter/fir.py:13-54``)."""

import numpy as np
import torch

from .conv import conv


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
