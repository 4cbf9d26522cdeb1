"""Adaptive phase-threshold and refractory dynamics
(``src/lava/lib/dl/slayer/neuron/dynamics/adaptive_phase_th.py:51-283``)."""

import torch

from .... import _ops
from . import _debug


def dynamics(re_input, im_input, im_state, ref_state, ref_decay, th_state, th_decay, th_scale, th0, w_scale,
             debug=False):
    """Threshold and refractory traces of a resonator that spikes when the real
    part exceeds ``threshold + refractory`` while the imaginary part crosses
    zero upwards.  Returns ``(threshold, refractory)``; no gradient.

    ``debug=True`` does not run a second implementation (there is none to compare with): it checks that the
    scaled states are integers below 2^30 in magnitude and that the device status word is clean.
    """
    threshold, refractory = _APTHDynamics.apply(
        re_input, im_input, im_state, ref_state, ref_decay, th_state, th_decay, th_scale, th0, w_scale)
    if debug:
        _debug.check_quantised(w_scale, threshold=threshold, refractory=refractory)
    return threshold, refractory


class _APTHDynamics(torch.autograd.Function):
    """No gradient flows through this op (``adaptive_phase_th.py:227-231``)."""

    @staticmethod
    def forward(ctx, re_input, im_input, im_state, ref_state, ref_decay, th_state, th_decay, th_scale, th0,
                w_scale):
        return _ops.apth_fwd(re_input, im_input, im_state, ref_state, ref_decay, th_state, th_decay, th_scale,
                             th0, w_scale)

    @staticmethod
    def backward(*_):
        return (None,) * 10


def persistent_ref_state(ref_state, spike, th_state):
    """Refractory state to carry over when the last time bin spiked."""
    spike = (spike > 0).to(ref_state.dtype)
    return ref_state + 2 * spike * th_state


def persistent_th_state(th_state, spike, th_step):
    """Threshold state to carry over when the last time bin spiked."""
    spike = (spike > 0).to(th_state.dtype)
    return th_state + spike * th_step
