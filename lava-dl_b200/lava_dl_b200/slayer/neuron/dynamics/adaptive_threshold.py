"""Adaptive threshold and refractory dynamics
(``src/lava/lib/dl/slayer/neuron/dynamics/adaptive_threshold.py:51-274``)."""

import torch

from .... import _ops
from . import _debug


def dynamics(input, ref_state, ref_decay, th_state, th_decay, th_scale, th0, w_scale, debug=False):
    """Threshold and refractory traces driven by the spikes of ``input``.

    .. math::
        \\vartheta[t] &= (1-\\alpha_{\\vartheta})\\,(\\vartheta[t-1] - \\vartheta_0) + \\vartheta_0 \\

        r[t] &= (1-\\alpha_r)\\,r[t-1] \\

        s[t] &= (x[t] - r[t]) \\geq \\vartheta[t] \\

        r[t] &= r[t] + 2\\,\\vartheta[t] \\

        \\vartheta[t] &= \\vartheta[t] + \\vartheta_{\\text{step}}

    Returns ``(threshold, refractory)``; no gradient flows through this op.

    ``debug=True`` does not run a second implementation (there is none to compare with): it checks that the
    scaled states are integers below 2^30 in magnitude and that the device status word is clean.
    """
    threshold, refractory = _ATHDynamics.apply(
        input, ref_state, ref_decay, th_state, th_decay, th_scale, th0, w_scale)
    if debug:
        _debug.check_quantised(w_scale, threshold=threshold, refractory=refractory)
    return threshold, refractory


class _ATHDynamics(torch.autograd.Function):
    """No gradient flows through this op; like the reference
    (``adaptive_threshold.py:230-234``) the backward hands ``None`` to every
    input, which autograd turns into zero gradients for learnable decays."""

    @staticmethod
    def forward(ctx, input, ref_state, ref_decay, th_state, th_decay, th_scale, th0, w_scale):
        return _ops.ath_fwd(input, ref_state, ref_decay, th_state, th_decay, th_scale, th0, w_scale)

    @staticmethod
    def backward(*_):
        return (None,) * 8


def persistent_ref_state(ref_state, spike, th_state):
    """Refractory state to carry over when the last time bin spiked."""
    spike = (spike > 0).to(ref_state.dtype)
    return ref_state + 2 * spike * th_state


def persistent_th_state(th_state, spike, th_step):
    """Threshold state to carry over when the last time bin spiked."""
    spike = (spike > 0).to(th_state.dtype)
    return th_state + spike * th_step
