"""``debug=True`` support for the dynamics functions.

In the reference ``debug`` runs the Python loop and the CUDA kernel and compares
them (``leaky_integrator.py:134-155``).  There is a single implementation here,
so the flag instead checks invariants of the result: the scaled states are
integers, they stay clear of the int32 range the kernels keep them in, and the
device reported no fault.

The reference's CPU path holds states as int64; the kernels hold them as int32
(as the reference's own CUDA kernels do) and are exact while every state stays
below 2^31 in magnitude.  Loihi states are 24 bit, so a network on the Loihi
grid never comes near; an unbounded recurrence (a voltage without reset driven
hard for a long time, a decay outside [0, 4096] that makes the state grow) can.
A wrap cannot be seen after the fact, so the check is a margin: any scaled
state at or beyond 2^30 raises.
"""

import torch

from .... import _native


def check_quantised(w_scale, **series):
    status = _native.device_status()
    if status:
        raise RuntimeError(f'device status word is {status:#x} after a dynamics kernel')
    for name, t in series.items():
        scaled = t.detach() * w_scale
        if not torch.equal(scaled, torch.round(scaled)):
            raise RuntimeError(f'{name} * w_scale is not integer valued')
        if scaled.numel() and float(scaled.abs().max()) >= float(1 << 30):
            raise RuntimeError(
                f'{name} * w_scale reaches {float(scaled.abs().max()):.4g}: within a factor of two of the int32 '
                f'range of the kernel states (the int64 reference would not wrap there)')
