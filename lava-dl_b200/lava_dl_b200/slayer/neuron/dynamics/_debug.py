"""``debug=True`` support for the dynamics functions.

In the reference ``debug`` runs the Python loop and the CUDA kernel and compares
them (``leaky_integrator.py:134-155``).  There is a single implementation here,
so the flag instead checks invariants of the result: the scaled states are
integers and the device reported no fault.
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
