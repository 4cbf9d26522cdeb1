"""B200-native implementation of lava-dl's SLAYER hot path.

``lava_dl_b200.slayer`` mirrors the part of ``lava.lib.dl.slayer`` that lies on
the path: ``neuron.{cuba,alif,rf,adrf}``, ``neuron.dynamics.*``, ``spike``,
``utils.time.shift``, ``utils.filter.{conv,corr,FIR}``, ``utils.quantize``,
``axon.delay``.  All arithmetic runs in hand-written sm_100a CUDA kernels behind
the C ABI declared in ``include/slayer_b200.h``; there is no CPU fallback.
"""

from . import slayer  # noqa: F401

__all__ = ['slayer']
