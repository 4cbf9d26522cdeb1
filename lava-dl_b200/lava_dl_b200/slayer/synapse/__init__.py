"""Synapses (mirror of ``lava.lib.dl.slayer.synapse``: dense, convolution and sum-pooling,
real and complex).

They are the producers of the hot path's input: ``torch.nn.Conv3d`` subclasses with a unit time
kernel, as in the reference (``src/lava/lib/dl/slayer/synapse/layer.py``), whose pooling and
convolution run on this library's own kernels (``sb_pool_fwd``, ``sb_conv_fwd`` on the tensor
cores) where the geometry allows.  They exist so that the blocks, and through them whole
networks, can be assembled around the neuron kernels.
"""

from . import complex
from .layer import Dense, Conv, Pool

__all__ = ['Dense', 'Conv', 'Pool', 'complex']
