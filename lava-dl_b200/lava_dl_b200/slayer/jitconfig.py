"""Kept for API compatibility with ``lava.lib.dl.slayer.jitconfig``
(``src/lava/lib/dl/slayer/jitconfig.py:9-18``).

Nothing is JIT-compiled here: the kernels are built ahead of time for sm_100a,
so ``TORCH_CUDA_ARCH_LIST`` is ignored.  ``VERBOSE`` makes the native loader
print the library path on first use.
"""

TORCH_CUDA_ARCH_LIST = None
VERBOSE = False
