"""Utilities on the hot path (mirror of ``lava.lib.dl.slayer.utils``)."""

from . import filter, time, int_utils, recurrent  # noqa: F401
from .quantize import quantize, quantize_hook_fx
from .quantize import MODE as QUANTIZE_MODE
from ..._ops import unpack_spikes
from .graphed import Graphed

__all__ = ['filter', 'time', 'int_utils', 'recurrent', 'quantize', 'quantize_hook_fx', 'QUANTIZE_MODE', 'unpack_spikes', 'Graphed']
