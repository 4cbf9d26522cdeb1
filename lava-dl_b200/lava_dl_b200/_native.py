"""ctypes binding of ``libslayer_b200.so`` (declared in ``include/slayer_b200.h``).

There is no fallback: if the library cannot be loaded, or a call fails, a
``RuntimeError`` is raised.  Tensors cross the boundary as raw device pointers;
every call is launched on ``torch.cuda.current_stream()`` of the tensor's
device.
"""

import ctypes
import os
from ctypes import (POINTER, Structure, c_char_p, c_double, c_float, c_int,
                    c_int64, c_uint, c_void_p)

import torch

from . import _build

_lib = None


class Geom(Structure):
    """Mirror of ``sb_geom``."""
    _fields_ = [('rows', c_int64), ('T', c_int64),
                ('rows_per_batch', c_int64), ('decay_block', c_int64)]


_P = c_void_p
_G = POINTER(Geom)
_I64 = c_int64

# name -> (restype, argtypes); mirrors include/slayer_b200.h one to one
SIGNATURES = {
    'sb_version': (c_int, []),
    'sb_last_error_string': (c_char_p, []),
    'sb_device_status': (c_int, [POINTER(c_uint)]),
    'sb_param_grad_scratch_bytes': (c_int64, [_I64, _I64]),
    'sb_uses_tma': (c_int, [_P, _I64]),
    'sb_li_fwd': (c_int, [_P, _P, _I64, _P, _P, _P, _G, c_float, c_int, _P]),
    'sb_li_bwd': (c_int, [_P, _P, _P, _I64, _P, _P, _P, _G, _P]),
    'sb_li_bwd_noalloc': (c_int, [_P, _P, _P, _I64, _P, _P, _G, _P]),
    'sb_ath_fwd': (c_int, [_P, _P, _P, _I64, _P, _P, _I64, _P, _P, _G, c_int, c_int, c_int, _P]),
    'sb_apth_fwd': (c_int, [_P, _P, _P, _P, _P, _I64, _P, _P, _I64, _P, _P, _G, c_int, c_int, c_int, _P]),
    'sb_res_fwd': (c_int, [_P, _P, _P, _P, _I64, _P, _P, _P, _P, _G, c_int, c_float, c_int, c_int, _P]),
    'sb_res_bwd': (c_int, [_P, _P, _P, _P, _P, _P, _I64, _P, _P, _P, _P, _P, _P, _G, _P]),
    'sb_adres_fwd': (c_int, [_P, _P, _P, _P, _I64, _P, _I64, _P, _I64, _P, _P, _P, _P,
                             _P, _P, _P, _P, _G, c_int, c_int, c_int, _P]),
    'sb_spike_fwd': (c_int, [_P, _P, c_float, _P, _I64, c_int, c_float, _P]),
    'sb_spike_bwd': (c_int, [_P, _P, c_float, _P, _P, _I64, c_float, c_float, c_int, _P]),
    'sb_cspike_fwd': (c_int, [_P, _P, _P, c_float, _P, _P, _I64, _I64, c_int, c_float, _P]),
    'sb_cspike_bwd': (c_int, [_P, _P, _P, c_float, _P, _P, _P, _I64, c_float, c_float, c_int, _P]),
    'sb_cuba_fwd': (c_int, [_P, _P, _I64, _P, _I64, _P, _P, _P, _P, _P, _P, _P, _P, _G,
                            c_double, c_int, c_int, c_float, c_int, _P, _P, _I64, c_float, _P]),
    'sb_cuba_fwd_packed': (c_int, [_P, _P, _I64, _P, _I64, _P, _P, _P, _P, _P, _P, _P, _G,
                                   c_double, c_int, c_int, _P, _P]),
    'sb_cuba_bwd': (c_int, [_P, _P, _P, c_float, _P, _P, _I64, _P, _I64, _P, _P, _P, _P, _P, _G,
                            c_float, c_float, c_int, c_int, _P]),
    'sb_cuba_recurrent_fwd': (c_int, [_P, _P, _P, _I64, _P, _I64, _P, _P, _P, _P, _P, _P, _P,
                                      _I64, _I64, _I64, c_double, c_int, c_int, c_float, _P]),
    'sb_cuba_recurrent_bwd': (c_int, [_P, _P, _P, _P, _I64, _I64, _I64, c_float, c_float, c_float, c_int, _P]),
    'sb_alif_fwd': (c_int, [_P, _P, _I64, _P, _I64, _P, _I64, _P, _I64, _P, _P, _P, _P,
                            _P, _P, _P, _P, _P, _P, _P, _P, _P, _G,
                            c_int, c_int, c_int, c_int, c_int, c_float, c_int, _P, _P]),
    'sb_rf_fwd': (c_int, [_P, _P, _P, _P, _I64, _P, _I64, _P, _I64, _P, _P, _P, _P,
                          _P, _P, _P, _P, _P, _P, _P, _P, _P, _G,
                          c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, _P, _P]),
    'sb_rf_bwd': (c_int, [_P, _P, _P, _P, c_float, _P, _P, _I64, _P, _P, _P, _P, _P, _P, _G,
                          c_float, c_float, c_int, c_int, _P]),
    'sb_shift': (c_int, [_P, _P, _I64, c_float, c_float, _P, _I64, _I64, _P]),
    'sb_sigma_fwd': (c_int, [_P, _P, _P, _P, _I64, _I64, _P]),
    'sb_sigma_bwd': (c_int, [_P, _P, _I64, _I64, _P]),
    'sb_delta_fwd': (c_int, [_P, _P, _I64, _P, _P, _P, _P, _P, _G, c_double, _P]),
    'sb_delta_bwd': (c_int, [_P, _P, _P, _I64, _P, _P, _P, _G, c_float, c_float, _P]),
    'sb_sdnn_relu_fwd': (c_int, [_P, _P, _P, _I64, _P, _I64, _P, _P, _P, _P, _P, _P, _P, _P, _G, c_double, _P]),
    'sb_sdnn_relu_bwd': (c_int, [_P, _P, _P, _P, _I64, _P, _P, _P, _G, c_float, c_float, _P]),
    'sb_fir_conv': (c_int, [_P, _P, _I64, c_float, _P, _I64, _I64, _P]),
    'sb_fir_corr': (c_int, [_P, _P, _I64, c_float, _P, _I64, _I64, _P]),
    'sb_fir_uses_tensor_cores': (c_int, [_I64, _I64, _I64]),
    'sb_shift_fir_fwd': (c_int, [_P, _P, _I64, c_float, c_float, _P, _I64, c_float, _P, _I64, _I64, _P]),
    'sb_pool_fwd': (c_int, [_P, _P, _P, _I64, _I64, _I64, _I64, _I64, _I64, _I64, _I64, _P]),
    'sb_pool_bwd': (c_int, [_P, _P, _P, _I64, _I64, _I64, _I64, _I64, _I64, _I64, _I64, _P]),
    'sb_conv_fwd': (c_int, [_P, _P, _P] + [_I64] * 10 + [_P]),
    'sb_conv_fwd_path': (c_int, [_P, _P, _P] + [_I64] * 10 + [c_int, _P]),
    'sb_conv_uses_tensor_cores': (c_int, [_I64] * 10),
    'sb_conv_fits_tensor_cores': (c_int, [_I64] * 10),
    'sb_conv_wgrad_scratch_bytes': (_I64, [_I64] * 7),
    'sb_conv_wgrad': (c_int, [_P, _P, _P, _P] + [_I64] * 10 + [_P]),
    'sb_conv_wgrad_fits': (c_int, [_I64] * 10),
    'sb_unpack_spikes_host': (c_int, [_P, _P, _I64, _I64, c_int, c_int, _P]),
    'sb_broadcast_fill': (c_int, [_P, _P, _I64, _P]),
    'sb_shift_fir_bwd': (c_int, [_P, _P, _I64, c_float, c_float, _P, _I64, c_float, _P, _I64, _I64, _P]),
}


def lib_path():
    return os.environ.get('SLAYER_B200_LIB') or _build.LIB_PATH


def load():
    """Load (building first if the library file is absent) and return the CDLL."""
    global _lib
    if _lib is not None:
        return _lib
    path = os.environ.get('SLAYER_B200_LIB') or _build.LIB_PATH  # the variable points at an alternative build
    if not os.path.exists(path):
        if path != _build.LIB_PATH:
            raise RuntimeError(f'SLAYER_B200_LIB points at {path}, which does not exist')
        _build.build()
    try:
        lib = ctypes.CDLL(path)
    except OSError as e:
        raise RuntimeError(
            f'libslayer_b200.so could not be loaded from {path}: {e}. '
            f'Build it with `python -m lava_dl_b200._build`. '
            f'There is no CPU or PyTorch fallback.'
        ) from e
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means header/library mismatch
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def last_error():
    s = load().sb_last_error_string()
    return s.decode() if s else ''


def check(rc, name):
    if rc != 0:
        raise RuntimeError(f'{name} failed ({rc}): {last_error()}')


def ptr(t):
    """Device pointer of a tensor (``None`` -> NULL)."""
    if t is None:
        return None
    return c_void_p(t.data_ptr())


def stream_of(t):
    return c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def require_cuda(*tensors):
    """The kernels are the only implementation: refuse anything not on a GPU."""
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError(
                'lava_dl_b200 runs on CUDA tensors only (sm_100a kernels, no CPU '
                f'fallback); got a tensor on {t.device}.'
            )
        if t.dtype != torch.float32:
            raise TypeError(f'expected float32 tensors, got {t.dtype}')


def call(name, device_tensor, *args):
    """Invoke an entry point with ``device_tensor``'s device current."""
    lib = load()
    with torch.cuda.device(device_tensor.device):
        rc = getattr(lib, name)(*args)
    check(rc, name)


def device_status():
    bits = c_uint(0)
    check(load().sb_device_status(ctypes.byref(bits)), 'sb_device_status')
    return bits.value


def scratch(rows, n, device):
    """Scratch tensor for one parameter-gradient output."""
    nbytes = load().sb_param_grad_scratch_bytes(rows, n)
    return torch.empty(max(nbytes // 8, 1), dtype=torch.float64, device=device)
