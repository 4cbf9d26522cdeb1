"""The C-ABI library: it loads without a GPU, exports exactly what
include/slayer_b200.h declares, and the ctypes binding covers every symbol.
No compute call is made here."""

import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, 'include', 'slayer_b200.h')


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r'/\*.*?\*/', '', text, flags=re.S)
    return sorted(set(re.findall(r'\b(sb_[a-z0-9_]+)\s*\(', text)))


@pytest.fixture(scope='module')
def lib():
    from lava_dl_b200 import _build
    path = _build.build()  # no-op when the library is up to date
    return ctypes.CDLL(path)


def test_header_declares_entry_points():
    syms = declared_symbols()
    assert len(syms) >= 25
    for must in ('sb_li_fwd', 'sb_li_bwd', 'sb_cuba_fwd', 'sb_cuba_bwd', 'sb_shift', 'sb_fir_conv', 'sb_fir_corr',
                 'sb_spike_fwd', 'sb_res_fwd', 'sb_res_bwd', 'sb_ath_fwd', 'sb_apth_fwd', 'sb_adres_fwd'):
        assert must in syms


def test_library_exports_every_declared_symbol(lib):
    missing = [s for s in declared_symbols() if not hasattr(lib, s)]
    assert not missing, f'declared in the header but not exported: {missing}'


def test_binding_matches_header():
    from lava_dl_b200 import _native
    assert sorted(_native.SIGNATURES) == declared_symbols()


def test_version_and_error_string(lib):
    lib.sb_version.restype = ctypes.c_int
    assert lib.sb_version() >= 100
    lib.sb_last_error_string.restype = ctypes.c_char_p
    assert lib.sb_last_error_string() is not None


def test_scratch_size_is_pure_arithmetic(lib):
    fn = lib.sb_param_grad_scratch_bytes
    fn.restype = ctypes.c_int64
    fn.argtypes = [ctypes.c_int64, ctypes.c_int64]
    shared = fn(1 << 20, 1)
    per_channel = fn(1 << 20, 512)
    assert shared >= ((1 << 20) // 32) * 8
    assert per_channel >= (1 << 20) * 8
    assert fn(0, 1) >= 0


def test_argument_errors_are_reported_without_a_gpu(lib):
    """Validation happens before any CUDA call, so bad arguments are rejected
    (not crashed on) even on a machine without a device."""
    from lava_dl_b200 import _native
    native = _native.load()
    g = _native.Geom(-1, 8, 1, 1)
    rc = native.sb_li_fwd(None, None, 1, None, None, None, ctypes.byref(g), 0.0, 4096, None)
    assert rc == -1
    assert 'geometry' in _native.last_error()
    g = _native.Geom(4, 8, 1, 1)
    rc = native.sb_cuba_fwd(None, None, 1, None, 1, None, None, None, None, None, None, None, None,
                            ctypes.byref(g), 1.25, 1000, 0, 1.0, 0, None, None, 0, 1.0, None)
    assert rc == -1 and 'power-of-two' in _native.last_error()
    rc = native.sb_fir_conv(None, None, 0, 1.0, None, 4, 8, None)
    assert rc == -1 and 'filter length' in _native.last_error()
