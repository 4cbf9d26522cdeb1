"""sb_li_bwd_noalloc: the entry point for hosts that cannot hand the library a
scratch buffer because they cannot allocate device memory (runtimes that plan
memory ahead of time and pass a custom op only inputs and outputs, processes
whose pool already owns the GPU).  Its scratch is an array inside the library,
so consecutive calls reuse the same memory with the previous call's contents
still in it.

Checked here, through the C ABI: calls in a row (shared and per-channel decays,
on the TMA kernels and on the plain-load ones, each reading slots the previous
call left dirty) agree with sb_li_bwd given fresh caller scratch and with the
CPU oracle; the largest problems the array holds are accepted and correct, the
next larger ones are refused.  The file name sorts last on purpose: a run that
stops at the first failure has already run every other test.
"""

import ctypes

import numpy as np
import pytest
import torch

from _util import assert_close, assert_exact, li_scale, pgrad_scale

pytestmark = pytest.mark.gpu


def _run(native, ops, cuda, shape, n_decay, seed, noalloc):
    rng = np.random.default_rng(seed)
    go = torch.tensor(rng.normal(size=shape).astype(np.float32), device=cuda)
    y = torch.tensor((np.round(rng.normal(0, 2, size=shape) * 4096) / 4096).astype(np.float32), device=cuda)
    dec = torch.tensor(np.round(rng.uniform(50, 2000, size=n_decay)).astype(np.float32), device=cuda)
    gx = torch.full(shape, float('nan'), device=cuda)
    gd = torch.full((n_decay,), float('nan'), device=cuda)
    g = ops.geom(go, n_decay)
    stream = native.stream_of(go)
    if noalloc:
        native.call('sb_li_bwd_noalloc', go, native.ptr(go), native.ptr(y), native.ptr(dec), n_decay, native.ptr(gx),
                    native.ptr(gd), g, stream)
    else:
        scratch = native.scratch(g.rows, n_decay, cuda)
        native.call('sb_li_bwd', go, native.ptr(go), native.ptr(y), native.ptr(dec), n_decay, native.ptr(gx),
                    native.ptr(gd), native.ptr(scratch), g, stream)
    torch.cuda.synchronize()
    return go, y, dec, gx, gd


def test_two_calls_in_a_row_match_the_caller_scratch_entry_point(cuda):
    from lava_dl_b200 import _native as native, _ops as ops
    from oracle import oracle as O
    cases = [((6, 96, 200), 1, 11),    # shared decay, TMA kernels, 18 warp partials + fold stage
             ((3, 5, 77), 5, 12),      # per-channel decay, plain-load kernels, one partial per row
             ((6, 96, 200), 1, 13),    # and back: the array now holds the per-channel call's leftovers
             ((4, 40, 64), 40, 14)]    # per-channel decay on the TMA kernels (T % 4 == 0, T >= 32)
    for shape, n, seed in cases:
        go, y, dec, gx_ref, gd_ref = _run(native, ops, cuda, shape, n, seed, noalloc=False)
        _, _, _, gx, gd = _run(native, ops, cuda, shape, n, seed, noalloc=True)
        assert_exact(gx, gx_ref, f'grad_x {shape}')
        assert_close(gd, gd_ref, f'grad_decay {shape}', scale=pgrad_scale(n, (gx_ref, y)))
        assert torch.isfinite(gd).all()
        gx_o, gd_o = O.li_bwd(go.cpu().numpy(), y.cpu().numpy(), dec.cpu().numpy())
        assert_close(gx, gx_o, f'grad_x against the oracle {shape}', scale=li_scale(go, dec))
        assert_close(gd, gd_o, f'grad_decay against the oracle {shape}', scale=pgrad_scale(n, (gx_o, y)))
    assert native.device_status() == 0


def test_the_largest_problems_the_array_holds(cuda):
    """Exactly at the capacity of the built-in array: 4 MiB = 524288 fp64 slots, of which the fold takes
    64 per decay value.  Shared decay: 32 rows per slot; per-channel decay: one slot per row."""
    from lava_dl_b200 import _native as native, _ops as ops
    from oracle import oracle as O
    lib = native.load()
    cap = 4 * 1024 * 1024
    slots = cap // 8
    shared_rows = 32 * (slots - 64)
    chan = 512
    chan_batch = (slots - 64 * chan) // chan
    for shape, n, seed in (((shared_rows // 64, 64, 4), 1, 21), ((chan_batch, chan, 32), chan, 22)):
        rows = shape[0] * shape[1]
        assert lib.sb_param_grad_scratch_bytes(rows, n) == cap
        go, y, dec, gx, gd = _run(native, ops, cuda, shape, n, seed, noalloc=True)
        gx_o, gd_o = O.li_bwd(go.cpu().numpy(), y.cpu().numpy(), dec.cpu().numpy())
        assert_close(gx, gx_o, f'grad_x at capacity {shape}', scale=li_scale(go, dec))
        assert_close(gd, gd_o, f'grad_decay at capacity {shape}', scale=pgrad_scale(n, (gx_o, y)))
    # one warp more (shared) / one batch more (per channel) no longer fits
    one = torch.zeros(4, device=cuda)
    for rows, rpb, n in ((shared_rows + 32, 64, 1), ((chan_batch + 1) * chan, chan, chan)):
        g = native.Geom(rows, 4, rpb, 1)
        rc = lib.sb_li_bwd_noalloc(native.ptr(one), native.ptr(one), native.ptr(one), n, native.ptr(one),
                                   native.ptr(one), ctypes.byref(g), None)
        assert rc == -1 and 'built-in area' in native.last_error()
    assert native.device_status() == 0


def test_problems_beyond_the_built_in_scratch_are_refused(cuda):
    from lava_dl_b200 import _native as native
    lib = native.load()
    cap = 4 * 1024 * 1024
    assert lib.sb_param_grad_scratch_bytes(600_000, 300) > cap  # per-channel: one slot per row
    g = native.Geom(600_000, 64, 300, 1)
    one = torch.zeros(4, device=cuda)
    rc = lib.sb_li_bwd_noalloc(native.ptr(one), native.ptr(one), native.ptr(one), 300, native.ptr(one),
                               native.ptr(one), ctypes.byref(g), None)
    assert rc == -1
    msg = native.last_error()
    assert 'built-in area' in msg and str(cap) in msg
