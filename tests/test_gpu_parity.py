"""CUDA kernels (called through the C ABI via lava_dl_b200._ops) against the CPU
oracle on seeded random inputs: every op, ragged and tiny shapes, both kernel
families (TMA-tiled and plain-load), shared and per-channel parameters."""

import zlib

import numpy as np
import pytest
import torch

from _util import (assert_close, assert_exact, assert_quantised_equal, cspike_term_scale, li_scale, pgrad_scale,
                   res_scale)
from oracle import oracle as O

pytestmark = pytest.mark.gpu

W = 4096

# (batch, channels, T): tiny, ragged, tile-boundary and TMA-eligible shapes
SHAPES = [(1, 1, 1), (2, 3, 2), (1, 31, 3), (2, 16, 31), (1, 32, 32), (3, 11, 33), (2, 5, 50), (1, 257, 64),
          (4, 64, 128), (2, 8, 200), (1, 40, 1000), (2, 33, 36)]


@pytest.fixture(scope='module')
def ops(cuda):
    from lava_dl_b200 import _ops
    return _ops


def rng_for(*key):
    return np.random.default_rng(zlib.crc32(repr(key).encode()))


def dev(a, cuda, misalign=False):
    """Upload; with misalign the tensor starts 4 bytes off a 16-byte boundary,
    which forces the plain-load kernels even when T % 4 == 0."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    if not misalign:
        return torch.tensor(a, device=cuda)
    buf = torch.empty(a.size + 1, dtype=torch.float32, device=cuda)
    view = buf[1:].view(a.shape)
    view.copy_(torch.tensor(a))
    return view


def quant(a):
    return (np.round(a * W) / W).astype(np.float32)


def decays(rng, n, lo=0, hi=4096):
    return np.round(rng.uniform(lo, hi, size=n)).astype(np.float32)


@pytest.mark.parametrize('shape', SHAPES)
@pytest.mark.parametrize('per_channel', [False, True])
@pytest.mark.parametrize('misalign', [False, True])
def test_li_fwd_bwd(shape, per_channel, misalign, cuda, ops):
    rng = rng_for('li', shape, per_channel)
    B, C, T = shape
    x = rng.normal(0.3, 1.0, size=shape).astype(np.float32)
    dec = decays(rng, C if per_channel else 1, 0, 2000)
    state = quant(rng.normal(0, 0.5, size=shape[:-1]))
    for thr in (None, 1.25 + 0.01 / W):
        want = O.li_fwd(x, dec, state, W, thr)
        got = ops.li_fwd(dev(x, cuda, misalign), dev(dec, cuda), dev(state, cuda), W, thr)
        assert_quantised_equal(got, want, W, f'li_fwd thr={thr}')
    go = rng.normal(size=shape).astype(np.float32)
    gi_want, gd_want = O.li_bwd(go, want, dec)
    gi, gd = ops.li_bwd(dev(go, cuda, misalign), dev(want, cuda, misalign), dev(dec, cuda), True)
    assert_close(gi, gi_want, 'li_bwd grad_in', scale=li_scale(go, dec))
    assert_close(gd, gd_want, 'li_bwd grad_decay', scale=pgrad_scale(dec.size, (gi_want, want)))
    gi2, none = ops.li_bwd(dev(go, cuda, misalign), None, dev(dec, cuda), False)
    assert none is None
    assert_exact(gi2, gi, 'li_bwd with and without decay gradient')


def test_li_final_state_and_nonpow2_scale(cuda, ops):
    rng = rng_for('li_final')
    shape = (2, 7, 45)
    x = rng.normal(0.3, 1.0, size=shape).astype(np.float32)
    for w in (W, 1000, 3):
        want = O.li_fwd(x, np.array([321.0]), np.array([0.25]), w, 0.9)
        got, fin = ops.li_fwd(dev(x, cuda), dev([321.0], cuda), dev([0.25], cuda), w, 0.9, want_final=True)
        assert_exact(got, want, f'li_fwd w_scale={w}')
        assert_exact(fin, want[..., -1], 'final state')


@pytest.mark.parametrize('shape', SHAPES)
@pytest.mark.parametrize('per_channel', [False, True])
def test_ath_apth(shape, per_channel, cuda, ops):
    rng = rng_for('ath', shape, per_channel)
    B, C, T = shape
    n = C if per_channel else 1
    x = rng.normal(0.5, 1.5, size=shape).astype(np.float32)
    rd, td = decays(rng, n, 0, 1000), decays(rng, n, 0, 1000)
    rs = quant(rng.uniform(-0.25, 0.75, size=shape[:-1]))
    ts = quant(rng.uniform(0.5, 1.5, size=shape[:-1]))
    th_w, ref_w = O.ath_fwd(x, rs, rd, ts, td, 0.5, 1.0, W)
    th, ref = ops.ath_fwd(dev(x, cuda), dev(rs, cuda), dev(rd, cuda), dev(ts, cuda), dev(td, cuda), 0.5, 1.0, W)
    assert_quantised_equal(th, th_w, W, 'ath threshold')
    assert_quantised_equal(ref, ref_w, W, 'ath refractory')

    re = rng.normal(0, 1.5, size=shape).astype(np.float32)
    im = rng.normal(0, 1.5, size=shape).astype(np.float32)
    ims = rng.normal(size=shape[:-1]).astype(np.float32)
    th_w, ref_w = O.apth_fwd(re, im, ims, rs, rd, ts, td, 0.25, 0.5, W)
    th, ref = ops.apth_fwd(dev(re, cuda), dev(im, cuda), dev(ims, cuda), dev(rs, cuda), dev(rd, cuda),
                           dev(ts, cuda), dev(td, cuda), 0.25, 0.5, W)
    assert_quantised_equal(th, th_w, W, 'apth threshold')
    assert_quantised_equal(ref, ref_w, W, 'apth refractory')


def sincos(rng, n):
    p = rng.uniform(3.0, 40.0, size=n)
    d = rng.uniform(0.02, 0.3, size=n)
    return (np.round(4096 * np.sin(2 * np.pi / p) * (1 - d)).astype(np.float32),
            np.round(4096 * np.cos(2 * np.pi / p) * (1 - d)).astype(np.float32))


@pytest.mark.parametrize('shape', SHAPES)
@pytest.mark.parametrize('per_channel', [False, True])
@pytest.mark.parametrize('misalign', [False, True])
def test_resonator(shape, per_channel, misalign, cuda, ops):
    rng = rng_for('res', shape, per_channel)
    B, C, T = shape
    sd, cd = sincos(rng, C if per_channel else 1)
    re_in = rng.normal(0, 0.5, size=shape).astype(np.float32)
    im_in = rng.normal(0, 0.5, size=shape).astype(np.float32)
    rs, ims = quant(rng.normal(0, 0.3, size=shape[:-1])), quant(rng.normal(0, 0.3, size=shape[:-1]))
    for thr in (None, 0.75, 0.0):
        re_w, im_w = O.res_fwd(re_in, im_in, sd, cd, rs, ims, W, thr)
        re, im = ops.res_fwd(dev(re_in, cuda, misalign), dev(im_in, cuda, misalign), dev(sd, cuda), dev(cd, cuda),
                             dev(rs, cuda), dev(ims, cuda), W, thr)
        assert_quantised_equal(re, re_w, W, f'res real thr={thr}')
        assert_quantised_equal(im, im_w, W, f'res imag thr={thr}')
    g_re = rng.normal(size=shape).astype(np.float32)
    g_im = rng.normal(size=shape).astype(np.float32)
    a_w, b_w, gs_w, gc_w = O.res_bwd(g_re, g_im, re_w, im_w, sd, cd)
    a, b, gs, gc = ops.res_bwd(dev(g_re, cuda, misalign), dev(g_im, cuda, misalign), dev(re_w, cuda, misalign),
                               dev(im_w, cuda, misalign), dev(sd, cuda), dev(cd, cuda), True)
    S_re, S_im = res_scale(g_re, g_im, sd, cd)
    S_p = pgrad_scale(sd.size, (a_w, re_w), (a_w, im_w), (b_w, re_w), (b_w, im_w))
    assert_close(a, a_w, 'res_bwd grad_re', scale=S_re)
    assert_close(b, b_w, 'res_bwd grad_im', scale=S_im)
    assert_close(gs, gs_w, 'res_bwd grad_sin', scale=S_p)
    assert_close(gc, gc_w, 'res_bwd grad_cos', scale=S_p)
    a2, b2, _, _ = ops.res_bwd(dev(g_re, cuda), dev(g_im, cuda), None, None, dev(sd, cuda), dev(cd, cuda), False)
    assert_exact(a2, a, 'res_bwd with and without parameter gradient')
    assert_exact(b2, b, 'res_bwd with and without parameter gradient')


@pytest.mark.parametrize('shape', SHAPES)
@pytest.mark.parametrize('per_channel', [False, True])
def test_adaptive_resonator(shape, per_channel, cuda, ops):
    rng = rng_for('adres', shape, per_channel)
    B, C, T = shape
    n = C if per_channel else 1
    sd, cd = sincos(rng, n)
    rd, td = decays(rng, n, 0, 1000), decays(rng, n, 0, 1000)
    re_in = rng.normal(0, 0.5, size=shape).astype(np.float32)
    im_in = rng.normal(0, 0.5, size=shape).astype(np.float32)
    st = [quant(rng.normal(0, 0.3, size=shape[:-1])) for _ in range(2)]
    refs = quant(rng.uniform(-0.25, 0.75, size=shape[:-1]))
    ths = quant(rng.uniform(0.25, 1.0, size=shape[:-1]))
    want = O.adres_fwd(re_in, im_in, sd, cd, rd, td, st[0], st[1], refs, ths, 0.25, 0.5, W)
    got = ops.adres_fwd(dev(re_in, cuda), dev(im_in, cuda), dev(sd, cuda), dev(cd, cuda), dev(rd, cuda),
                        dev(td, cuda), dev(st[0], cuda), dev(st[1], cuda), dev(refs, cuda), dev(ths, cuda), 0.25,
                        0.5, W)
    for g, w_, k in zip(got, want, ('real', 'imag', 'threshold', 'refractory')):
        assert_quantised_equal(g, w_, W, f'adres {k}')


@pytest.mark.parametrize('shape', SHAPES)
@pytest.mark.parametrize('graded', [False, True])
@pytest.mark.parametrize('tensor_thr', [False, True])
def test_spike_functions(shape, graded, tensor_thr, cuda, ops):
    rng = rng_for('spike', shape, graded, tensor_thr)
    v = quant(rng.normal(0.8, 1.0, size=shape))
    thr = rng.uniform(0.8, 1.4, size=shape).astype(np.float32) if tensor_thr else 1.25 + 0.01 / W
    thr_d = dev(thr, cuda) if tensor_thr else thr
    gs = rng.normal(size=shape).astype(np.float32)
    assert_exact(ops.spike_fwd(dev(v, cuda), thr_d, graded, 1), O.spike_fwd(v, thr, graded, 1), 'spike')
    assert_close(ops.spike_bwd(dev(v, cuda), thr_d, dev(gs, cuda), 125.0, 0.1, graded),
                 O.spike_bwd(v, thr, gs, 125.0, 0.1, graded), 'spike grad')

    re, im = quant(rng.normal(size=shape)), quant(rng.normal(size=shape))
    last = rng.normal(size=shape[:-1]).astype(np.float32)
    cthr = rng.uniform(0.2, 0.7, size=shape).astype(np.float32) if tensor_thr else 0.5
    cthr_d = dev(cthr, cuda) if tensor_thr else cthr
    assert_exact(ops.cspike_fwd(dev(re, cuda), dev(im, cuda), cthr_d, dev(last, cuda), graded, 1),
                 O.cspike_fwd(re, im, cthr, last, graded, 1), 'complex spike')
    gre, gim = ops.cspike_bwd(dev(re, cuda), dev(im, cuda), cthr_d, dev(gs, cuda), 0.25, 10.0, graded)
    gre_w, gim_w = O.cspike_bwd(re, im, cthr, gs, 0.25, 10.0, graded)
    t_re, t_im = cspike_term_scale(re, im, cthr, gs, 0.25, 10.0, graded)
    assert_close(gre, gre_w, 'complex spike grad_re', scale=t_re)
    assert_close(gim, gim_w, 'complex spike grad_im', scale=t_im)


@pytest.mark.parametrize('shape', SHAPES + [(2, 3, 4, 40)])
def test_shift(shape, cuda, ops):
    rng = rng_for('shift', shape)
    x = rng.uniform(size=shape).astype(np.float32)
    T = shape[-1]
    for sv in (0, 1, -1, 7, -7, T - 1, T, T + 5, -(T + 5)):
        assert_exact(ops.shift(dev(x, cuda), sv), O.shift(x, sv), f'shift {sv}')
    assert_exact(ops.shift(dev(x, cuda), 9, 2.0), O.shift(x, 9, 2.0), 'shift 9 at Ts=2')
    if len(shape) >= 3 and int(np.prod(shape[1:-1])) > 1:
        lut = rng.integers(-T - 2, T + 3, size=shape[1:-1]).astype(np.float32) + 0.4
        assert_exact(ops.shift(dev(x, cuda), dev(lut, cuda)), O.shift(x, lut), 'per-neuron shift')
        assert_exact(ops.shift(dev(x, cuda), dev(lut, cuda), 2.0), O.shift(x, lut, 2.0), 'per-neuron shift Ts=2')


@pytest.mark.parametrize('shape', SHAPES + [(2, 3, 1100), (1, 2, 2050)])
@pytest.mark.parametrize('K', [1, 2, 16, 50, 64, 100])
def test_fir(shape, K, cuda, ops):
    rng = rng_for('fir', shape, K)
    x = rng.uniform(size=shape).astype(np.float32)
    f = (np.exp(-np.arange(K) / 8) / 8 * (1 + 0.1 * rng.normal(size=K))).astype(np.float32)
    for corr in (False, True):
        for ts in (1.0, 2.0):
            assert_close(ops.fir(dev(x, cuda), dev(f, cuda), ts, corr), O.fir(x, f, ts, corr), f'fir corr={corr}')


@pytest.mark.parametrize('shape', [(2, 5, 50), (3, 16, 200), (2, 4, 1100), (1, 7, 1000)])
def test_fused_delay_filter(shape, cuda, ops):
    rng = rng_for('shift_fir', shape)
    T = shape[-1]
    x = (rng.uniform(size=shape) < 0.2).astype(np.float32)
    g = rng.normal(size=shape).astype(np.float32)
    f = (np.exp(-np.arange(64) / 8) / 8).astype(np.float32)
    lut = rng.integers(0, 63, size=shape[1:-1]).astype(np.float32)
    for sv, sv_d in ((lut, dev(lut, cuda)), (5, 5), (-3, -3)):
        want = O.conv(O.shift(x, sv), f)
        assert_close(ops.shift_fir(dev(x, cuda), sv_d, 1, dev(f, cuda), 1.0, backward=False), want, 'conv(shift(x))')
        neg = -sv
        want_b = O.shift(O.corr(g, f), neg)
        assert_close(ops.shift_fir(dev(g, cuda), sv_d, 1, dev(f, cuda), 1.0, backward=True), want_b,
                     'shift(corr(g), -d)')


def _fir_scale(x, f, ts, corr, shift=None):
    """Sum of the magnitudes of the terms each output adds up: the forward-error
    scale of the filter sum (equals |output| where nothing cancels), floored at
    1 % of its maximum like every other comparison.  With ``shift`` the filter
    runs on the unshifted input and its output is shifted: the tensor-core kernel
    computes an advanced row that way and subtracts what the dropped head of the
    row contributed, so those samples belong to the error scale."""
    s = O.fir(np.abs(x), np.abs(f), abs(ts), corr)
    if shift is not None:
        s = O.shift(s, shift)
    return np.maximum(s, 0.01 * s.max() + 1e-30)


# Shapes that take the tensor-core kernel (rows >= 128, T % 4 == 0, T >= 32, K <= 64):
# rows off the 128 grid, T off the 32 grid, single tile, many tiles.
TC_SHAPES = [(1, 128, 32), (1, 129, 36), (2, 100, 1000), (4, 64, 96), (3, 50, 260)]


@pytest.mark.parametrize('shape', TC_SHAPES)
@pytest.mark.parametrize('K', [1, 7, 32, 33, 64])
def test_fir_tensor_core(shape, K, cuda, ops):
    from lava_dl_b200 import _native as native
    rows = int(np.prod(shape[:-1]))
    assert native.load().sb_fir_uses_tensor_cores(K, rows, shape[-1]) == 1
    rng = rng_for('fir_tc', shape, K)
    f = (np.exp(-np.arange(K) / 8) / 8 * (1 + 0.3 * rng.normal(size=K))).astype(np.float32)
    for kind in ('uniform', 'normal', 'spikes'):
        if kind == 'uniform':
            x = rng.uniform(size=shape).astype(np.float32)
        elif kind == 'normal':
            x = rng.normal(size=shape).astype(np.float32)
        else:
            x = (rng.uniform(size=shape) < 0.05).astype(np.float32)
        for corr in (False, True):
            for ts in (1.0, 2.0):
                got = ops.fir(dev(x, cuda), dev(f, cuda), ts, corr)
                assert_close(got, O.fir(x, f, ts, corr), f'fir tc {kind} corr={corr} ts={ts}',
                             scale=_fir_scale(x, f, ts, corr))
    assert native.device_status() == 0


@pytest.mark.parametrize('shape', [(2, 130, 200), (1, 128, 1000), (2, 64, 36)])
def test_fused_delay_filter_tensor_core(shape, cuda, ops):
    from lava_dl_b200 import _native as native
    rng = rng_for('shift_fir_tc', shape)
    T = shape[-1]
    rows = int(np.prod(shape[:-1]))
    assert native.load().sb_fir_uses_tensor_cores(64, rows, T) == 1
    x = (rng.uniform(size=shape) < 0.2).astype(np.float32)
    g = rng.normal(size=shape).astype(np.float32)
    f = (np.exp(-np.arange(64) / 8) / 8).astype(np.float32)
    lut = rng.integers(0, 63, size=shape[1:-1]).astype(np.float32)
    mixed = rng.integers(-70, 71, size=shape[1:-1]).astype(np.float32)
    cases = [(lut, dev(lut, cuda)), (mixed, dev(mixed, cuda)), (0, 0), (5, 5), (-3, -3), (70, 70), (-70, -70),
             (T + 5, T + 5), (-(T + 5), -(T + 5))]
    for sv, sv_d in cases:
        shifted = O.shift(x, sv)
        want = O.conv(shifted, f)
        assert_close(ops.shift_fir(dev(x, cuda), sv_d, 1, dev(f, cuda), 1.0, backward=False), want,
                     f'conv(shift(x, {sv if np.isscalar(sv) else "lut"}))', scale=_fir_scale(x, f, 1.0, False, sv))
        neg = -sv
        cg = O.corr(g, f)
        want_b = O.shift(cg, neg)
        assert_close(ops.shift_fir(dev(g, cuda), sv_d, 1, dev(f, cuda), 1.0, backward=True), want_b,
                     'shift(corr(g), -d)', scale=_fir_scale(g, f, 1.0, True, neg))
    # Ts = 2 on the delay: d = int(shift / 2)
    want = O.conv(O.shift(x, lut, 2.0), f)
    assert_close(ops.shift_fir(dev(x, cuda), dev(lut, cuda), 2.0, dev(f, cuda), 1.0, backward=False), want,
                 'conv(shift(x, lut, Ts=2))')
    assert native.device_status() == 0


# --------------------------------------------------------------------------
# fused neuron passes against the oracle's un-fused call sequences
# --------------------------------------------------------------------------
@pytest.mark.parametrize('shape', SHAPES)
@pytest.mark.parametrize('per_channel', [False, True])
@pytest.mark.parametrize('misalign', [False, True])
def test_cuba_fused(shape, per_channel, misalign, cuda, ops):
    rng = rng_for('cuba', shape, per_channel)
    B, C, T = shape
    n = C if per_channel else 1
    x = rng.normal(0.3, 1.0, size=shape).astype(np.float32)
    cd, vd = decays(rng, n, 800, 1300), decays(rng, n, 50, 300)
    cs, vs = quant(rng.normal(0, 0.5, size=shape[:-1])), quant(rng.normal(0, 0.5, size=shape[:-1]))
    gs = rng.normal(size=shape).astype(np.float32)
    for graded in (False, True):
        want = O.cuba(x, 1.25, cd, vd, cstate=cs, vstate=vs, grad_spike=gs, graded=graded)
        r = ops.cuba_fwd(dev(x, cuda, misalign), dev(cd, cuda), dev(vd, cuda), dev(cs, cuda), dev(vs, cuda),
                         1.25 + 0.01 / W, W, want_current=True, want_spike=True, graded=graded)
        assert_quantised_equal(r['current'], want['current'], W, 'current')
        assert_quantised_equal(r['voltage'], want['voltage'], W, 'voltage')
        assert_exact(r['spike'], want['spike'], 'spike')
        assert_exact(r['final_c'], want['current'][..., -1], 'final current')
        assert_exact(r['final_v'], want['voltage'][..., -1], 'final voltage')
        assert_exact(r['final_s'], want['spike'][..., -1], 'final spike')
        r2 = ops.cuba_fwd(dev(x, cuda, misalign), dev(cd, cuda), dev(vd, cuda), dev(cs, cuda), dev(vs, cuda),
                          1.25 + 0.01 / W, W, want_current=False, want_spike=True, graded=graded)
        assert_exact(r2['spike'], want['spike'], 'spike (no current output)')
        assert_exact(r2['voltage'], r['voltage'], 'voltage (no current output)')
        gx, gcd, gvd = ops.cuba_bwd(dev(gs, cuda, misalign), r['voltage'], 1.25 + 0.01 / W, r['current'],
                                    dev(cd, cuda), dev(vd, cuda), 125.0, 0.1, graded, True)
        g_v = O.spike_bwd(want['voltage'], 1.25 + 0.01 / W, gs, 125.0, 0.1, graded)
        S_c = li_scale(g_v, vd)
        g_c, _ = O.li_bwd(g_v, want['voltage'], vd)
        assert_close(gx, want['grad_x'], 'grad_x', scale=li_scale(S_c, cd))
        assert_close(gcd, want['grad_current_decay'], 'grad current decay',
                     scale=pgrad_scale(cd.size, (want['grad_x'], want['current'])))
        assert_close(gvd, want['grad_voltage_decay'], 'grad voltage decay',
                     scale=pgrad_scale(vd.size, (g_c, want['voltage'])))
        gx2, _, _ = ops.cuba_bwd(dev(gs, cuda, misalign), r['voltage'], 1.25 + 0.01 / W, None, dev(cd, cuda),
                                 dev(vd, cuda), 125.0, 0.1, graded, False)
        assert_exact(gx2, gx, 'grad_x with and without decay gradients')


@pytest.mark.parametrize('shape', [(2, 3, 2), (3, 11, 33), (1, 257, 64), (4, 64, 128), (2, 33, 36)])
@pytest.mark.parametrize('per_channel', [False, True])
def test_decays_outside_the_clamp(shape, per_channel, cuda, ops):
    """The raw dynamics() calls accept any decay: 4096 - decay below 0 or above 4096 (the Neuron
    classes clamp to 0 .. 4096 first).  The kernels pick their short truncating multiply per warp only
    when every lane's multiplier is a plain decay; these inputs make warps take the general one,
    alone and mixed with in-range channels, plus a spike threshold that differs from the reset one."""
    rng = rng_for('wide', shape, per_channel)
    B, C, T = shape
    n = C if per_channel else 1

    def wide(k):
        d = decays(rng, n, -60, 4400)   # 4096 - d <= 4156: states grow at most 6.5-fold over 128 steps (int32 states)
        if per_channel and n > 2:
            d[:: 3] = decays(rng, len(d[:: 3]), 0, 4096)   # in-range channels next to out-of-range ones
        else:
            d[0] = (-50.0, 4200.0, 4096.0, 0.0)[k % 4]
        return d

    x = rng.normal(0.3, 1.0, size=shape).astype(np.float32)
    st = [quant(rng.normal(0, 0.5, size=shape[:-1])) for _ in range(4)]
    for k in range(2):
        dec = wide(k)
        for thr in (None, 0.9):
            want = O.li_fwd(x, dec, st[0], W, thr)
            got = ops.li_fwd(dev(x, cuda), dev(dec, cuda), dev(st[0], cuda), W, thr)
            assert_quantised_equal(got, want, W, f'li_fwd decay={dec[:3]} thr={thr}')
        cd, vd = wide(k), wide(k + 1)
        want = O.cuba(x, 1.25, cd, vd, cstate=st[0], vstate=st[1])
        r = ops.cuba_fwd(dev(x, cuda), dev(cd, cuda), dev(vd, cuda), dev(st[0], cuda), dev(st[1], cuda),
                         1.25 + 0.01 / W, W, want_current=True, want_spike=True)
        assert_quantised_equal(r['current'], want['current'], W, 'current')
        assert_quantised_equal(r['voltage'], want['voltage'], W, 'voltage')
        assert_exact(r['spike'], want['spike'], 'spike')
        td, rd = wide(k + 2), wide(k + 3)
        ths, refs = quant(rng.uniform(0.8, 1.5, size=shape[:-1])), quant(rng.uniform(0.0, 0.5, size=shape[:-1]))
        th_w, ref_w = O.ath_fwd(x, refs, rd, ths, td, 0.5, 1.0, W)
        th, ref = ops.ath_fwd(dev(x, cuda), dev(refs, cuda), dev(rd, cuda), dev(ths, cuda), dev(td, cuda), 0.5, 1.0, W)
        assert_quantised_equal(th, th_w, W, 'ath threshold')
        assert_quantised_equal(ref, ref_w, W, 'ath refractory')
        want = O.alif(x, 1.0, 0.5, cd, vd, td, rd, cstate=st[0], vstate=st[1], th_state=ths, ref_state=refs)
        args = (dev(x, cuda), dev(cd, cuda), dev(vd, cuda), dev(rd, cuda), dev(td, cuda), dev(st[0], cuda),
                dev(st[1], cuda), dev(refs, cuda), dev(ths, cuda), 0.5, 1.0, W)
        outs, _ = ops.alif_fwd(*args, dynamics_mode=True)
        for o, key in zip(outs, ('current', 'voltage', 'threshold', 'refractory')):
            assert_quantised_equal(o, want[key], W, key)
        (spike, _, _), _ = ops.alif_fwd(*args, dynamics_mode=False)
        assert_exact(spike, want['spike'], 'alif spike')
    # spike threshold and reset threshold that differ: no reset at all (threshold <= 0 disables it)
    cd, vd = decays(rng, n, 800, 1300), decays(rng, n, 50, 300)
    r = ops.cuba_fwd(dev(x, cuda), dev(cd, cuda), dev(vd, cuda), dev(st[0], cuda), dev(st[1], cuda),
                     -0.5, W, want_current=True, want_spike=True)
    cur = O.li_fwd(x, cd, st[0], W)
    vol = O.li_fwd(cur, vd, st[1], W)
    assert_quantised_equal(r['current'], cur, W, 'current without reset')
    assert_quantised_equal(r['voltage'], vol, W, 'voltage without reset')
    assert_exact(r['spike'], O.spike_fwd(vol, -0.5), 'spike without reset')
    # sin / cos beyond the pre-shifted multiplier's range take the general product
    sd = np.full(n, float(1 << 27), np.float32)
    cdk = np.full(n, -float((1 << 27) + 4096), np.float32)
    small = (x * 1e-3).astype(np.float32)
    zero = np.zeros(shape[:-1], np.float32)
    re_w, im_w = O.res_fwd(small, small, sd, cdk, zero, zero, W, None)
    re, im = ops.res_fwd(dev(small, cuda), dev(small, cuda), dev(sd, cuda), dev(cdk, cuda), dev(zero, cuda),
                         dev(zero, cuda), W, None)
    # such multipliers grow the state 32768-fold per step: the first two steps stay inside int32
    keep = min(T, 2)
    assert np.abs(re_w[..., :keep]).max() * W < 2 ** 31 and np.abs(im_w[..., :keep]).max() * W < 2 ** 31
    assert_quantised_equal(re[..., :keep], re_w[..., :keep], W, 'resonator with huge sin/cos (real)')
    assert_quantised_equal(im[..., :keep], im_w[..., :keep], W, 'resonator with huge sin/cos (imag)')


@pytest.mark.parametrize('shape', SHAPES + [(3, 40, 96), (2, 70, 416)])
@pytest.mark.parametrize('misalign', [False, True])
@pytest.mark.parametrize('want_voltage', [False, True])
def test_cuba_packed_spikes(shape, misalign, want_voltage, cuda, ops):
    """Spikes as 32-step bit words, with and without the voltage series, with and without the
    one-step delay: unpacked they are the fp32 spike tensor of the oracle."""
    rng = rng_for('packed', shape)
    B, C, T = shape
    x = rng.normal(0.3, 1.0, size=shape).astype(np.float32)
    cd, vd = decays(rng, C, 800, 1300), decays(rng, C, 50, 300)
    cs, vs = quant(rng.normal(0, 0.5, size=shape[:-1])), quant(rng.normal(0, 0.5, size=shape[:-1]))
    head = (rng.uniform(size=shape[:-1]) < 0.5).astype(np.float32)
    want = O.cuba(x, 1.25, cd, vd, cstate=cs, vstate=vs)
    for delay in (0, 1):
        r = ops.cuba_fwd_packed(dev(x, cuda, misalign), dev(cd, cuda), dev(vd, cuda), dev(cs, cuda), dev(vs, cuda),
                                1.25 + 0.01 / W, W, want_voltage=want_voltage, spike_delay=delay,
                                delay_head=dev(head, cuda) if delay else None)
        bits = r['spike_bits']
        assert bits.dtype == torch.int32 and tuple(bits.shape) == (B, C, (T + 31) // 32)
        spike = want['spike']
        if delay:
            spike = np.concatenate([head[..., None], spike[..., :-1]], axis=-1)
        assert_exact(ops.unpack_spikes(bits, T), spike, f'unpacked spikes (delay {delay})')
        tail = ops.unpack_spikes(bits, 32 * bits.shape[-1])[..., T:]
        assert not bool(tail.any()), 'bits past the end of the row must be zero'
        if want_voltage:
            assert_quantised_equal(r['voltage'], want['voltage'], W, 'voltage')
        else:
            assert r['voltage'] is None
        assert_exact(r['final_v'], want['voltage'][..., -1], 'final voltage')
        assert_exact(r['final_s'], want['spike'][..., -1], 'final spike')


@pytest.mark.parametrize('shape', SHAPES)
@pytest.mark.parametrize('misalign', [False, True])
def test_cuba_forward_without_the_voltage_series(shape, misalign, cuda, ops):
    """What ``Neuron.forward`` runs when nothing will be differentiated: fp32 spikes and the final
    states, the voltage series left unwritten -- with and without the one-step delay and an axonal
    delay table.  The spikes are those of the oracle; a neuron in ``no_grad`` takes this path."""
    rng = rng_for('novolt', shape)
    B, C, T = shape
    x = rng.normal(0.3, 1.0, size=shape).astype(np.float32)
    cd, vd = decays(rng, C, 800, 1300), decays(rng, C, 50, 300)
    cs, vs = quant(rng.normal(0, 0.5, size=shape[:-1])), quant(rng.normal(0, 0.5, size=shape[:-1]))
    head = (rng.uniform(size=shape[:-1]) < 0.5).astype(np.float32)
    axon = rng.integers(0, min(62, T), size=C).astype(np.float32)
    want = O.cuba(x, 1.25, cd, vd, cstate=cs, vstate=vs)
    args = (dev(x, cuda, misalign), dev(cd, cuda), dev(vd, cuda), dev(cs, cuda), dev(vs, cuda), 1.25 + 0.01 / W, W)
    for delay, use_axon in ((0, False), (1, False), (1, True)):
        kw = dict(want_current=False, want_spike=True, spike_delay=delay, delay_head=dev(head, cuda) if delay else None,
                  axon_delay=dev(axon, cuda) if use_axon else None)
        full = ops.cuba_fwd(*args, **kw)
        lean = ops.cuba_fwd(*args, want_voltage=False, **kw)
        assert lean['voltage'] is None
        assert_exact(lean['spike'], full['spike'].cpu().numpy(), f'spikes without the voltage series (delay {delay}, axon {use_axon})')
        if not use_axon:
            spike = want['spike']
            if delay:
                spike = np.concatenate([head[..., None], spike[..., :-1]], axis=-1)
            assert_exact(lean['spike'], spike, f'spikes against the oracle (delay {delay})')
        assert_exact(lean['final_c'], want['current'][..., -1], 'final current')
        assert_exact(lean['final_v'], want['voltage'][..., -1], 'final voltage')
        assert_exact(lean['final_s'], want['spike'][..., -1], 'final spike')
    with pytest.raises(RuntimeError):
        ops.cuba_fwd(*args, want_current=True, want_spike=True, want_voltage=False)


@pytest.mark.parametrize('shape', SHAPES)
@pytest.mark.parametrize('misalign', [False, True])
def test_cuba_fused_step_delay(shape, misalign, cuda, ops):
    """Spikes written one step late inside the kernel == shift(spike, 1) with the head
    value at t = 0, and the backward reads the gradient of the late series."""
    rng = rng_for('cuba_delay', shape)
    x = rng.normal(0.3, 1.0, size=shape).astype(np.float32)
    cd, vd = np.array([1024.0], np.float32), np.array([123.0], np.float32)
    gs = rng.normal(size=shape).astype(np.float32)
    head = (rng.uniform(size=shape[:-1]) < 0.5).astype(np.float32)
    want = O.cuba(x, 1.25, cd, vd)
    late = O.shift(want['spike'], 1)
    for h, h_dev in ((None, None), (head, dev(head, cuda))):
        r = ops.cuba_fwd(dev(x, cuda, misalign), dev(cd, cuda), dev(vd, cuda), dev(np.zeros(shape[:-1]), cuda),
                         dev(np.zeros(shape[:-1]), cuda), 1.25 + 0.01 / W, W, want_current=True, want_spike=True,
                         spike_delay=1, delay_head=h_dev)
        expect = late.copy()
        if h is not None:
            expect[..., 0] = h
        assert_exact(r['spike'], expect, 'late spikes')
        assert_exact(r['final_s'], want['spike'][..., -1], 'undelayed last spike')
        assert_quantised_equal(r['voltage'], want['voltage'], W, 'voltage')
    # gradient of the late series: g_spike[t] = g_late[t + 1]
    g_early = O.shift(gs, -1)
    ref = O.cuba(x, 1.25, cd, vd, grad_spike=g_early)
    gx, gcd, gvd = ops.cuba_bwd(dev(gs, cuda, misalign), r['voltage'], 1.25 + 0.01 / W, r['current'], dev(cd, cuda),
                                dev(vd, cuda), 125.0, 0.1, False, True, spike_delay=1)
    g_v = O.spike_bwd(want['voltage'], 1.25 + 0.01 / W, g_early, 125.0, 0.1, False)
    assert_close(gx, ref['grad_x'], 'grad_x', scale=li_scale(li_scale(g_v, vd), cd))
    g_c, _ = O.li_bwd(g_v, want['voltage'], vd)
    assert_close(gcd, ref['grad_current_decay'], 'grad current decay',
                 scale=pgrad_scale(1, (ref['grad_x'], want['current'])))
    assert_close(gvd, ref['grad_voltage_decay'], 'grad voltage decay', scale=pgrad_scale(1, (g_c, want['voltage'])))


@pytest.mark.parametrize('shape', SHAPES)
@pytest.mark.parametrize('graded', [False, True])
def test_alif_margin_form(shape, graded, cuda, ops):
    """The training forward of the ALIF neuron writes voltage - (threshold + refractory) as one
    series: exactly the difference of the two series of the three-output kernel, and the backward
    pass on it (threshold 0) returns the same input gradient, bit for bit."""
    rng = rng_for('margin', shape)
    B, C, T = shape
    zeros = dev(np.zeros(shape[:-1]), cuda)
    x = rng.normal(0.2, 1.0, size=shape).astype(np.float32)
    gs = rng.normal(size=shape).astype(np.float32)
    cd, vd = decays(rng, C, 700, 900), decays(rng, C, 150, 250)
    td, rd = decays(rng, C, 300, 500), decays(rng, C, 300, 500)
    ths = quant(rng.uniform(0.8, 1.5, size=shape[:-1]))
    args = (dev(x, cuda), dev(cd, cuda), dev(vd, cuda), dev(rd, cuda), dev(td, cuda), zeros, zeros, zeros,
            dev(ths, cuda), 0.5, 1.0, W)
    for delay in ((0,) if graded else (0, 1)):
        (spike, voltage, thsum), fin_full = ops.alif_fwd(*args, dynamics_mode=False, graded=graded, spike_delay=delay)
        (spike_m, margin, none), fin = ops.alif_fwd(*args, dynamics_mode=False, graded=graded, spike_delay=delay, margin=True)
        assert none is None
        assert_exact(spike_m, spike.cpu().numpy(), 'spikes of the margin form')
        assert_exact(margin, (voltage - thsum).cpu().numpy(), 'margin = voltage - (threshold + refractory)')
        for k in fin:
            assert_exact(fin[k], fin_full[k].cpu().numpy(), k)
        g_two, _, _ = ops.cuba_bwd(dev(gs, cuda), voltage, thsum, None, dev(cd, cuda), dev(vd, cuda), 100.0, 0.1, graded,
                                   False, spike_delay=delay)
        g_one, _, _ = ops.cuba_bwd(dev(gs, cuda), margin, 0.0, None, dev(cd, cuda), dev(vd, cuda), 100.0, 0.1, graded,
                                   False, spike_delay=delay)
        assert_exact(g_one, g_two.cpu().numpy(), 'input gradient from the margin')


@pytest.mark.parametrize('shape', SHAPES)
@pytest.mark.parametrize('graded', [False, True])
def test_adrf_margin_form(shape, graded, cuda, ops):
    """The training forward of the adaptive resonator without sin / cos gradients writes
    re - (threshold + refractory) and im: the difference of the series of the four-output kernel,
    and the backward pass on it (threshold 0) returns the same input gradients, bit for bit."""
    rng = rng_for('rmargin', shape)
    B, C, T = shape
    zeros = dev(np.zeros(shape[:-1]), cuda)
    re_in = rng.normal(0, 0.5, size=shape).astype(np.float32)
    im_in = rng.normal(0, 0.5, size=shape).astype(np.float32)
    gs = rng.normal(size=shape).astype(np.float32)
    sd, cdk = sincos(rng, C)
    td, rd = decays(rng, C, 300, 500), decays(rng, C, 300, 500)
    ths = quant(rng.uniform(0.3, 0.8, size=shape[:-1]))
    ad = dict(ref_decay=dev(rd, cuda), th_decay=dev(td, cuda), ref_state=zeros, th_state=dev(ths, cuda), th_step=0.25, th0=0.5)
    a = (dev(re_in, cuda), dev(im_in, cuda), dev(sd, cuda), dev(cdk, cuda), zeros, zeros, 0.5, W)
    for delay in ((0,) if graded else (0, 1)):
        full, fin_full = ops.rf_fwd(*a, adaptive=ad, graded=graded, spike_delay=delay)
        lean, fin = ops.rf_fwd(*a, adaptive=ad, graded=graded, spike_delay=delay, margin=True)
        assert lean[3] is None
        assert_exact(lean[0], full[0].cpu().numpy(), 'spikes of the margin form')
        assert_exact(lean[1], (full[1] - full[3]).cpu().numpy(), 'margin = re - (threshold + refractory)')
        assert_exact(lean[2], full[2].cpu().numpy(), 'imaginary series')
        for k in fin:
            assert_exact(fin[k], fin_full[k].cpu().numpy(), k)
        two = ops.rf_bwd(dev(gs, cuda), full[1], full[2], full[3], dev(sd, cuda), dev(cdk, cuda), 50.0, 0.1, graded, False,
                         spike_delay=delay)
        one = ops.rf_bwd(dev(gs, cuda), lean[1], lean[2], 0.0, dev(sd, cuda), dev(cdk, cuda), 50.0, 0.1, graded, False,
                         spike_delay=delay)
        assert_exact(one[0], two[0].cpu().numpy(), 'grad_re from the margin')
        assert_exact(one[1], two[1].cpu().numpy(), 'grad_im from the margin')
    with pytest.raises(ValueError):
        ops.rf_fwd(*a, adaptive=None, margin=True)


@pytest.mark.parametrize('shape', SHAPES)
def test_alif_and_resonator_spikes_only(shape, cuda, ops):
    """The forward kernels of the ALIF, RF and ADRF neurons without the series that only the
    backward pass reads (what ``forward`` runs when nothing will be differentiated): the same
    spikes and final states as the full kernels and as the oracle, with and without the one-step delay."""
    rng = rng_for('lean', shape)
    B, C, T = shape
    head = (rng.uniform(size=shape[:-1]) < 0.5).astype(np.float32)
    zeros = dev(np.zeros(shape[:-1]), cuda)
    x = rng.normal(0.2, 1.0, size=shape).astype(np.float32)
    cd, vd = decays(rng, C, 700, 900), decays(rng, C, 150, 250)
    td, rd = decays(rng, C, 300, 500), decays(rng, C, 300, 500)
    ths = quant(rng.uniform(0.8, 1.5, size=shape[:-1]))
    want = O.alif(x, 1.0, 0.5, cd, vd, td, rd, th_state=ths)
    args = (dev(x, cuda), dev(cd, cuda), dev(vd, cuda), dev(rd, cuda), dev(td, cuda), zeros, zeros, zeros,
            dev(ths, cuda), 0.5, 1.0, W)
    for delay in (0, 1):
        kw = dict(dynamics_mode=False, spike_delay=delay, delay_head=dev(head, cuda) if delay else None)
        full, fin_full = ops.alif_fwd(*args, **kw)
        lean, fin = ops.alif_fwd(*args, spikes_only=True, **kw)
        assert lean[1] is None and lean[2] is None
        assert_exact(lean[0], full[0].cpu().numpy(), f'ALIF spikes only (delay {delay})')
        if not delay:
            assert_exact(lean[0], want['spike'], 'ALIF spikes only against the oracle')
        for k in fin:
            assert_exact(fin[k], fin_full[k].cpu().numpy(), f'ALIF {k}')
    with pytest.raises(ValueError):
        ops.alif_fwd(*args, dynamics_mode=True, spikes_only=True)

    re_in = rng.normal(0, 0.5, size=shape).astype(np.float32)
    im_in = rng.normal(0, 0.5, size=shape).astype(np.float32)
    sd, cdk = sincos(rng, C)
    for adaptive in (False, True):
        if adaptive:
            want = O.adrf(re_in, im_in, 0.5, 0.25, sd, cdk, td, rd, th_state=ths)
            ad = dict(ref_decay=dev(rd, cuda), th_decay=dev(td, cuda), ref_state=zeros, th_state=dev(ths, cuda),
                      th_step=0.25, th0=0.5)
        else:
            want = O.rf(re_in, im_in, 0.5, sd, cdk)
            ad = None
        for delay in (0, 1):
            kw = dict(adaptive=ad, spike_delay=delay, delay_head=dev(head, cuda) if delay else None)
            a = (dev(re_in, cuda), dev(im_in, cuda), dev(sd, cuda), dev(cdk, cuda), zeros, zeros, 0.5, W)
            full, fin_full = ops.rf_fwd(*a, **kw)
            lean, fin = ops.rf_fwd(*a, spikes_only=True, **kw)
            assert all(o is None for o in lean[1:])
            assert_exact(lean[0], full[0].cpu().numpy(), f'resonator spikes only (adaptive={adaptive}, delay {delay})')
            if not delay:
                assert_exact(lean[0], want['spike'], f'resonator spikes only against the oracle (adaptive={adaptive})')
            for k in fin:
                if adaptive or k not in ('final_th', 'final_ref'):   # the plain resonator has no threshold state
                    assert_exact(fin[k], fin_full[k].cpu().numpy(), f'resonator {k}')


@pytest.mark.parametrize('shape', SHAPES)
def test_alif_and_resonator_fused_step_delay(shape, cuda, ops):
    """The one-step delay on the spike store of the ALIF, RF and ADRF forward kernels, and the
    backward passes reading the gradient of the late series: same results as delaying the spikes
    (advancing the gradient) in a separate pass."""
    rng = rng_for('other_delay', shape)
    B, C, T = shape
    head = (rng.uniform(size=shape[:-1]) < 0.5).astype(np.float32)
    gs = rng.normal(size=shape).astype(np.float32)
    g_early = O.shift(gs, -1)
    zeros = dev(np.zeros(shape[:-1]), cuda)

    def late_of(spike, h):
        out = O.shift(spike, 1)
        if h is not None:
            out[..., 0] = h
        return out

    # ALIF
    x = rng.normal(0.2, 1.0, size=shape).astype(np.float32)
    cd, vd = decays(rng, C, 700, 900), decays(rng, C, 150, 250)
    td, rd = decays(rng, C, 300, 500), decays(rng, C, 300, 500)
    ths = quant(rng.uniform(0.8, 1.5, size=shape[:-1]))
    want = O.alif(x, 1.0, 0.5, cd, vd, td, rd, th_state=ths, grad_spike=g_early)
    args = (dev(x, cuda), dev(cd, cuda), dev(vd, cuda), dev(rd, cuda), dev(td, cuda), zeros, zeros, zeros,
            dev(ths, cuda), 0.5, 1.0, W)
    for h in (None, head):
        (spike, voltage, thsum), fin = ops.alif_fwd(*args, dynamics_mode=False, spike_delay=1,
                                                    delay_head=None if h is None else dev(h, cuda))
        assert_exact(spike, late_of(want['spike'], h), 'late ALIF spikes')
        assert_exact(fin['final_s'], want['spike'][..., -1], 'undelayed last spike')
        assert_quantised_equal(voltage, want['voltage'], W, 'voltage')
    gx, _, _ = ops.cuba_bwd(dev(gs, cuda), voltage, thsum, None, dev(cd, cuda), dev(vd, cuda), 100.0, 0.1, False, False,
                            spike_delay=1)
    g_v = O.spike_bwd(want['voltage'], want['threshold'] + want['refractory'], g_early, 100.0, 0.1, False)
    assert_close(gx, want['grad_x'], 'ALIF grad_x of the late series', scale=li_scale(li_scale(g_v, vd), cd))

    # RF and ADRF
    re_in = rng.normal(0, 0.5, size=shape).astype(np.float32)
    im_in = rng.normal(0, 0.5, size=shape).astype(np.float32)
    sd, cdk = sincos(rng, C)
    for adaptive in (False, True):
        if adaptive:
            want = O.adrf(re_in, im_in, 0.5, 0.25, sd, cdk, td, rd, th_state=ths, grad_spike=g_early)
            ad = dict(ref_decay=dev(rd, cuda), th_decay=dev(td, cuda), ref_state=zeros, th_state=dev(ths, cuda),
                      th_step=0.25, th0=0.5)
            tau, srho = 50.0, 0.1
        else:
            want = O.rf(re_in, im_in, 0.5, sd, cdk, grad_spike=g_early)
            ad, tau, srho = None, 0.25, 10.0
        for h in (None, head):
            outs, fin = ops.rf_fwd(dev(re_in, cuda), dev(im_in, cuda), dev(sd, cuda), dev(cdk, cuda), zeros, zeros, 0.5,
                                   W, adaptive=ad, spike_delay=1, delay_head=None if h is None else dev(h, cuda))
            assert_exact(outs[0], late_of(want['spike'], h), f'late resonator spikes (adaptive={adaptive})')
            assert_exact(fin['final_s'], want['spike'][..., -1], 'undelayed last spike')
        thr = outs[3] if adaptive else 0.5
        gre, gim, _, _ = ops.rf_bwd(dev(gs, cuda), outs[1], outs[2], thr, dev(sd, cuda), dev(cdk, cuda), tau, srho,
                                    False, False, spike_delay=1)
        thr_np = (want['threshold'] + want['refractory']) if adaptive else 0.5
        s_re, s_im = cspike_term_scale(want['real'], want['imag'], thr_np, g_early, tau, srho, False)
        S_re, S_im = res_scale(s_re, s_im, sd, cdk)
        assert_close(gre, want['grad_re'], 'resonator grad_re of the late series', scale=S_re)
        assert_close(gim, want['grad_im'], 'resonator grad_im of the late series', scale=S_im)


@pytest.mark.parametrize('shape', [(2, 5, 50), (1, 257, 64), (4, 64, 128), (2, 8, 200), (3, 11, 33), (2, 3, 2)])
@pytest.mark.parametrize('misalign', [False, True])
def test_cuba_fused_axon_delay(shape, misalign, cuda, ops):
    """Step delay + per-neuron axonal delay written by the neuron kernel ==
    shift(shift(spike, 1) with head, delay) of the oracle, bit for bit."""
    from lava_dl_b200 import _native as native
    rng = rng_for('cuba_axon_delay', shape)
    T = shape[-1]
    x = rng.normal(0.3, 1.0, size=shape).astype(np.float32)
    cd, vd = np.array([1024.0], np.float32), np.array([123.0], np.float32)
    head = (rng.uniform(size=shape[:-1]) < 0.5).astype(np.float32)
    want = O.cuba(x, 1.25, cd, vd)
    zeros = dev(np.zeros(shape[:-1]), cuda)
    for ts, lo, hi in ((1.0, 0, 63), (2.0, 0, 125), (1.0, 31, 34), (1.0, 62, 63)):
        lut = (rng.integers(lo, hi, size=shape[1:-1]) + rng.uniform(0, 0.9, size=shape[1:-1])).astype(np.float32)
        for step in (1, 0):
            for h, h_dev in ((None, None), (head, dev(head, cuda))):
                if step == 0 and h is not None:
                    continue
                late = O.shift(want['spike'], 1) if step else want['spike'].copy()
                if h is not None:
                    late[..., 0] = h
                expect = O.shift(late, lut, ts)
                r = ops.cuba_fwd(dev(x, cuda, misalign), dev(cd, cuda), dev(vd, cuda), zeros, zeros, 1.25 + 0.01 / W, W,
                                 want_current=False, want_spike=True, spike_delay=step, delay_head=h_dev,
                                 axon_delay=dev(lut, cuda), axon_delay_ts=ts)
                assert_exact(r['spike'], expect, f'delayed spikes ts={ts} step={step} T={T}')
                assert_exact(r['final_s'], want['spike'][..., -1], 'undelayed last spike')
    assert native.device_status() == 0


@pytest.mark.parametrize('shape', SHAPES)
@pytest.mark.parametrize('per_channel', [False, True])
def test_alif_fused(shape, per_channel, cuda, ops):
    rng = rng_for('alif', shape, per_channel)
    B, C, T = shape
    n = C if per_channel else 1
    x = rng.normal(0.2, 1.0, size=shape).astype(np.float32)
    cd, vd = decays(rng, n, 700, 900), decays(rng, n, 150, 250)
    td, rd = decays(rng, n, 300, 500), decays(rng, n, 300, 500)
    st = [quant(rng.normal(0, 0.5, size=shape[:-1])) for _ in range(2)]
    ths = quant(rng.uniform(0.8, 1.5, size=shape[:-1]))
    refs = quant(rng.uniform(0.0, 0.5, size=shape[:-1]))
    gs = rng.normal(size=shape).astype(np.float32)
    want = O.alif(x, 1.0, 0.5, cd, vd, td, rd, cstate=st[0], vstate=st[1], th_state=ths, ref_state=refs,
                  grad_spike=gs)
    args = (dev(x, cuda), dev(cd, cuda), dev(vd, cuda), dev(rd, cuda), dev(td, cuda), dev(st[0], cuda),
            dev(st[1], cuda), dev(refs, cuda), dev(ths, cuda), 0.5, 1.0, W)
    outs, fin = ops.alif_fwd(*args, dynamics_mode=True)
    for o, k in zip(outs, ('current', 'voltage', 'threshold', 'refractory')):
        assert_quantised_equal(o, want[k], W, k)
    (spike, voltage, thsum), fin = ops.alif_fwd(*args, dynamics_mode=False)
    assert_exact(spike, want['spike'], 'spike')
    assert_exact(thsum, want['threshold'] + want['refractory'], 'threshold + refractory')
    assert_exact(fin['final_th'], want['threshold'][..., -1], 'final threshold')
    assert_exact(fin['final_ref'], want['refractory'][..., -1], 'final refractory')
    assert_exact(fin['final_s'], want['spike'][..., -1], 'final spike')
    gx, _, _ = ops.cuba_bwd(dev(gs, cuda), voltage, thsum, None, dev(cd, cuda), dev(vd, cuda), 100.0, 0.1, False,
                            False)
    g_v = O.spike_bwd(want['voltage'], want['threshold'] + want['refractory'], gs, 100.0, 0.1, False)
    assert_close(gx, want['grad_x'], 'grad_x', scale=li_scale(li_scale(g_v, vd), cd))


@pytest.mark.parametrize('shape', SHAPES)
@pytest.mark.parametrize('per_channel', [False, True])
@pytest.mark.parametrize('adaptive', [False, True])
def test_rf_fused(shape, per_channel, adaptive, cuda, ops):
    rng = rng_for('rf', shape, per_channel, adaptive)
    B, C, T = shape
    n = C if per_channel else 1
    sd, cd = sincos(rng, n)
    td, rd = decays(rng, n, 300, 500), decays(rng, n, 300, 500)
    re_in = rng.normal(0, 0.5, size=shape).astype(np.float32)
    im_in = rng.normal(0, 0.5, size=shape).astype(np.float32)
    rs, ims = quant(rng.normal(0, 0.3, size=shape[:-1])), quant(rng.normal(0, 0.3, size=shape[:-1]))
    ths = quant(rng.uniform(0.3, 0.8, size=shape[:-1]))
    refs = quant(rng.uniform(0.0, 0.3, size=shape[:-1]))
    gs = rng.normal(size=shape).astype(np.float32)
    for graded in (False, True):
        if adaptive:
            want = O.adrf(re_in, im_in, 0.5, 0.25, sd, cd, td, rd, re_state=rs, im_state=ims, th_state=ths,
                          ref_state=refs, grad_spike=gs, graded=graded)
            ad = dict(ref_decay=dev(rd, cuda), th_decay=dev(td, cuda), ref_state=dev(refs, cuda),
                      th_state=dev(ths, cuda), th_step=0.25, th0=0.5)
            tau, srho = 50.0, 0.1
        else:
            want = O.rf(re_in, im_in, 0.5, sd, cd, re_state=rs, im_state=ims, grad_spike=gs, graded=graded)
            ad = None
            tau, srho = 0.25, 10.0
        outs, fin = ops.rf_fwd(dev(re_in, cuda), dev(im_in, cuda), dev(sd, cuda), dev(cd, cuda), dev(rs, cuda),
                               dev(ims, cuda), 0.5, W, graded=graded, adaptive=ad)
        assert_exact(outs[0], want['spike'], 'spike')
        assert_quantised_equal(outs[1], want['real'], W, 'real')
        assert_quantised_equal(outs[2], want['imag'], W, 'imag')
        assert_exact(fin['final_s'], want['spike'][..., -1], 'final spike')
        thr = 0.5
        if adaptive:
            assert_exact(outs[3], want['threshold'] + want['refractory'], 'threshold + refractory')
            thr = outs[3]
            dyn, _ = ops.rf_fwd(dev(re_in, cuda), dev(im_in, cuda), dev(sd, cuda), dev(cd, cuda), dev(rs, cuda),
                                dev(ims, cuda), 0.5, W, adaptive=ad, dynamics_mode=True)
            for o, k in zip(dyn, ('real', 'imag', 'threshold', 'refractory')):
                assert_quantised_equal(o, want[k], W, k)
        gre, gim, gsn, gcs = ops.rf_bwd(dev(gs, cuda), outs[1], outs[2], thr, dev(sd, cuda), dev(cd, cuda), tau,
                                        srho, graded, True)
        thr_np = (want['threshold'] + want['refractory']) if adaptive else 0.5
        s_re, s_im = cspike_term_scale(want['real'], want['imag'], thr_np, gs, tau, srho, graded)
        S_re, S_im = res_scale(s_re, s_im, sd, cd)
        S_p = pgrad_scale(sd.size, (want['grad_re'], want['real']), (want['grad_re'], want['imag']),
                          (want['grad_im'], want['real']), (want['grad_im'], want['imag']))
        assert_close(gre, want['grad_re'], 'grad_re', scale=S_re)
        assert_close(gim, want['grad_im'], 'grad_im', scale=S_im)
        assert_close(gsn, want['grad_sin_decay'], 'grad_sin', scale=S_p)
        assert_close(gcs, want['grad_cos_decay'], 'grad_cos', scale=S_p)


# --------------------------------------------------------------------------
# sigma-delta family
# --------------------------------------------------------------------------
@pytest.mark.parametrize('shape', SHAPES)
@pytest.mark.parametrize('misalign', [False, True])
def test_sigma(shape, misalign, cuda, ops):
    rng = rng_for('sigma', shape)
    x = rng.normal(0.1, 1.0, size=shape).astype(np.float32)
    st = rng.normal(size=shape[:-1]).astype(np.float32)
    out, fin = ops.sigma_fwd(dev(x, cuda, misalign), None, want_final=True)
    want = O.sigma(x)
    assert_exact(out, want, 'running sum')
    assert_exact(fin, want[..., -1], 'final state')
    assert_exact(ops.sigma_fwd(dev(x, cuda, misalign), dev(st, cuda)), O.sigma(x, st), 'running sum on a kept state')
    assert_exact(ops.sigma_bwd(dev(x, cuda, misalign)), O.sigma(x, reverse=True), 'adjoint')


@pytest.mark.parametrize('shape', SHAPES)
@pytest.mark.parametrize('per_channel', [False, True])
def test_delta(shape, per_channel, cuda, ops):
    rng = rng_for('delta', shape, per_channel)
    n = shape[1] if per_channel else 1
    x = np.cumsum(rng.normal(0, 0.3, size=shape), axis=-1).astype(np.float32)
    thr = rng.uniform(0.1, 0.6, size=n).astype(np.float32)
    pre = rng.normal(size=shape[:-1]).astype(np.float32)
    res = rng.normal(0, 0.1, size=shape[:-1]).astype(np.float32)
    go = rng.normal(size=shape).astype(np.float32)
    for states in ((None, None), (pre, res)):
        want = O.delta_fwd(x, thr, states[0], states[1], 4096)
        sd = [None if s is None else dev(s, cuda) for s in states]
        out, dlt, fres = ops.delta_fwd(dev(x, cuda), dev(thr, cuda), sd[0], sd[1], 4096, want_delta=True)
        assert_exact(out, want['out'], 'delta output')
        assert_exact(dlt, want['delta_input'], 'difference')
        assert_exact(fres, want['residual'], 'final residual')
        out2, none, _ = ops.delta_fwd(dev(x, cuda), dev(thr, cuda), sd[0], sd[1], 4096, want_delta=False)
        assert none is None
        assert_exact(out2, want['out'], 'delta output (difference not saved)')
    assert_exact(ops.delta_fwd(dev(x, cuda), dev(thr, cuda), None, None, 0, False)[0],
                 O.delta_fwd(x, thr, scale=0)['out'], 'unquantised')
    gx_want, gthr_want = O.delta_bwd(go, want['delta_input'], thr, 0.7, 1.3)
    gx, gthr = ops.delta_bwd(dev(go, cuda), dlt, dev(thr, cuda), 0.7, 1.3, True)
    assert_exact(gx, gx_want, 'grad_x')
    # scale of the threshold gradient: the sum of the magnitudes of its terms
    d = want['delta_input'].astype(np.float64)
    th = thr.astype(np.float64).reshape((1, -1) + (1,) * (len(shape) - 2)) if n > 1 else float(thr[0])
    sub = np.abs(d) - th
    mag = np.where(sub > 0, np.abs(d) * 1.3 * np.exp(-np.abs(sub) / 0.7) / th, 1.0) * np.abs(go)
    scale = mag.sum(axis=tuple(i for i in range(mag.ndim) if i != 1)) if n > 1 else np.array([mag.sum()])
    assert_close(gthr, gthr_want, 'grad threshold', scale=scale + 1e-30)
    assert_exact(ops.delta_bwd(dev(go, cuda), None, dev(thr, cuda), 1.0, 1.0, False)[0], gx_want, 'grad_x only')


@pytest.mark.parametrize('shape', SHAPES + [(2, 3, 4, 64), (1, 2, 3, 5, 40)])
@pytest.mark.parametrize('bias_kind', ['none', 'scalar', 'neuron'])
def test_sigma_delta_relu_fused(shape, bias_kind, cuda, ops):
    rng = rng_for('sdnn', shape, bias_kind)
    x = rng.normal(0.02, 0.15, size=shape).astype(np.float32)
    thr = rng.uniform(0.05, 0.2, size=shape[1]).astype(np.float32)
    bias = {'none': None, 'scalar': np.array([0.05], np.float32),
            'neuron': rng.normal(0, 0.2, size=shape[1:-1]).astype(np.float32)}[bias_kind]
    ss = rng.normal(0, 0.3, size=shape[:-1]).astype(np.float32)
    pre = np.abs(rng.normal(0, 0.3, size=shape[:-1])).astype(np.float32)
    res = rng.normal(0, 0.05, size=shape[:-1]).astype(np.float32)
    for states in ((None, None, None), (ss, pre, res)):
        want = O.sdnn_relu(x, thr, bias, states[0], states[1], states[2], 4096)
        sd = [None if s is None else dev(s, cuda) for s in states]
        r = ops.sdnn_relu_fwd(dev(x, cuda), dev(thr, cuda), None if bias is None else dev(bias, cuda), sd[0], sd[1],
                              sd[2], 4096)
        assert_exact(r['out'], want['out'], 'sigma-delta relu output')
        assert_exact(r['final_sigma'], want['sigma'][..., -1], 'sigma state')
        assert_exact(r['final_pre'], want['pre'], 'delta pre state')
        assert_exact(r['final_residual'], want['residual'], 'delta residual state')
    # training variant: same output, activation and difference saved, one-pass backward
    r = ops.sdnn_relu_fwd(dev(x, cuda), dev(thr, cuda), None if bias is None else dev(bias, cuda), sd[0], sd[1], sd[2],
                          4096, want_act=True, want_delta=True)
    assert_exact(r['out'], want['out'], 'output with saves')
    assert_exact(r['activation'], want['act'], 'saved activation')
    assert_exact(r['delta_input'], want['delta_input'], 'saved difference')
    go = rng.normal(size=shape).astype(np.float32)
    g_act, gthr_want = O.delta_bwd(go, want['delta_input'], thr, 0.7, 1.3)
    gx_want = O.sigma((g_act * (want['act'] > 0)).astype(np.float32), reverse=True)
    gx, gthr = ops.sdnn_relu_bwd(dev(go, cuda), r['activation'], r['delta_input'], dev(thr, cuda), 0.7, 1.3, True)
    assert_exact(gx, gx_want, 'grad_x, one-pass backward')
    d = want['delta_input'].astype(np.float64)
    th = thr.astype(np.float64).reshape((1, -1) + (1,) * (len(shape) - 2))
    sub = np.abs(d) - th
    mag = np.where(sub > 0, np.abs(d) * 1.3 * np.exp(-np.abs(sub) / 0.7) / th, 1.0) * np.abs(go)
    assert_close(gthr, gthr_want, 'grad threshold', scale=mag.sum(axis=tuple(i for i in range(mag.ndim) if i != 1)) + 1e-30)
    assert_exact(ops.sdnn_relu_bwd(dev(go, cuda), r['activation'], None, dev(thr, cuda), 1.0, 1.0, False)[0], gx_want,
                 'grad_x only')


def test_empty_inputs(cuda, ops):
    for shape in ((0, 4, 16), (2, 4, 0)):
        x = torch.empty(shape, device=cuda)
        st = torch.zeros(shape[:-1], device=cuda)
        d = torch.tensor([100.0], device=cuda)
        assert ops.li_fwd(x, d, st, W).shape == x.shape
        assert ops.shift(x, 3).shape == x.shape
        assert ops.fir(x, torch.ones(4, device=cuda), 1.0, False).shape == x.shape
        assert ops.spike_fwd(x, 1.0, False, 1).shape == x.shape


def test_device_status_clean(cuda):
    from lava_dl_b200 import _native
    assert _native.device_status() == 0


def _recurrent_scale(voltage, grad_spike, rec, thr, graded):
    """Magnitude of the terms that make up grad_z of the recurrent walk: the same
    reverse recursion on absolute values."""
    B, C, T = voltage.shape
    out = np.zeros_like(voltage, dtype=np.float64)
    carry = np.zeros((B, C))
    sg = np.abs(O.spike_bwd(voltage, thr, np.ones_like(voltage), 125.0, 0.1, graded)).astype(np.float64)
    for t in range(T - 1, -1, -1):
        out[..., t] = sg[..., t] * (np.abs(grad_spike[..., t]) + carry)
        carry = out[..., t] @ np.abs(rec).astype(np.float64)
    return out


@pytest.mark.parametrize('shape', [(1, 1, 1), (2, 3, 2), (3, 40, 50), (2, 33, 36), (5, 257, 67), (2, 1024, 33),
                                   (4, 512, 100), (1, 100, 300),
                                   (151, 48, 20), (150, 130, 9)])   # more samples than SMs: two per CTA in the backward
@pytest.mark.parametrize('graded', [False, True])
@pytest.mark.parametrize('per_neuron', [False, True])
def test_cuba_recurrent(shape, graded, per_neuron, cuda, ops):
    """One launch for s[t] = CUBA(z[t] + R s[t-1]) and its gradient, against the oracle's
    step-by-step walk (one neuron call per time step, state handed over)."""
    B, C, T = shape
    rng = rng_for('cuba_recurrent', shape, graded, per_neuron)
    z = rng.normal(0.25, 0.9, size=shape).astype(np.float32)
    # recurrent weights on the 8-bit grid (multiples of 2/64), mostly inhibitory so activity stays bounded
    rec = (np.round(rng.normal(-0.02, 0.5 / np.sqrt(C), size=(C, C)) * 32) / 32).astype(np.float32)
    n = C if per_neuron else 1
    cd = np.round(rng.uniform(400, 1600, size=n)).astype(np.float32)
    vd = np.round(rng.uniform(60, 600, size=n)).astype(np.float32)
    cs = (np.round(rng.normal(0, 0.5, size=(B, C)) * W) / W).astype(np.float32)
    vs = (np.round(rng.uniform(-0.5, 1.0, size=(B, C)) * W) / W).astype(np.float32)
    gs = rng.normal(size=shape).astype(np.float32)
    thr = 1.25 + 0.01 / W
    want = O.cuba_recurrent(z, rec, 1.25, cd, vd, cstate=cs, vstate=vs, grad_spike=gs, graded=graded)
    r = ops.cuba_recurrent_fwd(dev(z, cuda), dev(rec, cuda), dev(cd, cuda), dev(vd, cuda), dev(cs, cuda),
                               dev(vs, cuda), thr, W, graded=graded)
    if graded:
        # graded spike values times weights are inexact in fp32: the order of the feedback sum shows
        assert_exact(r['spike'] != 0, want['spike'] != 0, 'spike pattern')
        assert_close(r['spike'], want['spike'], 'graded spike values')
        assert_close(r['voltage'], want['voltage'], 'voltage', scale=1.0)
    else:
        assert_exact(r['spike'], want['spike'], 'spikes')
        assert_quantised_equal(r['voltage'], want['voltage'], W, 'voltage')
        assert_quantised_equal(r['final_c'], want['final_c'], W, 'final current')
        fv = r['final_v'] * (1 - (r['final_s'] > 0).float())
        assert_quantised_equal(fv, want['final_v'], W, 'final voltage after hand-over')
    gz = ops.cuba_recurrent_bwd(dev(gs, cuda), dev(want['voltage'], cuda), dev(rec, cuda), thr, 125.0, 0.1, graded)
    assert_close(gz, want['grad_z'], 'grad_z', scale=_recurrent_scale(want['voltage'], gs, rec, thr, graded))
