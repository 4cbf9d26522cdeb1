"""The CPU oracle against outputs of lava-dl itself (tests/golden/*.npz, made by
tests/golden/make_golden.py).  This is what pins the oracle; it runs without a
GPU."""

import numpy as np
import pytest

from _util import (assert_close, assert_exact, assert_quantised_equal, golden_cases, load_golden)
from oracle import oracle as O


def thr_of(g):
    t = g['threshold']
    return None if (t.ndim == 0 and float(t) < 0) else (float(t) if t.ndim == 0 else t)


@pytest.mark.parametrize('name', golden_cases('li_'))
def test_leaky_integrator(name):
    g = load_golden(name)
    w = int(g['w_scale'])
    y = O.li_fwd(g['x'], g['decay'], g['state'], w, thr_of(g))
    if w & (w - 1) == 0:
        assert_quantised_equal(y, g['y'], w, 'li output')
    assert_exact(y, g['y'], 'li output')
    if 'grad_in' in g:
        gi, gd = O.li_bwd(g['grad_out'], g['y'], g['decay'])
        assert_close(gi, g['grad_in'], 'li grad_in')
        assert_close(gd, g['grad_decay'], 'li grad_decay')


@pytest.mark.parametrize('name', golden_cases('ath_'))
def test_adaptive_threshold(name):
    g = load_golden(name)
    w = int(g['w_scale'])
    th, ref = O.ath_fwd(g['x'], g['ref_state'], g['ref_decay'], g['th_state'], g['th_decay'],
                        float(g['th_scale']), float(g['th0']), w)
    assert_quantised_equal(th, g['threshold'], w, 'threshold')
    assert_quantised_equal(ref, g['refractory'], w, 'refractory')


@pytest.mark.parametrize('name', golden_cases('apth_'))
def test_adaptive_phase_threshold(name):
    g = load_golden(name)
    w = int(g['w_scale'])
    th, ref = O.apth_fwd(g['re'], g['im'], g['im_state'], g['ref_state'], g['ref_decay'], g['th_state'],
                         g['th_decay'], float(g['th_scale']), float(g['th0']), w)
    assert_quantised_equal(th, g['threshold'], w, 'threshold')
    assert_quantised_equal(ref, g['refractory'], w, 'refractory')


@pytest.mark.parametrize('name', golden_cases('res_'))
def test_resonator(name):
    g = load_golden(name)
    w = int(g['w_scale'])
    re, im = O.res_fwd(g['re_in'], g['im_in'], g['sin_decay'], g['cos_decay'], g['re_state'], g['im_state'], w,
                       thr_of(g))
    assert_quantised_equal(re, g['re'], w, 'real')
    assert_quantised_equal(im, g['im'], w, 'imag')
    a, b, gs, gc = O.res_bwd(g['grad_re'], g['grad_im'], g['re'], g['im'], g['sin_decay'], g['cos_decay'])
    assert_close(a, g['grad_re_in'], 'grad_re_in')
    assert_close(b, g['grad_im_in'], 'grad_im_in')
    assert_close(gs, g['grad_sin'], 'grad_sin')
    assert_close(gc, g['grad_cos'], 'grad_cos')


@pytest.mark.parametrize('name', golden_cases('adres_'))
def test_adaptive_resonator(name):
    g = load_golden(name)
    w = int(g['w_scale'])
    re, im, th, ref = O.adres_fwd(g['re_in'], g['im_in'], g['sin_decay'], g['cos_decay'], g['ref_decay'],
                                  g['th_decay'], g['re_state'], g['im_state'], g['ref_state'], g['th_state'],
                                  float(g['th_scale']), float(g['th0']), w)
    for got, key in ((re, 're'), (im, 'im'), (th, 'threshold'), (ref, 'refractory')):
        assert_quantised_equal(got, g[key], w, key)
    a, b, gs, gc = O.res_bwd(g['grad_re'], g['grad_im'], g['re'], g['im'], g['sin_decay'], g['cos_decay'])
    assert_close(a, g['grad_re_in'], 'grad_re_in')
    assert_close(b, g['grad_im_in'], 'grad_im_in')
    assert_close(gs, g['grad_sin'], 'grad_sin')
    assert_close(gc, g['grad_cos'], 'grad_cos')


@pytest.mark.parametrize('name', golden_cases('spike_'))
def test_spike(name):
    g = load_golden(name)
    thr = g['threshold'] if g['threshold'].ndim else float(g['threshold'])
    graded = bool(g['graded'])
    s = O.spike_fwd(g['v'], thr, graded, 1)
    assert_exact(s, g['spike'], 'spike')
    gv = O.spike_bwd(g['v'], thr, g['grad_spike'], float(g['tau_rho']), float(g['scale_rho']), graded)
    assert_close(gv, g['grad_v'], 'grad_v')


@pytest.mark.parametrize('name', golden_cases('cspike_'))
def test_complex_spike(name):
    g = load_golden(name)
    thr = g['threshold'] if g['threshold'].ndim else float(g['threshold'])
    graded = bool(g['graded'])
    s = O.cspike_fwd(g['re'], g['im'], thr, g['imag_last'], graded, 1)
    assert_exact(s, g['spike'], 'spike')
    gre, gim = O.cspike_bwd(g['re'], g['im'], thr, g['grad_spike'], float(g['tau_rho']), float(g['scale_rho']),
                            graded)
    assert_close(gre, g['grad_re'], 'grad_re')
    assert_close(gim, g['grad_im'], 'grad_im')


@pytest.mark.parametrize('name', golden_cases('shift_'))
def test_shift(name):
    g = load_golden(name)
    sv = g['shift'] if g['shift'].ndim else float(g['shift'])
    assert_exact(O.shift(g['x'], sv, float(g['sampling_time'])), g['out'], 'shift')


@pytest.mark.parametrize('name', golden_cases('fir_'))
def test_fir(name):
    g = load_golden(name)
    ts = float(g['sampling_time'])
    assert_close(O.conv(g['x'], g['filter'], ts), g['conv'], 'conv')
    assert_close(O.corr(g['x'], g['filter'], ts), g['corr'], 'corr')
    assert_close(O.corr(g['grad_out'], g['filter'], ts), g['grad_conv'], 'conv backward')


def test_delay_filter_chain():
    g = load_golden('delay_fir_chain')
    y = O.conv(O.shift(g['x'], g['delay']), g['filter'])
    assert_close(y, g['out'], 'conv(delay(x))')
    gx = O.shift(O.corr(g['grad_out'], g['filter']), -g['delay'])
    assert_close(gx, g['grad_x'], 'grad_x')


# --------------------------------------------------------------------------
# neuron-level sequences
# --------------------------------------------------------------------------
S = 4096


@pytest.mark.parametrize('name', golden_cases('neuron_cuba_'))
def test_cuba_neuron(name):
    g = load_golden(name)
    graded = 'graded' in name
    r = O.cuba(g['x'], 1.25, g['param_current_decay'], g['param_voltage_decay'], grad_spike=g['grad_spike'],
               graded=graded)
    assert_exact(r['spike'], g['spike'], 'spike')
    assert_quantised_equal(r['current'], g['dyn0'], S, 'current')
    assert_quantised_equal(r['voltage'], g['dyn1'], S, 'voltage')
    assert_close(r['grad_x'], g['grad_in0'], 'grad_x')
    if 'grad_current_decay' in g:
        assert_close(r['grad_current_decay'], g['grad_current_decay'], 'grad current decay')
        assert_close(r['grad_voltage_decay'], g['grad_voltage_decay'], 'grad voltage decay')


@pytest.mark.parametrize('name', golden_cases('neuron_alif_'))
def test_alif_neuron(name):
    g = load_golden(name)
    r = O.alif(g['x'], 1.0, 0.5, g['param_current_decay'], g['param_voltage_decay'], g['param_threshold_decay'],
               g['param_refractory_decay'], grad_spike=g['grad_spike'])
    assert_exact(r['spike'], g['spike'], 'spike')
    for i, k in enumerate(('current', 'voltage', 'threshold', 'refractory')):
        assert_quantised_equal(r[k], g[f'dyn{i}'], S, k)
    assert_close(r['grad_x'], g['grad_in0'], 'grad_x')
    if 'grad_current_decay' in g:
        assert_close(r['grad_current_decay'], g['grad_current_decay'], 'grad current decay')
        assert_close(r['grad_voltage_decay'], g['grad_voltage_decay'], 'grad voltage decay')


def test_rf_neuron():
    g = load_golden('neuron_rf_shared')
    r = O.rf(g['re_in'], g['im_in'], 0.5, g['param_sin_decay'], g['param_cos_decay'], grad_spike=g['grad_spike'])
    assert_exact(r['spike'], g['spike'], 'spike')
    assert_quantised_equal(r['real'], g['dyn0'], S, 'real')
    assert_quantised_equal(r['imag'], g['dyn1'], S, 'imag')
    assert_close(r['grad_re'], g['grad_in0'], 'grad_re')
    assert_close(r['grad_im'], g['grad_in1'], 'grad_im')
    assert_close(r['grad_sin_decay'], g['grad_sin_decay'], 'grad_sin')
    assert_close(r['grad_cos_decay'], g['grad_cos_decay'], 'grad_cos')


@pytest.mark.parametrize('name', golden_cases('neuron_adrf_'))
def test_adrf_neuron(name):
    g = load_golden(name)
    r = O.adrf(g['re_in'], g['im_in'], 0.5, 0.25, g['param_sin_decay'], g['param_cos_decay'],
               g['param_threshold_decay'], g['param_refractory_decay'], grad_spike=g['grad_spike'])
    assert_exact(r['spike'], g['spike'], 'spike')
    for i, k in enumerate(('real', 'imag', 'threshold', 'refractory')):
        assert_quantised_equal(r[k], g[f'dyn{i}'], S, k)
    assert_close(r['grad_re'], g['grad_in0'], 'grad_re')
    assert_close(r['grad_im'], g['grad_in1'], 'grad_im')
    if 'grad_sin_decay' in g:
        assert_close(r['grad_sin_decay'], g['grad_sin_decay'], 'grad_sin')
        assert_close(r['grad_cos_decay'], g['grad_cos_decay'], 'grad_cos')


def test_rf_iz_neuron():
    g = load_golden('neuron_rfiz_shared')
    r = O.rf_iz(g['re_in'], g['im_in'], 0.5, g['param_sin_decay'], g['param_cos_decay'], grad_spike=g['grad_spike'])
    assert_exact(r['spike'], g['spike'], 'spike')
    assert_quantised_equal(r['real'], g['dyn0'], S, 'real')
    assert_quantised_equal(r['imag'], g['dyn1'], S, 'imag')
    assert_close(r['grad_re'], g['grad_in0'], 'grad_re')
    assert_close(r['grad_im'], g['grad_in1'], 'grad_im')
    assert_close(r['grad_sin_decay'], g['grad_sin_decay'], 'grad_sin')
    assert_close(r['grad_cos_decay'], g['grad_cos_decay'], 'grad_cos')


def test_adrf_iz_neuron():
    g = load_golden('neuron_adrfiz_shared')
    r = O.adrf_iz(g['re_in'], g['im_in'], 0.5, 0.25, g['param_sin_decay'], g['param_cos_decay'], 410.0, 410.0,
                  grad_spike=g['grad_spike'])
    assert_exact(r['spike'], g['spike'], 'spike')
    for i, k in enumerate(('real', 'imag', 'threshold', 'refractory')):
        assert_quantised_equal(r[k], g[f'dyn{i}'], S, k)
    assert_close(r['grad_re'], g['grad_in0'], 'grad_re')
    assert_close(r['grad_im'], g['grad_in1'], 'grad_im')
    assert_close(r['grad_sin_decay'], g['grad_sin_decay'], 'grad_sin')
    assert_close(r['grad_cos_decay'], g['grad_cos_decay'], 'grad_cos')


# --------------------------------------------------------------------------
# sigma-delta family
# --------------------------------------------------------------------------
def test_sigma():
    g = load_golden('sigma_persistent')
    s1 = O.sigma(g['x'])
    assert_exact(s1, g['out1'], 'cumsum')
    assert_exact(O.sigma(g['x'], state=s1[..., -1]), g['out2'], 'cumsum on top of the kept state')
    assert_exact(O.sigma(g['grad_out'], reverse=True), g['grad_x'], 'adjoint')


def test_delta_shared():
    g = load_golden('delta_shared')
    r = O.delta_fwd(g['x'], g['threshold'])
    assert_exact(r['out'], g['out1'], 'delta output')
    gx, gthr = O.delta_bwd(g['grad_out'], r['delta_input'], g['threshold'], float(g['tau_grad']),
                           float(g['scale_grad']))
    assert_exact(gx, g['grad_x'], 'grad_x')
    assert_close(gthr, g['grad_threshold'], 'grad_threshold')
    r2 = O.delta_fwd(g['x'], g['threshold'], pre_state=g['x'][..., -1], residual_state=r['residual'])
    assert_exact(r2['out'], g['out2'], 'second call with kept states')
    assert_exact(r2['residual'], g['residual'], 'residual state')


def test_delta_per_channel():
    g = load_golden('delta_chan_rank4')
    assert_exact(O.delta_fwd(g['x'], g['threshold'])['out'], g['out'], 'delta output, one threshold per channel')


def test_sigma_delta_neuron():
    g = load_golden('neuron_sdnn_shared')
    r = O.sdnn_relu(g['x'], g['threshold'])
    assert_exact(r['out'], g['out1'], 'sigma-delta relu output')
    # backward: delta -> relu mask -> adjoint of the running sum
    g_act, gthr = O.delta_bwd(g['grad_out'], r['delta_input'], g['threshold'], float(g['tau_grad']),
                              float(g['scale_grad']))
    gx = O.sigma((g_act * (r['act'] > 0)).astype(np.float32), reverse=True)
    assert_close(gx, g['grad_x'], 'grad_x')
    assert_close(gthr, g['grad_threshold'], 'grad_threshold')
    r2 = O.sdnn_relu(g['x'], g['threshold'], sigma_state=r['sigma'][..., -1], pre_state=r['pre'],
                     residual_state=r['residual'])
    assert_exact(r2['out'], g['out2'], 'second call with kept states')
    g = load_golden('neuron_sdnn_bias_rank4')
    assert_exact(O.sdnn_relu(g['x'], g['threshold'], bias=g['bias'])['out'], g['out'], 'per-neuron bias')


def _dense_q(weight, w_scale=64):
    """Dense synapse weights after the neuron's 8-bit pre-hook (neuron/base.py quantize_8bit)."""
    w = np.asarray(weight, dtype=np.float32).reshape(weight.shape[0], weight.shape[1])
    step = np.float32(2 / w_scale)
    return np.clip(np.round(w / step) * step, -256 / w_scale, 254 / w_scale).astype(np.float32)


def _step_delay(s):
    out = np.zeros_like(s)
    out[..., 1:] = s[..., :-1]
    return out


def test_recurrent_block():
    g = load_golden('block_cuba_recurrent')
    w_in, w_rec = _dense_q(g['weight_in']), _dense_q(g['weight_rec'])
    z = np.einsum('oi,bit->bot', w_in, g['x']).astype(np.float32)
    go = np.zeros_like(g['grad_out'])
    go[..., :-1] = g['grad_out'][..., 1:]           # gradient of the one-step delay
    r = O.cuba_recurrent(z, w_rec, 1.25, 0.25 * 4096, 0.03 * 4096, grad_spike=go)
    assert_exact(_step_delay(r['spike']), g['out1'], 'recurrent spikes')
    assert_close(np.einsum('oi,bot->bit', w_in, r['grad_z']), g['grad_x'], 'grad x')
    assert_close(np.einsum('bot,bit->oi', r['grad_z'], g['x']), g['grad_weight_in'].reshape(w_in.shape), 'grad W')
    assert_close(r['grad_rec'], g['grad_weight_rec'].reshape(w_rec.shape), 'grad R')
    assert not g['grad_current_decay'].any() and not g['grad_voltage_decay'].any()
    r2 = O.cuba_recurrent(z, w_rec, 1.25, 0.25 * 4096, 0.03 * 4096, cstate=r['final_c'], vstate=r['final_v'])
    assert_exact(_step_delay(r2['spike']), g['out2'], 'second call, persistent neuron state')


def test_recurrent_block_graded():
    g = load_golden('block_cuba_recurrent_graded')
    w_in, w_rec = _dense_q(g['weight_in']), _dense_q(g['weight_rec'])
    z = np.einsum('oi,bit->bot', w_in, g['x']).astype(np.float32)
    r = O.cuba_recurrent(z, w_rec, 1.25, g['current_decay'], g['voltage_decay'], graded=True)
    # the case is built so that every product and sum is exact in fp32 (see make_golden.py)
    assert_quantised_equal(r['spike'], g['out'], S, 'graded recurrent spikes')
