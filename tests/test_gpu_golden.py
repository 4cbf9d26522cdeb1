"""The CUDA path, driven through the lava-dl-shaped Python API, against outputs
of lava-dl itself (tests/golden/*.npz).  Mirrors test_oracle_golden.py."""

import numpy as np
import pytest
import torch

from _util import (assert_close, assert_exact, assert_quantised_equal, cspike_term_scale, golden_cases, li_scale,
                   load_golden, pgrad_scale, res_scale)
from oracle import oracle as O

pytestmark = pytest.mark.gpu

S = 4096


def T(a, cuda, grad=False):
    t = torch.tensor(np.asarray(a), dtype=torch.float32, device=cuda)
    return t.requires_grad_(True) if grad else t


def thr_of(g):
    t = g['threshold']
    return None if (t.ndim == 0 and float(t) < 0) else float(t)


@pytest.fixture(scope='module')
def slayer(cuda):
    import lava_dl_b200.slayer as s
    return s


@pytest.mark.parametrize('name', golden_cases('li_'))
def test_leaky_integrator(name, cuda, slayer):
    g = load_golden(name)
    w = int(g['w_scale'])
    li = slayer.neuron.dynamics.leaky_integrator
    x, dec = T(g['x'], cuda, True), T(g['decay'], cuda, True)
    y = li.dynamics(x, dec, T(g['state'], cuda), w, threshold=thr_of(g), debug=(w & (w - 1) == 0))
    assert_exact(y, g['y'], 'li output')
    if 'grad_in' in g:
        y.backward(T(g['grad_out'], cuda))
        assert_close(x.grad, g['grad_in'], 'li grad_in', scale=li_scale(g['grad_out'], g['decay']))
        assert_close(dec.grad, g['grad_decay'], 'li grad_decay',
                     scale=pgrad_scale(g['decay'].size, (g['grad_in'], g['y'])))


@pytest.mark.parametrize('name', golden_cases('ath_'))
def test_adaptive_threshold(name, cuda, slayer):
    g = load_golden(name)
    w = int(g['w_scale'])
    th, ref = slayer.neuron.dynamics.adaptive_threshold.dynamics(
        T(g['x'], cuda), T(g['ref_state'], cuda), T(g['ref_decay'], cuda), T(g['th_state'], cuda),
        T(g['th_decay'], cuda), float(g['th_scale']), float(g['th0']), w, debug=True)
    assert_quantised_equal(th, g['threshold'], w, 'threshold')
    assert_quantised_equal(ref, g['refractory'], w, 'refractory')


@pytest.mark.parametrize('name', golden_cases('apth_'))
def test_adaptive_phase_threshold(name, cuda, slayer):
    g = load_golden(name)
    w = int(g['w_scale'])
    th, ref = slayer.neuron.dynamics.adaptive_phase_th.dynamics(
        T(g['re'], cuda), T(g['im'], cuda), T(g['im_state'], cuda), T(g['ref_state'], cuda),
        T(g['ref_decay'], cuda), T(g['th_state'], cuda), T(g['th_decay'], cuda), float(g['th_scale']),
        float(g['th0']), w)
    assert_quantised_equal(th, g['threshold'], w, 'threshold')
    assert_quantised_equal(ref, g['refractory'], w, 'refractory')


@pytest.mark.parametrize('name', golden_cases('res_'))
def test_resonator(name, cuda, slayer):
    g = load_golden(name)
    w = int(g['w_scale'])
    re_in, im_in = T(g['re_in'], cuda, True), T(g['im_in'], cuda, True)
    sd, cd = T(g['sin_decay'], cuda, True), T(g['cos_decay'], cuda, True)
    re, im = slayer.neuron.dynamics.resonator.dynamics(
        re_in, im_in, sd, cd, T(g['re_state'], cuda), T(g['im_state'], cuda), w, threshold=thr_of(g))
    assert_quantised_equal(re, g['re'], w, 'real')
    assert_quantised_equal(im, g['im'], w, 'imag')
    (re * T(g['grad_re'], cuda) + im * T(g['grad_im'], cuda)).sum().backward()
    S_re, S_im = res_scale(g['grad_re'], g['grad_im'], g['sin_decay'], g['cos_decay'])
    S_p = pgrad_scale(g['sin_decay'].size, (g['grad_re_in'], g['re']), (g['grad_re_in'], g['im']),
                      (g['grad_im_in'], g['re']), (g['grad_im_in'], g['im']))
    assert_close(re_in.grad, g['grad_re_in'], 'grad_re_in', scale=S_re)
    assert_close(im_in.grad, g['grad_im_in'], 'grad_im_in', scale=S_im)
    assert_close(sd.grad, g['grad_sin'], 'grad_sin', scale=S_p)
    assert_close(cd.grad, g['grad_cos'], 'grad_cos', scale=S_p)


@pytest.mark.parametrize('name', golden_cases('adres_'))
def test_adaptive_resonator(name, cuda, slayer):
    g = load_golden(name)
    w = int(g['w_scale'])
    re_in, im_in = T(g['re_in'], cuda, True), T(g['im_in'], cuda, True)
    sd, cd = T(g['sin_decay'], cuda, True), T(g['cos_decay'], cuda, True)
    re, im, th, ref = slayer.neuron.dynamics.adaptive_resonator.dynamics(
        re_in, im_in, sd, cd, T(g['ref_decay'], cuda), T(g['th_decay'], cuda), T(g['re_state'], cuda),
        T(g['im_state'], cuda), T(g['ref_state'], cuda), T(g['th_state'], cuda), float(g['th_scale']),
        float(g['th0']), w)
    for got, key in ((re, 're'), (im, 'im'), (th, 'threshold'), (ref, 'refractory')):
        assert_quantised_equal(got, g[key], w, key)
    (re * T(g['grad_re'], cuda) + im * T(g['grad_im'], cuda)).sum().backward()
    S_re, S_im = res_scale(g['grad_re'], g['grad_im'], g['sin_decay'], g['cos_decay'])
    S_p = pgrad_scale(g['sin_decay'].size, (g['grad_re_in'], g['re']), (g['grad_re_in'], g['im']),
                      (g['grad_im_in'], g['re']), (g['grad_im_in'], g['im']))
    assert_close(re_in.grad, g['grad_re_in'], 'grad_re_in', scale=S_re)
    assert_close(im_in.grad, g['grad_im_in'], 'grad_im_in', scale=S_im)
    assert_close(sd.grad, g['grad_sin'], 'grad_sin', scale=S_p)
    assert_close(cd.grad, g['grad_cos'], 'grad_cos', scale=S_p)


@pytest.mark.parametrize('name', golden_cases('spike_'))
def test_spike(name, cuda, slayer):
    g = load_golden(name)
    thr = T(g['threshold'], cuda) if g['threshold'].ndim else float(g['threshold'])
    graded = bool(g['graded'])
    v = T(g['v'], cuda, True)
    s = slayer.spike.Spike.apply(v, thr, float(g['tau_rho']), float(g['scale_rho']), graded,
                                 torch.zeros(v.shape[:-1], device=cuda), 1)
    assert_exact(s, g['spike'], 'spike')
    s.backward(T(g['grad_spike'], cuda))
    assert_close(v.grad, g['grad_v'], 'grad_v')


@pytest.mark.parametrize('name', golden_cases('cspike_'))
def test_complex_spike(name, cuda, slayer):
    g = load_golden(name)
    thr = T(g['threshold'], cuda) if g['threshold'].ndim else float(g['threshold'])
    graded = bool(g['graded'])
    re, im = T(g['re'], cuda, True), T(g['im'], cuda, True)
    s = slayer.spike.complex.Spike.apply(re, im, thr, float(g['tau_rho']), float(g['scale_rho']), graded,
                                         T(g['imag_last'], cuda), 1)
    assert_exact(s, g['spike'], 'spike')
    s.backward(T(g['grad_spike'], cuda))
    t_re, t_im = cspike_term_scale(g['re'], g['im'], g['threshold'] if g['threshold'].ndim else float(g['threshold']),
                                   g['grad_spike'], float(g['tau_rho']), float(g['scale_rho']), graded)
    assert_close(re.grad, g['grad_re'], 'grad_re', scale=t_re)
    assert_close(im.grad, g['grad_im'], 'grad_im', scale=t_im)


@pytest.mark.parametrize('name', golden_cases('shift_'))
def test_shift(name, cuda, slayer):
    g = load_golden(name)
    sv = T(g['shift'], cuda) if g['shift'].ndim else float(g['shift'])
    out = slayer.utils.time.shift(T(g['x'], cuda), sv, float(g['sampling_time']))
    assert_exact(out, g['out'], 'shift')


@pytest.mark.parametrize('name', golden_cases('fir_'))
def test_fir(name, cuda, slayer):
    g = load_golden(name)
    ts = float(g['sampling_time'])
    x = T(g['x'], cuda, True)
    f = T(g['filter'], cuda)
    y = slayer.utils.filter.conv(x, f, ts)
    assert_close(y, g['conv'], 'conv')
    y.backward(T(g['grad_out'], cuda))
    assert_close(x.grad, g['grad_conv'], 'conv backward')
    assert_close(slayer.utils.filter.corr(T(g['x'], cuda), f, ts), g['corr'], 'corr')


def test_delay_filter_chain(cuda, slayer):
    g = load_golden('delay_fir_chain')
    x = T(g['x'], cuda, True)
    y = slayer.utils.filter.conv(slayer.axon.delay(x, T(g['delay'], cuda)), T(g['filter'], cuda))
    assert_close(y, g['out'], 'conv(delay(x))')
    y.backward(T(g['grad_out'], cuda))
    assert_close(x.grad, g['grad_x'], 'grad_x')


# --------------------------------------------------------------------------
# neuron classes
# --------------------------------------------------------------------------
def _bind_params(neuron, g, names, arg, cuda):
    """Bind the shape (first call) and then install the golden parameters."""
    with torch.no_grad():
        neuron(arg)
        for k in names:
            getattr(neuron, k).data = T(g[f'param_{k}'], cuda)
        for name, buf in neuron.named_buffers():
            if name.endswith('_state'):
                buf.zero_()
                if name == 'threshold_state':
                    buf.add_(neuron.threshold)
    return neuron


def _neuron_scales(kind, g, neuron):
    """Magnitude scans for the input and parameter gradients of a neuron (see _util)."""
    gs = g['grad_spike']
    graded = bool(neuron.graded_spike)
    if kind in ('cuba', 'alif'):
        cur, vol = g['dyn0'], g['dyn1']
        cd, vd = np.round(g['param_current_decay']), np.round(g['param_voltage_decay'])
        thr = (neuron.threshold + neuron.threshold_eps) if kind == 'cuba' else g['dyn2'] + g['dyn3']
        g_v = O.spike_bwd(vol, thr, gs, neuron.tau_rho * 100, neuron.scale_rho * 0.1, graded)
        g_c, _ = O.li_bwd(g_v, vol, vd)
        return {'grad_in0': li_scale(li_scale(g_v, vd), cd),
                'grad_current_decay': pgrad_scale(cd.size, (g['grad_in0'], cur)),
                'grad_voltage_decay': pgrad_scale(vd.size, (g_c, vol))}
    re, im = g['dyn0'], g['dyn1']
    sd, cd = np.round(g['param_sin_decay']), np.round(g['param_cos_decay'])
    if kind == 'rf':
        thr, tau, srho = neuron.threshold, neuron.tau_rho * 0.5, neuron.scale_rho * 10
    else:
        thr, tau, srho = g['dyn2'] + g['dyn3'], neuron.tau_rho * 100, neuron.scale_rho * 0.1
    s_re, s_im = cspike_term_scale(re, im, thr, gs, tau, srho, graded)
    S_re, S_im = res_scale(s_re, s_im, sd, cd)
    S_p = pgrad_scale(sd.size, (g['grad_in0'], re), (g['grad_in0'], im), (g['grad_in1'], re), (g['grad_in1'], im))
    return {'grad_in0': S_re, 'grad_in1': S_im, 'grad_sin_decay': S_p, 'grad_cos_decay': S_p}


def _check_neuron(make, g, names, input_keys, dyn_keys, split, cuda, kind):
    ins = [T(g[k], cuda, True) for k in input_keys]
    arg = ins[0] if len(ins) == 1 else tuple(ins)
    plain = [T(g[k], cuda) for k in input_keys]
    parg = plain[0] if len(plain) == 1 else tuple(plain)

    n = _bind_params(make().to(cuda), g, names, parg, cuda)
    spike = n(arg)
    assert_exact(spike, g['spike'], 'spike')
    (spike * T(g['grad_spike'], cuda)).sum().backward()
    scales = _neuron_scales(kind, g, n)
    for i, t in enumerate(ins):
        assert_close(t.grad, g[f'grad_in{i}'], f'grad_in{i}', scale=scales[f'grad_in{i}'])
    for k in names:
        if f'grad_{k}' not in g:
            assert getattr(n, k).grad is None, f'{k} is not learnable in this case'
        elif f'grad_{k}' in scales:
            assert_close(getattr(n, k).grad, g[f'grad_{k}'], f'grad_{k}', scale=scales[f'grad_{k}'])
        else:  # threshold / refractory decays: the reference leaves exact zeros
            assert_exact(getattr(n, k).grad, g[f'grad_{k}'], f'grad_{k}')

    with torch.no_grad():
        m = _bind_params(make().to(cuda), g, names, parg, cuda)
        for i, (t, k) in enumerate(zip(m.dynamics(parg), dyn_keys)):
            assert_quantised_equal(t, g[f'dyn{i}'], S, k)

        p = make().to(cuda)
        p.persistent_state = True
        _bind_params(p, g, names, parg, cuda)
        a = [t[..., :split].contiguous() for t in plain]
        b = [t[..., split:].contiguous() for t in plain]
        s1 = p(a[0] if len(a) == 1 else tuple(a))
        s2 = p(b[0] if len(b) == 1 else tuple(b))
        assert_exact(torch.cat([s1, s2], dim=-1), g['spike_split'], 'persistent-state split run')
        assert_exact(torch.cat([s1, s2], dim=-1), g['spike'], 'split run equals one-shot run')
        for name, buf in p.named_buffers():
            if name.endswith('_state'):
                assert_quantised_equal(buf, g[f'final_{name}'], S, f'final {name}')


def test_cuba_shared(cuda, slayer):
    g = load_golden('neuron_cuba_shared')
    _check_neuron(lambda: slayer.neuron.cuba.Neuron(1.25, 0.25, 0.03, requires_grad=True), g,
                  ['current_decay', 'voltage_decay'], ['x'], ['current', 'voltage'], 30, cuda, 'cuba')


def test_cuba_per_channel_graded(cuda, slayer):
    g = load_golden('neuron_cuba_chan_graded')
    _check_neuron(lambda: slayer.neuron.cuba.Neuron(1.25, 0.25, 0.03, shared_param=False, requires_grad=True,
                                                    graded_spike=True), g,
                  ['current_decay', 'voltage_decay'], ['x'], ['current', 'voltage'], 32, cuda, 'cuba')


def test_cuba_rank4(cuda, slayer):
    g = load_golden('neuron_cuba_rank4')
    _check_neuron(lambda: slayer.neuron.cuba.Neuron(1.25, 0.25, 0.03), g, ['current_decay', 'voltage_decay'],
                  ['x'], ['current', 'voltage'], 32, cuda, 'cuba')


ALIF_P = ['current_decay', 'voltage_decay', 'threshold_decay', 'refractory_decay']


def test_alif_shared(cuda, slayer):
    g = load_golden('neuron_alif_shared')
    _check_neuron(lambda: slayer.neuron.alif.Neuron(1.0, 0.5, 0.2, 0.05, 0.1, 0.1), g, ALIF_P, ['x'],
                  ['current', 'voltage', 'threshold', 'refractory'], 40, cuda, 'alif')


def test_alif_per_channel(cuda, slayer):
    g = load_golden('neuron_alif_chan')
    _check_neuron(lambda: slayer.neuron.alif.Neuron(1.0, 0.5, 0.2, 0.05, 0.1, 0.1, shared_param=False,
                                                    requires_grad=True), g, ALIF_P, ['x'],
                  ['current', 'voltage', 'threshold', 'refractory'], 33, cuda, 'alif')


def test_rf_shared(cuda, slayer):
    g = load_golden('neuron_rf_shared')
    _check_neuron(lambda: slayer.neuron.rf.Neuron(0.5, 10, 0.1, requires_grad=True), g,
                  ['sin_decay', 'cos_decay'], ['re_in', 'im_in'], ['real', 'imag'], 37, cuda, 'rf')


ADRF_P = ['sin_decay', 'cos_decay', 'threshold_decay', 'refractory_decay']


def test_adrf_per_channel(cuda, slayer):
    g = load_golden('neuron_adrf_chan')
    _check_neuron(lambda: slayer.neuron.adrf.Neuron(0.5, 0.25, [10, 40], 0.1, 0.1, 0.1, shared_param=False,
                                                    requires_grad=True), g, ADRF_P, ['re_in', 'im_in'],
                  ['real', 'imag', 'threshold', 'refractory'], 32, cuda, 'adrf')


def test_adrf_shared(cuda, slayer):
    g = load_golden('neuron_adrf_shared')
    _check_neuron(lambda: slayer.neuron.adrf.Neuron(0.5, 0.25, 12, 0.1, 0.1, 0.1), g, ADRF_P,
                  ['re_in', 'im_in'], ['real', 'imag', 'threshold', 'refractory'], 50, cuda, 'adrf')


# --------------------------------------------------------------------------
# Izhikevich-reset variants: dynamics() + spike() (the reference's adrf_iz.forward is broken)
# --------------------------------------------------------------------------
def _check_iz(make, g, oracle_run, cuda):
    ins = [T(g['re_in'], cuda, True), T(g['im_in'], cuda, True)]
    n = make().to(cuda)
    dyn = n.dynamics(tuple(ins))
    spike = n.spike(*dyn)
    assert_exact(spike, g['spike'], 'spike')
    for i, t in enumerate(dyn):
        assert_quantised_equal(t, g[f'dyn{i}'], S, f'dyn{i}')
    (spike * T(g['grad_spike'], cuda)).sum().backward()
    want = oracle_run()
    S_re, S_im = res_scale(np.zeros_like(want['grad_imag_series']), want['grad_imag_series'],
                           np.round(g['param_sin_decay']), np.round(g['param_cos_decay']))
    S_p = pgrad_scale(1, (g['grad_in0'], g['dyn0']), (g['grad_in0'], g['dyn1']), (g['grad_in1'], g['dyn0']),
                      (g['grad_in1'], g['dyn1']))
    assert_close(ins[0].grad, g['grad_in0'], 'grad_re', scale=S_re)
    assert_close(ins[1].grad, g['grad_in1'], 'grad_im', scale=S_im)
    assert_close(n.sin_decay.grad, g['grad_sin_decay'], 'grad_sin', scale=S_p)
    assert_close(n.cos_decay.grad, g['grad_cos_decay'], 'grad_cos', scale=S_p)
    with torch.no_grad():
        p = make().to(cuda)
        p.persistent_state = True
        outs = []
        for sl in (slice(None, 41), slice(41, None)):
            a = T(g['re_in'][..., sl], cuda)
            b = T(g['im_in'][..., sl], cuda)
            outs.append(p.spike(*p.dynamics((a, b))))
        assert_exact(torch.cat(outs, dim=-1), g['spike_split'], 'persistent-state split run')
        for name, buf in p.named_buffers():
            if name.endswith('_state'):
                assert_quantised_equal(buf, g[f'final_{name}'], S, f'final {name}')


def test_rf_iz(cuda, slayer):
    g = load_golden('neuron_rfiz_shared')
    _check_iz(lambda: slayer.neuron.rf_iz.Neuron(0.5, 10, 0.1, requires_grad=True), g,
              lambda: O.rf_iz(g['re_in'], g['im_in'], 0.5, g['param_sin_decay'], g['param_cos_decay'],
                              grad_spike=g['grad_spike']), cuda)


def test_adrf_iz(cuda, slayer):
    g = load_golden('neuron_adrfiz_shared')
    _check_iz(lambda: slayer.neuron.adrf_iz.Neuron(0.5, 0.25, 12, 0.1, 0.1, 0.1, requires_grad=True), g,
              lambda: O.adrf_iz(g['re_in'], g['im_in'], 0.5, 0.25, g['param_sin_decay'], g['param_cos_decay'],
                                410.0, 410.0, grad_spike=g['grad_spike']), cuda)
    n = slayer.neuron.adrf_iz.Neuron(0.5, 0.25, 12, 0.1, 0.1, 0.1).to(cuda)
    out = n((T(g['re_in'], cuda), T(g['im_in'], cuda)))  # forward() works here (TypeError in the reference)
    assert_exact(out, g['spike'], 'forward')


# --------------------------------------------------------------------------
# sigma-delta family through the module API
# --------------------------------------------------------------------------
def test_sigma_module(cuda, slayer):
    g = load_golden('sigma_persistent')
    sig = slayer.dendrite.Sigma(persistent_state=True)
    x = T(g['x'], cuda, True)
    s1 = sig(x)
    (s1 * T(g['grad_out'], cuda)).sum().backward()
    assert_exact(s1, g['out1'], 'running sum')
    assert_exact(x.grad, g['grad_x'], 'adjoint')
    assert_exact(sig(T(g['x'], cuda)), g['out2'], 'second call continues the sum')


def test_delta_module(cuda, slayer):
    g = load_golden('delta_shared')
    dl = slayer.axon.Delta(threshold=0.5, scale=S, tau_grad=float(g['tau_grad']), scale_grad=float(g['scale_grad']),
                           shared_param=True, persistent_state=True, requires_grad=True).to(cuda)
    x = T(g['x'], cuda, True)
    y1 = dl(x)
    (y1 * T(g['grad_out'], cuda)).sum().backward()
    assert_exact(y1, g['out1'], 'delta output')
    assert_exact(x.grad, g['grad_x'], 'grad_x')
    assert_close(dl.threshold.grad, g['grad_threshold'], 'grad_threshold')
    assert_exact(dl(T(g['x'], cuda)), g['out2'], 'second call with kept states')
    assert_exact(dl.residual_state, g['residual'], 'residual state')
    with pytest.raises(NotImplementedError):
        slayer.axon.Delta(threshold=0.5, cum_error=True)
    g = load_golden('delta_chan_rank4')
    dl = slayer.axon.Delta(threshold=0.3, scale=S, shared_param=False).to(cuda)
    dl(T(g['x'], cuda))   # first call fixes the shape and expands the threshold
    dl.threshold.data = T(g['threshold'], cuda).reshape(dl.threshold.shape)
    assert_exact(dl(T(g['x'], cuda)), g['out'], 'one threshold per channel')


def test_sigma_delta_neuron(cuda, slayer):
    relu = torch.nn.functional.relu
    g = load_golden('neuron_sdnn_shared')
    nrn = slayer.neuron.sigma_delta.Neuron(threshold=0.1, activation=relu, tau_grad=float(g['tau_grad']),
                                           scale_grad=float(g['scale_grad']), shared_param=True,
                                           persistent_state=True, requires_grad=True).to(cuda)
    x = T(g['x'], cuda, True)
    y1 = nrn(x)                       # gradients wanted: sigma, relu and delta as separate passes
    (y1 * T(g['grad_out'], cuda)).sum().backward()
    assert_exact(y1, g['out1'], 'sigma-delta output')
    assert_close(x.grad, g['grad_x'], 'grad_x')
    assert_close(nrn.delta.threshold.grad, g['grad_threshold'], 'grad_threshold')
    with torch.no_grad():
        y2 = nrn(T(g['x'], cuda))     # no gradients: the one-pass kernel, continuing the kept states
    assert_exact(y2, g['out2'], 'second call (one-pass kernel) with kept states')
    g = load_golden('neuron_sdnn_bias_rank4')
    nrn = slayer.neuron.sigma_delta.Neuron(threshold=0.05, activation=relu, shared_param=False).to(cuda)
    C, H = g['x'].shape[1:3]
    nrn.set_bias(T(g['bias'], cuda).reshape(C, H))
    x = T(g['x'], cuda)
    assert_exact(nrn(x), g['out'], 'per-neuron bias, one-pass kernel')
    nrn2 = slayer.neuron.sigma_delta.Neuron(threshold=0.05, activation=torch.relu, shared_param=False).to(cuda)
    nrn2.set_bias(T(g['bias'], cuda).reshape(C, H))
    assert_exact(nrn2(x), g['out'], 'per-neuron bias, separate passes')


def test_sigma_delta_block_network(cuda, slayer):
    """Delta-encoding input block + two dense sigma-delta blocks against the reference's
    blocks: events bit-exact layer by layer, gradients to 1e-5."""
    g = load_golden('network_sdnn_dense')
    relu = torch.nn.functional.relu
    p = dict(threshold=0.1, activation=relu, tau_grad=0.5, scale_grad=1.0, requires_grad=False)
    blk = slayer.block.sigma_delta
    net = torch.nn.ModuleList([blk.Input(dict(p)), blk.Dense(dict(p), 12, 10, weight_scale=2),
                               blk.Dense(dict(p), 10, 4, weight_scale=2)]).to(cuda)
    net[1].synapse.weight.data = T(g['weight1'], cuda)
    net[2].synapse.weight.data = T(g['weight2'], cuda)
    x = T(g['x'], cuda, True)
    y = x
    for i, layer in enumerate(net):
        y = layer(y)
        assert_exact(y, g[f'act{i}'], f'layer {i} events')
    (y * T(g['grad_out'], cuda)).sum().backward()
    assert_close(x.grad, g['grad_x'], 'grad_x')
    assert_close(net[1].synapse.weight.grad, g['grad_weight1'], 'grad weight 1')
    assert_close(net[2].synapse.weight.grad, g['grad_weight2'], 'grad weight 2')
    with torch.no_grad():           # inference: every neuron runs as the one-pass kernel
        y = T(g['x'], cuda)
        for i, layer in enumerate(net):
            y = layer(y)
            assert_exact(y, g[f'act{i}'], f'layer {i} events, one-pass kernels')


def test_recurrent_block(cuda, slayer):
    """Dense recurrent CUBA block against the reference's block (per-step Python loop):
    spikes bit-exact for two consecutive calls (the neuron state persists), gradients to 1e-5."""
    g = load_golden('block_cuba_recurrent')
    p = dict(threshold=1.25, current_decay=0.25, voltage_decay=0.03, requires_grad=True)
    blk = slayer.block.cuba.Recurrent(p, 24, 40, weight_scale=3, delay_shift=True).to(cuda)
    blk.input_synapse.weight.data = T(g['weight_in'], cuda)
    blk.recurrent_synapse.weight.data = T(g['weight_rec'], cuda)
    x = T(g['x'], cuda, True)
    # the dense synapses are library convolutions: keep them in fp32 so that 1e-5 applies to the whole block
    with torch.backends.cudnn.flags(allow_tf32=False):
        y = blk(x)
        assert_exact(y, g['out1'], 'recurrent block spikes')
        (y * T(g['grad_out'], cuda)).sum().backward()
    assert_close(x.grad, g['grad_x'], 'grad_x')
    assert_close(blk.input_synapse.weight.grad, g['grad_weight_in'], 'grad input weight')
    assert_close(blk.recurrent_synapse.weight.grad, g['grad_weight_rec'], 'grad recurrent weight')
    for k in ('current_decay', 'voltage_decay'):     # zero in the reference, zero or absent here
        grad = getattr(blk.neuron, k).grad
        assert grad is None or not grad.any()
        assert not g[f'grad_{k}'].any()
    with torch.no_grad():
        assert_exact(blk(T(g['x'], cuda)), g['out2'], 'second call, persistent neuron state')


def test_recurrent_block_graded(cuda, slayer):
    g = load_golden('block_cuba_recurrent_graded')
    p = dict(threshold=1.25, current_decay=[0.2, 0.4], voltage_decay=[0.02, 0.1], shared_param=False,
             graded_spike=True)
    blk = slayer.block.cuba.Recurrent(p, 17, 33, weight_scale=2, delay_shift=False).to(cuda)
    blk.input_synapse.weight.data = T(g['weight_in'], cuda)
    blk.recurrent_synapse.weight.data = T(g['weight_rec'], cuda)
    # graded (float) inputs through the library convolution of the dense synapse: fp32, not TF32
    with torch.no_grad(), torch.backends.cudnn.flags(allow_tf32=False):
        blk(T(g['x'], cuda))                       # binds shapes, samples per-neuron decays
        blk.neuron.current_decay.data = T(g['current_decay'], cuda).reshape(blk.neuron.current_decay.shape)
        blk.neuron.voltage_decay.data = T(g['voltage_decay'], cuda).reshape(blk.neuron.voltage_decay.shape)
        blk.neuron.current_state = torch.zeros(1, device=cuda)
        blk.neuron.voltage_state = torch.zeros(1, device=cuda)
        y = blk(T(g['x'], cuda))
    assert_exact(y, g['out'], 'graded spikes (every product and sum of this case is exact in fp32)')


def test_firbank(cuda, slayer):
    """Learnable filter bank: outputs, input gradient and weight gradient of the reference's
    conv3d-based module, on rank-3 and rank-4 inputs; same state_dict key."""
    g = load_golden('firbank')
    bank = slayer.utils.filter.FIRBank(3, 9, scale=2).to(cuda)
    assert list(bank.state_dict().keys()) == ['weight']
    bank.load_state_dict({'weight': torch.tensor(g['weight'])})
    x = torch.tensor(g['x'], device=cuda, requires_grad=True)
    out = bank(x)
    mag = np.abs(g['weight']).sum() * np.abs(g['x']).max()
    assert_close(out, g['out'], 'filter bank output', scale=mag)
    (out * torch.tensor(g['grad_out'], device=cuda)).sum().backward()
    gmag = np.abs(g['weight']).sum() * np.abs(g['grad_out']).max() * 3
    assert_close(x.grad, g['grad_x'], 'filter bank input gradient', scale=gmag)
    wmag = np.abs(g['grad_out']).max() * np.abs(g['x']).sum()
    assert_close(bank.weight.grad, g['grad_weight'], 'filter bank weight gradient', scale=wmag)
    with torch.no_grad():
        out4 = bank(torch.tensor(g['x4'], device=cuda))
    assert_close(out4, g['out4'], 'filter bank output, rank 4', scale=np.abs(g['weight']).sum() * np.abs(g['x4']).max())
