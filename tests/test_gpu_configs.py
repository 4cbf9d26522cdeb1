"""The benchmark configurations themselves, through the public classes, against the CPU oracle on
identical seeded CPU inputs: the CUBA layer at its full size (forward and backward), batch slices of
the ALIF, adaptive resonate-and-fire and delay + filter configurations at their full neuron count and
length, and a slice of the headline shape [64, 8192, 2000] wide enough (1024 warps) to run the same
full-grid, three-boxes-per-stage kernel instance that the benchmark times."""

import numpy as np
import pytest
import torch

from _util import assert_close, assert_exact, assert_quantised_equal, li_scale, pgrad_scale, res_scale, \
    cspike_term_scale
from oracle import oracle as O

pytestmark = pytest.mark.gpu

S = 4096  # state scale of the four neuron classes: scale (64) * 64


@pytest.fixture(scope='module')
def slayer(cuda):
    import lava_dl_b200.slayer as slayer
    return slayer


@pytest.fixture(scope='module', autouse=True)
def oracle_threads():
    import os
    O.set_threads(os.cpu_count() or 1)


def seeded(shape, mean, std, seed):
    g = torch.Generator().manual_seed(seed)
    return mean + std * torch.randn(shape, generator=g)


def _cuba_case(shape, seed, cuda, slayer, backward):
    x_cpu = seeded(shape, 0.3, 1.0, seed)
    neuron = slayer.neuron.cuba.Neuron(threshold=1.25, current_decay=0.25, voltage_decay=0.03,
                                       requires_grad=backward).to(cuda)
    x = x_cpu.to(cuda).requires_grad_(backward)
    spike = neuron(x)
    gs = np.ones(shape, np.float32) if backward else None
    cd = neuron.current_decay.detach().cpu().numpy()
    vd = neuron.voltage_decay.detach().cpu().numpy()
    want = O.cuba(x_cpu.numpy(), 1.25, cd, vd, grad_spike=gs)
    assert_exact(spike, want['spike'], 'spike')
    with torch.no_grad():
        current, voltage = neuron.dynamics(x.detach())
    assert_quantised_equal(current, want['current'], S, 'current')
    assert_quantised_equal(voltage, want['voltage'], S, 'voltage')
    if not backward:
        return
    spike.sum().backward()
    thr = 1.25 + 0.01 / S
    g_v = O.spike_bwd(want['voltage'], thr, gs, 125.0, 0.1, False)
    g_c, _ = O.li_bwd(g_v, want['voltage'], O.quantize(vd))
    assert_close(x.grad, want['grad_x'], 'cfg cuba grad_x', scale=li_scale(li_scale(g_v, O.quantize(vd)), O.quantize(cd)))
    assert_close(neuron.current_decay.grad, want['grad_current_decay'], 'cfg cuba grad current decay',
                 scale=pgrad_scale(1, (want['grad_x'], want['current'])))
    assert_close(neuron.voltage_decay.grad, want['grad_voltage_decay'], 'cfg cuba grad voltage decay',
                 scale=pgrad_scale(1, (g_c, want['voltage'])))


def test_cfg0_cuba_full_size(cuda, slayer):
    """[16, 512, 1000], N(0.3, 1), threshold 1.25, decays 0.25 / 0.03, sum-of-spikes loss."""
    _cuba_case((16, 512, 1000), 0, cuda, slayer, backward=True)


def test_headline_shape_slice(cuda, slayer):
    """[4, 8192, 2000] of the [64, 8192, 2000] headline shape: 32768 rows = 1024 warps, so every SM
    holds its full set of resident warps and the last stage of each row is ragged (2000 = 20 * 96 + 80)."""
    _cuba_case((4, 8192, 2000), 1, cuda, slayer, backward=True)


def test_cfg1_alif_slice(cuda, slayer):
    """[2, 4096, 2000] of [64, 4096, 2000], N(0.2, 1)."""
    shape = (2, 4096, 2000)
    x_cpu = seeded(shape, 0.2, 1.0, 2)
    neuron = slayer.neuron.alif.Neuron(threshold=1.0, threshold_step=0.5, current_decay=0.2, voltage_decay=0.05,
                                       threshold_decay=0.1, refractory_decay=0.1).to(cuda)
    x = x_cpu.to(cuda).requires_grad_(True)
    spike = neuron(x)
    p = {k: getattr(neuron, k).detach().cpu().numpy() for k in
         ('current_decay', 'voltage_decay', 'threshold_decay', 'refractory_decay')}
    gs = np.ones(shape, np.float32)
    want = O.alif(x_cpu.numpy(), 1.0, 0.5, p['current_decay'], p['voltage_decay'], p['threshold_decay'],
                  p['refractory_decay'], grad_spike=gs)
    assert_exact(spike, want['spike'], 'spike')
    with torch.no_grad():
        outs = neuron.dynamics(x.detach())
    for o, k in zip(outs, ('current', 'voltage', 'threshold', 'refractory')):
        assert_quantised_equal(o, want[k], S, k)
    spike.sum().backward()
    g_v = O.spike_bwd(want['voltage'], want['threshold'] + want['refractory'], gs, 100.0, 0.1, False)
    assert_close(x.grad, want['grad_x'], 'cfg alif grad_x',
                 scale=li_scale(li_scale(g_v, O.quantize(p['voltage_decay'])), O.quantize(p['current_decay'])))


def test_cfg2_adrf_slice(cuda, slayer):
    """[2, 8192, 1000] of [64, 8192, 1000] per component, N(0, 0.5); one period per neuron, uniform in
    10 .. 40 steps, decay 0.1, set explicitly as sin/cos decays on both sides."""
    shape = (2, 8192, 1000)
    re_cpu, im_cpu = seeded(shape, 0.0, 0.5, 3), seeded(shape, 0.0, 0.5, 4)
    neuron = slayer.neuron.adrf.Neuron(threshold=0.5, threshold_step=0.25, period=[10, 40], decay=0.1,
                                       threshold_decay=0.1, refractory_decay=0.1, shared_param=False,
                                       requires_grad=True).to(cuda)
    with torch.no_grad():
        neuron((torch.zeros(1, shape[1], 4, device=cuda), torch.zeros(1, shape[1], 4, device=cuda)))  # binds the shape
        period = 10 + 30 * torch.rand(shape[1], generator=torch.Generator().manual_seed(5))
        neuron.sin_decay.data = (4096 * torch.sin(2 * np.pi / period) * 0.9).to(cuda)
        neuron.cos_decay.data = (4096 * torch.cos(2 * np.pi / period) * 0.9).to(cuda)
    re = re_cpu.to(cuda).requires_grad_(True)
    im = im_cpu.to(cuda).requires_grad_(True)
    spike = neuron((re, im))
    p = {k: getattr(neuron, k).detach().cpu().numpy() for k in
         ('sin_decay', 'cos_decay', 'threshold_decay', 'refractory_decay')}
    gs = np.ones(shape, np.float32)
    want = O.adrf(re_cpu.numpy(), im_cpu.numpy(), 0.5, 0.25, p['sin_decay'], p['cos_decay'], p['threshold_decay'],
                  p['refractory_decay'], grad_spike=gs)
    assert_exact(spike, want['spike'], 'spike')
    with torch.no_grad():
        outs = neuron.dynamics((re.detach(), im.detach()))
    for o, k in zip(outs, ('real', 'imag', 'threshold', 'refractory')):
        assert_quantised_equal(o, want[k], S, k)
    spike.sum().backward()
    thsum = want['threshold'] + want['refractory']
    sd, cd = O.quantize(p['sin_decay']), O.quantize(p['cos_decay'])
    s_re, s_im = cspike_term_scale(want['real'], want['imag'], thsum, gs, 50.0, 0.1, False)
    S_re, S_im = res_scale(s_re, s_im, sd, cd)
    S_p = pgrad_scale(sd.size, (want['grad_re'], want['real']), (want['grad_re'], want['imag']),
                      (want['grad_im'], want['real']), (want['grad_im'], want['imag']))
    assert_close(re.grad, want['grad_re'], 'cfg adrf grad real input', scale=S_re)
    assert_close(im.grad, want['grad_im'], 'cfg adrf grad imag input', scale=S_im)
    assert_close(neuron.sin_decay.grad, want['grad_sin_decay'], 'cfg adrf grad sin decay', scale=S_p)
    assert_close(neuron.cos_decay.grad, want['grad_cos_decay'], 'cfg adrf grad cos decay', scale=S_p)


def test_cfg3_delay_filter_slice(cuda, slayer):
    """[2, 16384, 1000] of [128, 16384, 1000]: Bernoulli(0.05) spikes, per-neuron delays 0 .. 62,
    64-tap filter exp(-t / 8) / 8; y = conv(shift(s, delay), filter), loss y.sum()."""
    shape = (2, 16384, 1000)
    g = torch.Generator().manual_seed(6)
    s_cpu = (torch.rand(shape, generator=g) < 0.05).float()
    delay_cpu = torch.randint(0, 63, (shape[1],), generator=g).float()
    filt_cpu = torch.exp(-torch.arange(64).float() / 8) / 8
    s = s_cpu.to(cuda).requires_grad_(True)
    delay, filt = delay_cpu.to(cuda), filt_cpu.to(cuda)
    shifted = slayer.axon.delay(s, delay)
    y = slayer.utils.filter.conv(shifted, filt)
    sh_w = O.shift(s_cpu.numpy(), delay_cpu.numpy())
    assert_exact(shifted, sh_w, 'shift')
    y_w = O.conv(sh_w, filt_cpu.numpy())
    # all terms are non-negative: the sum of term magnitudes is the value itself
    assert_close(y, y_w, 'cfg3 conv(shift(s))', scale=np.abs(y_w))
    y.sum().backward()
    g_w = O.shift(O.corr(np.ones(shape, np.float32), filt_cpu.numpy()), -delay_cpu.numpy())
    assert_close(s.grad, g_w, 'cfg3 grad of the spike input', scale=np.abs(g_w))
    # the fused form of the same chain (what the delay + filter benchmark times)
    from lava_dl_b200 import _ops
    y2 = _ops.shift_fir(s.detach(), delay, 1, filt, 1.0, backward=False)
    assert_close(y2, y_w, 'cfg3 fused delay + filter', scale=np.abs(y_w))
    g2 = _ops.shift_fir(torch.ones(shape, device=cuda), delay, 1, filt, 1.0, backward=True)
    assert_close(g2, g_w, 'cfg3 fused delay + filter backward', scale=np.abs(g_w))
