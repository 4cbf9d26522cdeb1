"""Generates the golden vectors under tests/golden/ by running lava-dl itself.

Run where the reference checkout is available (it is NOT needed to run the
tests, only to regenerate the fixtures):

    python tests/golden/make_golden.py /path/to/lava-dl

The reference's CPU code path (the Python loops in
src/lava/lib/dl/slayer/neuron/dynamics/*.py, spike/*.py, utils/time/shift.py,
utils/filter/conv.py and the neuron classes) is imported unmodified;
matplotlib and h5py, which the package imports at top level but the hot path
never touches, are stubbed.  Every case stores its inputs, parameters and the
reference's outputs in one .npz; tests replay the inputs through the oracle
(CPU) and through the CUDA kernels (GPU).
"""

import os
import sys
import types

import numpy as np


def import_reference(root):
    class _Stub(types.ModuleType):
        def __getattr__(self, k):
            if k.startswith('__'):
                raise AttributeError(k)
            return type(k, (), {})

    for m in ['matplotlib', 'matplotlib.pyplot', 'matplotlib.animation', 'h5py']:
        sys.modules[m] = _Stub(m)
    sys.path.insert(0, os.path.join(root, 'src'))
    import lava.lib.dl.slayer as slayer
    return slayer


def main():
    if len(sys.argv) < 2:
        sys.exit('usage: python tests/golden/make_golden.py /path/to/lava-dl')
    root = sys.argv[1]
    out_dir = os.path.dirname(os.path.abspath(__file__))
    slayer = import_reference(root)
    import torch
    from lava.lib.dl.slayer.neuron.dynamics import (leaky_integrator, adaptive_threshold, resonator,
                                                    adaptive_phase_th, adaptive_resonator)
    from lava.lib.dl.slayer.spike import Spike
    from lava.lib.dl.slayer.spike import complex as cspike
    from lava.lib.dl.slayer.utils.time import shift
    from lava.lib.dl.slayer.utils.filter import conv, corr
    from lava.lib.dl.slayer.axon import delay as axon_delay

    torch.set_num_threads(4)
    gen = torch.Generator().manual_seed(20240607)

    def randn(*shape, mean=0.0, std=1.0):
        return mean + std * torch.randn(*shape, generator=gen)

    def rand(*shape):
        return torch.rand(*shape, generator=gen)

    def npy(t):
        return t.detach().cpu().numpy().copy()

    cases = {}

    def save(name, **arrays):
        cases[name] = {k: (npy(v) if torch.is_tensor(v) else np.asarray(v)) for k, v in arrays.items()}

    W = 4096
    B, C, T = 3, 5, 77  # T deliberately not a multiple of 4 or 32
    B2, C2, H2, T2 = 2, 3, 4, 64  # NCHWT-like (rank 4), T multiple of 32

    # ------------------------------------------------------------------
    # leaky integrator
    # ------------------------------------------------------------------
    for tag, shape, dec, thr in [
        ('shared_nothr', (B, C, T), torch.tensor([410.0]), None),
        ('shared_thr', (B, C, T), torch.tensor([123.0]), 1.25 + 0.01 / 4096),
        ('chan_thr', (B, C, T), torch.tensor([100., 500., 1024., 3000., 4096.]), 0.5),
        ('chan_nothr_T64', (B2, C2, T2), torch.tensor([0., 204.8, 2047.5]), None),
        ('rank2', (7, 40), torch.tensor([300.0]), 1.0),
    ]:
        x = randn(*shape, mean=0.3)
        state = (randn(*shape[:-1]) * 0.5 * W).round() / W
        dec = dec.clone().requires_grad_(True)
        xin = x.clone().requires_grad_(True)
        y = leaky_integrator.dynamics(xin, dec, state, W, threshold=thr)
        go = randn(*shape)
        y.backward(go)
        save(f'li_{tag}', x=x, decay=dec, state=state, threshold=np.float64(-1 if thr is None else thr),
             w_scale=W, y=y, grad_out=go, grad_in=xin.grad, grad_decay=dec.grad)
    # scalar (1-element) state and non power-of-two scale
    x = randn(B, C, T, mean=0.2)
    y = leaky_integrator.dynamics(x, torch.tensor([700.0]), torch.tensor([0.37]), 1000, threshold=0.8)
    save('li_w1000', x=x, decay=np.array([700.0], np.float32), state=np.array([0.37], np.float32),
         threshold=np.float64(0.8), w_scale=1000, y=y)

    # ------------------------------------------------------------------
    # adaptive threshold / adaptive phase threshold
    # ------------------------------------------------------------------
    for tag, shape, rd, td in [
        ('shared', (B, C, T), torch.tensor([410.0]), torch.tensor([205.0])),
        ('chan', (B, C, T), torch.tensor([100., 300., 500., 700., 900.]),
         torch.tensor([50., 150., 250., 350., 450.])),
    ]:
        x = randn(*shape, mean=0.5, std=1.5)
        ref_state = (rand(*shape[:-1]) * W).round() / W - 0.25
        th_state = 1.0 + (rand(*shape[:-1]) * W).round() / W - 0.5
        th, ref = adaptive_threshold.dynamics(x, ref_state, rd, th_state, td, 0.5, 1.0, W)
        save(f'ath_{tag}', x=x, ref_state=ref_state, ref_decay=rd, th_state=th_state, th_decay=td,
             th_scale=0.5, th0=1.0, w_scale=W, threshold=th, refractory=ref)

        re = randn(*shape, std=1.5)
        im = randn(*shape, std=1.5)
        im_state = randn(*shape[:-1])
        th, ref = adaptive_phase_th.dynamics(re, im, im_state, ref_state, rd, th_state, td, 0.25, 0.5, W)
        save(f'apth_{tag}', re=re, im=im, im_state=im_state, ref_state=ref_state, ref_decay=rd,
             th_state=th_state, th_decay=td, th_scale=0.25, th0=0.5, w_scale=W, threshold=th, refractory=ref)

    # ------------------------------------------------------------------
    # resonator / adaptive resonator
    # ------------------------------------------------------------------
    def sincos(periods, decay=0.1):
        p = torch.as_tensor(periods, dtype=torch.float32)
        return (4096 * torch.sin(2 * np.pi / p) * (1 - decay)).round(), \
               (4096 * torch.cos(2 * np.pi / p) * (1 - decay)).round()

    for tag, shape, periods, thr in [
        ('shared', (B, C, T), [10.0], None),
        ('chan', (B, C, T), [4.0, 8.0, 16.0, 25.0, 40.0], None),
        ('shared_reset', (B, C, T), [12.0], 0.75),
        ('chan_T64', (B2, C2, T2), [5.0, 9.0, 33.0], None),
        ('neg_cos', (B, C, T), [3.0], None),  # period < 4 -> negative cos_decay
    ]:
        sd, cd = sincos(periods)
        sd = sd.clone().requires_grad_(True)
        cd = cd.clone().requires_grad_(True)
        re_in = randn(*shape, std=0.5).requires_grad_(True)
        im_in = randn(*shape, std=0.5).requires_grad_(True)
        re_state = (randn(*shape[:-1]) * 0.3 * W).round() / W
        im_state = (randn(*shape[:-1]) * 0.3 * W).round() / W
        re, im = resonator.dynamics(re_in, im_in, sd, cd, re_state, im_state, W, threshold=thr)
        g_re, g_im = randn(*shape), randn(*shape)
        (re * g_re + im * g_im).sum().backward()
        save(f'res_{tag}', re_in=re_in, im_in=im_in, sin_decay=sd, cos_decay=cd, re_state=re_state,
             im_state=im_state, threshold=np.float64(-1 if thr is None else thr), w_scale=W, re=re, im=im,
             grad_re=g_re, grad_im=g_im, grad_re_in=re_in.grad, grad_im_in=im_in.grad, grad_sin=sd.grad,
             grad_cos=cd.grad)

    for tag, shape, periods, rd, td in [
        ('shared', (B, C, T), [10.0], torch.tensor([410.0]), torch.tensor([205.0])),
        ('chan', (B, C, T), [4.0, 8.0, 16.0, 25.0, 40.0], torch.tensor([100., 300., 500., 700., 900.]),
         torch.tensor([50., 150., 250., 350., 450.])),
    ]:
        sd, cd = sincos(periods)
        sd = sd.clone().requires_grad_(True)
        cd = cd.clone().requires_grad_(True)
        re_in = randn(*shape, std=0.5).requires_grad_(True)
        im_in = randn(*shape, std=0.5).requires_grad_(True)
        re_state = (randn(*shape[:-1]) * 0.3 * W).round() / W
        im_state = (randn(*shape[:-1]) * 0.3 * W).round() / W
        ref_state = (rand(*shape[:-1]) * W).round() / W - 0.25
        th_state = 0.5 + (rand(*shape[:-1]) * W).round() / W * 0.5
        re, im, th, ref = adaptive_resonator.dynamics(
            re_in, im_in, sd, cd, rd, td, re_state, im_state, ref_state, th_state, 0.25, 0.5, W)
        g_re, g_im = randn(*shape), randn(*shape)
        (re * g_re + im * g_im).sum().backward()
        save(f'adres_{tag}', re_in=re_in, im_in=im_in, sin_decay=sd, cos_decay=cd, ref_decay=rd, th_decay=td,
             re_state=re_state, im_state=im_state, ref_state=ref_state, th_state=th_state, th_scale=0.25,
             th0=0.5, w_scale=W, re=re, im=im, threshold=th, refractory=ref, grad_re=g_re, grad_im=g_im,
             grad_re_in=re_in.grad, grad_im_in=im_in.grad, grad_sin=sd.grad, grad_cos=cd.grad)

    # ------------------------------------------------------------------
    # spike functions
    # ------------------------------------------------------------------
    for tag, graded, tensor_thr in [('bin_scalar', False, False), ('bin_tensor', False, True),
                                    ('graded_scalar', True, False), ('graded_tensor', True, True)]:
        v = (randn(B, C, T, mean=0.8, std=1.0) * W).round() / W
        v.requires_grad_(True)
        thr = (1.0 + 0.3 * rand(B, C, T)) if tensor_thr else (1.25 + 0.01 / 4096)
        s = Spike.apply(v, thr, 1.25 * 100, 0.1, graded, torch.zeros(B, C), 1)
        gs = randn(B, C, T)
        s.backward(gs)
        save(f'spike_{tag}', v=v, threshold=thr if tensor_thr else np.float64(thr), tau_rho=1.25 * 100,
             scale_rho=0.1, graded=graded, spike=s, grad_spike=gs, grad_v=v.grad)

        re = (randn(B, C, T, std=1.0) * W).round() / W
        im = (randn(B, C, T, std=1.0) * W).round() / W
        re.requires_grad_(True)
        im.requires_grad_(True)
        cthr = (0.3 + 0.3 * rand(B, C, T)) if tensor_thr else 0.5
        last = randn(B, C)
        s = cspike.Spike.apply(re, im, cthr, 0.5 * 0.5, 10.0, graded, last, 1)
        gs = randn(B, C, T)
        s.backward(gs)
        save(f'cspike_{tag}', re=re, im=im, threshold=cthr if tensor_thr else np.float64(cthr), tau_rho=0.25,
             scale_rho=10.0, graded=graded, imag_last=last, spike=s, grad_spike=gs, grad_re=re.grad,
             grad_im=im.grad)

    # ------------------------------------------------------------------
    # shift / filter
    # ------------------------------------------------------------------
    x = rand(B, C, T)
    for tag, sv in [('p10', 10), ('m7', -7), ('zero', 0), ('big', 200)]:
        save(f'shift_{tag}', x=x, shift=np.float64(sv), sampling_time=1.0, out=shift(x, sv))
    lut = torch.tensor([0., 3., -5., 62.4, 76.0])
    save('shift_lut', x=x, shift=lut, sampling_time=1.0, out=shift(x, lut))
    x4 = rand(B2, C2, H2, T2)
    lut4 = torch.randint(-8, 40, (C2, H2), generator=gen).float()
    save('shift_lut_rank4', x=x4, shift=lut4, sampling_time=1.0, out=shift(x4, lut4))
    save('shift_scalar_ts2', x=x, shift=np.float64(9), sampling_time=2.0, out=shift(x, 9, 2.0))

    for tag, K, ts in [('k50', 50, 1.0), ('k64_ts2', 64, 2.0), ('k1', 1, 1.0), ('k100', 100, 1.0)]:
        x = rand(B, C, T).requires_grad_(True)
        f = torch.exp(-torch.arange(K).float() / 8) / 8 * (1 + 0.1 * randn(K))
        y = conv(x, f, ts)
        g = randn(B, C, T)
        y.backward(g)
        z = corr(x.detach(), f, ts)
        save(f'fir_{tag}', x=x, filter=f, sampling_time=ts, conv=y, corr=z, grad_out=g, grad_conv=x.grad)

    # delay (shift with autograd) followed by filter: the config-3 chain
    x = (rand(B, C, T) < 0.2).float().requires_grad_(True)
    d = torch.tensor([0., 1., 5., 30., 62.])
    f = torch.exp(-torch.arange(64).float() / 8) / 8
    y = conv(axon_delay(x, d), f)
    g = randn(B, C, T)
    y.backward(g)
    save('delay_fir_chain', x=x, delay=d, filter=f, out=y, grad_out=g, grad_x=x.grad)

    # ------------------------------------------------------------------
    # neuron classes: forward, backward, persistent-state split
    # ------------------------------------------------------------------
    def run_neuron(make, inputs, param_names, set_params=None, split=None):
        """Forward+backward of spike.sum()-like loss; optional two-chunk run with persistent state."""
        res = {}
        n = make()
        ins = [i.clone().requires_grad_(True) for i in inputs]
        arg = ins[0] if len(ins) == 1 else tuple(ins)
        if set_params is not None:
            with torch.no_grad():
                n(arg)  # binds the shape and samples per-channel parameters
                for k, v in set_params.items():
                    getattr(n, k).data = v.clone()
            n2 = n
            for name, buf in n2.named_buffers():
                if name.endswith('_state'):
                    buf.zero_()
                    if name == 'threshold_state':
                        buf.add_(n2.threshold)
        spike = n(arg)
        g = randn(*spike.shape)
        (spike * g).sum().backward()
        res['spike'] = spike
        res['grad_spike'] = g
        for i, t in enumerate(ins):
            res[f'grad_in{i}'] = t.grad
        for k in param_names:
            p = getattr(n, k)
            res[f'param_{k}'] = p.data
            if p.grad is not None:
                res[f'grad_{k}'] = p.grad
        with torch.no_grad():
            m = make()
            if set_params is not None:
                m(arg)
                for k, v in set_params.items():
                    getattr(m, k).data = v.clone()
                for name, buf in m.named_buffers():
                    if name.endswith('_state'):
                        buf.zero_()
                        if name == 'threshold_state':
                            buf.add_(m.threshold)
            dyn = m.dynamics(arg)
            for i, t in enumerate(dyn):
                res[f'dyn{i}'] = t
        if split is not None:
            with torch.no_grad():
                p = make()
                p.persistent_state = True
                if set_params is not None:
                    p(arg)
                    for k, v in set_params.items():
                        getattr(p, k).data = v.clone()
                    for name, buf in p.named_buffers():
                        if name.endswith('_state'):
                            buf.zero_()
                            if name == 'threshold_state':
                                buf.add_(p.threshold)
                a = [i[..., :split] for i in inputs]
                b = [i[..., split:] for i in inputs]
                s1 = p(a[0] if len(a) == 1 else tuple(a))
                s2 = p(b[0] if len(b) == 1 else tuple(b))
                res['spike_split'] = torch.cat([s1, s2], dim=-1)
                for name, buf in p.named_buffers():
                    if name.endswith('_state'):
                        res[f'final_{name}'] = buf
        return res

    x = randn(B, C, T, mean=0.3)
    r = run_neuron(lambda: slayer.neuron.cuba.Neuron(1.25, 0.25, 0.03, requires_grad=True), [x],
                   ['current_decay', 'voltage_decay'], split=30)
    save('neuron_cuba_shared', x=x, **r)
    r = run_neuron(lambda: slayer.neuron.cuba.Neuron(1.25, 0.25, 0.03, shared_param=False, requires_grad=True,
                                                     graded_spike=True), [x],
                   ['current_decay', 'voltage_decay'],
                   set_params={'current_decay': torch.tensor([900., 1000., 1024., 1100., 1200.]),
                               'voltage_decay': torch.tensor([100., 120., 123., 130., 140.])}, split=32)
    save('neuron_cuba_chan_graded', x=x, **r)
    x4 = randn(B2, C2, H2, T2, mean=0.3)
    r = run_neuron(lambda: slayer.neuron.cuba.Neuron(1.25, 0.25, 0.03), [x4], ['current_decay', 'voltage_decay'],
                   split=32)
    save('neuron_cuba_rank4', x=x4, **r)

    x = randn(B, C, T, mean=0.2)
    r = run_neuron(lambda: slayer.neuron.alif.Neuron(1.0, 0.5, 0.2, 0.05, 0.1, 0.1), [x],
                   ['current_decay', 'voltage_decay', 'threshold_decay', 'refractory_decay'], split=40)
    save('neuron_alif_shared', x=x, **r)
    r = run_neuron(lambda: slayer.neuron.alif.Neuron(1.0, 0.5, 0.2, 0.05, 0.1, 0.1, shared_param=False,
                                                     requires_grad=True), [x],
                   ['current_decay', 'voltage_decay', 'threshold_decay', 'refractory_decay'],
                   set_params={'current_decay': torch.tensor([800., 810., 819., 830., 840.]),
                               'voltage_decay': torch.tensor([200., 203., 205., 207., 210.]),
                               'threshold_decay': torch.tensor([400., 405., 410., 415., 420.]),
                               'refractory_decay': torch.tensor([380., 395., 410., 425., 440.])}, split=33)
    save('neuron_alif_chan', x=x, **r)

    re_in, im_in = randn(B, C, T, std=0.5), randn(B, C, T, std=0.5)
    r = run_neuron(lambda: slayer.neuron.rf.Neuron(0.5, 10, 0.1, requires_grad=True), [re_in, im_in],
                   ['sin_decay', 'cos_decay'], split=37)
    save('neuron_rf_shared', re_in=re_in, im_in=im_in, **r)
    sd, cd = sincos([10., 15., 20., 30., 40.])
    r = run_neuron(lambda: slayer.neuron.adrf.Neuron(0.5, 0.25, [10, 40], 0.1, 0.1, 0.1, shared_param=False,
                                                     requires_grad=True), [re_in, im_in],
                   ['sin_decay', 'cos_decay', 'threshold_decay', 'refractory_decay'],
                   set_params={'sin_decay': sd, 'cos_decay': cd,
                               'threshold_decay': torch.full((5,), 410.),
                               'refractory_decay': torch.full((5,), 410.)}, split=32)
    save('neuron_adrf_chan', re_in=re_in, im_in=im_in, **r)
    r = run_neuron(lambda: slayer.neuron.adrf.Neuron(0.5, 0.25, 12, 0.1, 0.1, 0.1), [re_in, im_in],
                   ['sin_decay', 'cos_decay', 'threshold_decay', 'refractory_decay'], split=50)
    save('neuron_adrf_shared', re_in=re_in, im_in=im_in, **r)

    # Izhikevich-reset variants.  adrf_iz.forward raises TypeError in the reference
    # (adrf_iz.py:669-670), so its golden run calls dynamics() and spike() itself.
    def iz_case(make, adaptive):
        res = {}
        n = make()
        ins = [re_in.clone().requires_grad_(True), im_in.clone().requires_grad_(True)]
        dyn = n.dynamics(tuple(ins))
        spike = n.spike(*dyn)
        g = randn(*spike.shape)
        (spike * g).sum().backward()
        res.update(spike=spike, grad_spike=g, grad_in0=ins[0].grad, grad_in1=ins[1].grad)
        for i, t in enumerate(dyn):
            res[f'dyn{i}'] = t
        for k in ['sin_decay', 'cos_decay']:
            res[f'param_{k}'] = getattr(n, k).data
            res[f'grad_{k}'] = getattr(n, k).grad
        with torch.no_grad():
            p = make()
            p.persistent_state = True
            outs = []
            for a, b in ((re_in[..., :41], im_in[..., :41]), (re_in[..., 41:], im_in[..., 41:])):
                outs.append(p.spike(*p.dynamics((a, b))))
            res['spike_split'] = torch.cat(outs, dim=-1)
            for name, buf in p.named_buffers():
                if name.endswith('_state'):
                    res[f'final_{name}'] = buf
        return res

    save('neuron_rfiz_shared', re_in=re_in, im_in=im_in,
         **iz_case(lambda: slayer.neuron.rf_iz.Neuron(0.5, 10, 0.1, requires_grad=True), False))
    save('neuron_adrfiz_shared', re_in=re_in, im_in=im_in,
         **iz_case(lambda: slayer.neuron.adrf_iz.Neuron(0.5, 0.25, 12, 0.1, 0.1, 0.1, requires_grad=True), True))

    # ------------------------------------------------------------------
    # a small CUBA conv network built from the reference's blocks (the layer
    # sequence of the full-network benchmark config, scaled down)
    # ------------------------------------------------------------------
    neuron_p = dict(threshold=1.25, current_decay=0.25, voltage_decay=0.03, requires_grad=True)
    blk = slayer.block.cuba
    torch.manual_seed(99)
    net = torch.nn.ModuleList([
        blk.Pool(neuron_p, 4), blk.Conv(neuron_p, 2, 16, 5, padding=2, weight_scale=4), blk.Pool(neuron_p, 2),
        blk.Conv(neuron_p, 16, 32, 3, padding=1, weight_scale=3), blk.Pool(neuron_p, 2), blk.Flatten(),
        blk.Dense(neuron_p, 128, 64, weight_scale=3), blk.Dense(neuron_p, 64, 11, weight_scale=3, delay=True),
    ])
    x_net = (rand(2, 2, 32, 32, 40) < 0.08).float()
    with torch.no_grad():  # first call: binds shapes, samples the random axonal delays
        y = x_net
        for layer in net:
            y = layer(y)
        net[7].delay.delay.data = torch.tensor([0., 1., 2., 3., 5., 7., 0., 4., 6., 1., 2.])
    xin = x_net.clone().requires_grad_(True)
    acts, y = {}, xin
    for i, layer in enumerate(net):
        y = layer(y)
        acts[f'act{i}'] = y
    g_net = randn(*y.shape)
    (y * g_net).sum().backward()
    net_arrays = dict(x=x_net, grad_out=g_net, grad_x=xin.grad, delay=net[7].delay.delay.data,
                      grad_delay=net[7].delay.delay.grad, **acts)
    for i, layer in enumerate(net):
        if hasattr(layer, 'synapse'):
            net_arrays[f'weight{i}'] = layer.synapse.weight.data
            if layer.synapse.weight.grad is not None:
                net_arrays[f'grad_weight{i}'] = layer.synapse.weight.grad
        if hasattr(layer, 'neuron'):
            for k in ('current_decay', 'voltage_decay'):
                net_arrays[f'grad_{k}{i}'] = getattr(layer.neuron, k).grad
    print('network spike counts per layer:', [int(acts[f'act{i}'].sum()) for i in range(len(net))])
    save('network_cuba_conv', **net_arrays)

    # ------------------------------------------------------------------
    # sigma-delta family (dendrite/sigma.py, axon/delta.py, neuron/sigma_delta.py).
    # cum_error=True and the gradient of a per-channel threshold raise inside the
    # reference itself with this torch, so they have no vectors.
    x = randn(B, C, T, std=0.7)
    sig = slayer.dendrite.Sigma(persistent_state=True)
    xs = x.clone().requires_grad_()
    s1 = sig(xs)
    g = randn(B, C, T)
    (s1 * g).sum().backward()
    s2 = sig(x)
    save('sigma_persistent', x=x, out1=s1, grad_out=g, grad_x=xs.grad, out2=s2)

    dl = slayer.axon.Delta(threshold=0.5, scale=W, tau_grad=0.7, scale_grad=1.3, shared_param=True,
                           persistent_state=True, requires_grad=True)
    xs = x.clone().requires_grad_()
    y1 = dl(xs)
    (y1 * g).sum().backward()
    y2 = dl(x)
    save('delta_shared', x=x, threshold=dl.threshold.data.clone(), out1=y1, grad_out=g, grad_x=xs.grad,
         grad_threshold=dl.threshold.grad, out2=y2, residual=dl.residual_state, tau_grad=0.7, scale_grad=1.3)

    dl = slayer.axon.Delta(threshold=0.3, scale=W, shared_param=False)
    dl.threshold.data = torch.tensor([0.3])
    x4 = randn(B2, C2, H2, T2, std=0.5)
    y = dl(x4)
    dl.threshold.data = torch.linspace(0.1, 0.6, C2).reshape(C2, 1)
    y = dl(x4)
    save('delta_chan_rank4', x=x4, threshold=dl.threshold.data.reshape(-1).clone(), out=y)

    relu = torch.nn.functional.relu
    nrn = slayer.neuron.sigma_delta.Neuron(threshold=0.1, activation=relu, tau_grad=0.5, scale_grad=1.0,
                                           shared_param=True, persistent_state=True, requires_grad=True)
    xin = (0.15 * randn(B, C, T)).requires_grad_()
    y1 = nrn(xin)
    (y1 * g).sum().backward()
    y2 = nrn(xin.detach())
    save('neuron_sdnn_shared', x=xin, threshold=nrn.delta.threshold.data.clone(), out1=y1, grad_out=g,
         grad_x=xin.grad, grad_threshold=nrn.delta.threshold.grad, out2=y2, tau_grad=0.5 , scale_grad=1.0)

    nrn = slayer.neuron.sigma_delta.Neuron(threshold=0.05, activation=relu, shared_param=False)
    nrn.set_bias(torch.linspace(-0.2, 0.3, C2 * H2).reshape(C2, H2))   # one bias per neuron
    x4 = 0.1 * randn(B2, C2, H2, T2)
    y = nrn(x4)
    save('neuron_sdnn_bias_rank4', x=x4, threshold=nrn.delta.threshold.data.reshape(-1).clone(),
         bias=nrn.bias.data.reshape(-1).clone(), out=y)

    # sigma-delta blocks: delta-encoding input block and two dense blocks
    sdp = dict(threshold=0.1, activation=relu, tau_grad=0.5, scale_grad=1.0, requires_grad=False)
    sblk = slayer.block.sigma_delta
    snet = torch.nn.ModuleList([sblk.Input(dict(sdp)), sblk.Dense(dict(sdp), 12, 10, weight_scale=2),
                                sblk.Dense(dict(sdp), 10, 4, weight_scale=2)])
    for layer in snet[1:]:
        layer.synapse.weight.data = 0.4 * randn(*layer.synapse.weight.shape)
    xs = torch.cumsum(0.08 * randn(B, 12, T), dim=-1)
    xin = xs.clone().requires_grad_()
    acts, y = {}, xin
    for i, layer in enumerate(snet):
        y = layer(y)
        acts[f'act{i}'] = y
    g_s = randn(*y.shape)
    (y * g_s).sum().backward()
    save('network_sdnn_dense', x=xs, grad_out=g_s, grad_x=xin.grad, weight1=snet[1].synapse.weight.data,
         weight2=snet[2].synapse.weight.data, grad_weight1=snet[1].synapse.weight.grad,
         grad_weight2=snet[2].synapse.weight.grad, **acts)
    print('sigma-delta network event counts per layer:', [int((acts[f'act{i}'] != 0).sum()) for i in range(3)])

    # ------------------------------------------------------------------
    # dense recurrent CUBA block (block/base.py:1460-1488 over utils/recurrent.py:45-112):
    # two forward calls (the neuron state persists between them) and one backward
    # ------------------------------------------------------------------
    torch.manual_seed(5)
    rec = slayer.block.cuba.Recurrent(dict(threshold=1.25, current_decay=0.25, voltage_decay=0.03,
                                           requires_grad=True), 24, 40, weight_scale=3, delay_shift=True)
    xr = (rand(3, 24, 50) < 0.2).float()
    xin = xr.clone().requires_grad_(True)
    y1 = rec(xin)
    g_r = randn(*y1.shape)
    (y1 * g_r).sum().backward()
    with torch.no_grad():
        y2 = rec(xr)
    save('block_cuba_recurrent', x=xr, weight_in=rec.input_synapse.weight.data,
         weight_rec=rec.recurrent_synapse.weight.data, out1=y1, grad_out=g_r, grad_x=xin.grad,
         grad_weight_in=rec.input_synapse.weight.grad, grad_weight_rec=rec.recurrent_synapse.weight.grad,
         grad_current_decay=rec.neuron.current_decay.grad, grad_voltage_decay=rec.neuron.voltage_decay.grad, out2=y2)
    torch.manual_seed(6)
    rec = slayer.block.cuba.Recurrent(dict(threshold=1.25, current_decay=[0.2, 0.4], voltage_decay=[0.02, 0.1],
                                           shared_param=False, graded_spike=True), 17, 33, weight_scale=2,
                                      delay_shift=False)
    # weak, slightly inhibitory feedback and inputs on a 1/8 grid: graded values stay small enough for every
    # product and sum to be exact in fp32, so the result does not depend on the order of summation
    rec.recurrent_synapse.weight.data = rec.recurrent_synapse.weight.data * 0.5 - 0.04
    xg = (rand(2, 17, 37) < 0.25).float() * torch.round(rand(2, 17, 37) * 16) / 8
    with torch.no_grad():
        yg = rec(xg)
    save('block_cuba_recurrent_graded', x=xg, weight_in=rec.input_synapse.weight.data,
         weight_rec=rec.recurrent_synapse.weight.data, current_decay=rec.neuron.current_decay.data,
         voltage_decay=rec.neuron.voltage_decay.data, out=yg)
    print('recurrent block spike counts:', int(y1.sum()), int(y2.sum()), int((yg != 0).sum()))

    # ------------------------------------------------------------------
    # learnable filter bank (utils/filter/fir.py:57-100) and replication in time (utils/time/replicate.py)
    # ------------------------------------------------------------------
    from lava.lib.dl.slayer.utils.filter import FIRBank
    from lava.lib.dl.slayer.utils.time import replicate
    torch.manual_seed(7)
    bank = FIRBank(3, 9, scale=2)
    xb = randn(2, 5, 41)
    xin = xb.clone().requires_grad_(True)
    yb = bank(xin)
    g_b = randn(*yb.shape)
    (yb * g_b).sum().backward()
    xb4 = randn(2, 3, 2, 37)
    with torch.no_grad():
        yb4 = bank(xb4)
    save('firbank', x=xb, weight=bank.weight.data, out=yb, grad_out=g_b, grad_x=xin.grad,
         grad_weight=bank.weight.grad, x4=xb4, out4=yb4)
    xr2 = randn(3, 4)
    xr4 = randn(2, 3, 2, 2)
    save('replicate', x2=xr2, out2=replicate(xr2, 5), x4=xr4, out4=replicate(xr4, 3))

    # ------------------------------------------------------------------
    # blocks of the other families and the per-time-step callers:
    # ALIF recurrent block, winner-takes-all blocks, resonator networks with complex synapses,
    # input / average / sigma-delta output blocks
    # ------------------------------------------------------------------
    alif_p = dict(threshold=1.0, threshold_step=0.5, current_decay=0.2, voltage_decay=0.05, threshold_decay=0.1,
                  refractory_decay=0.1, requires_grad=True)
    torch.manual_seed(8)
    rec = slayer.block.alif.Recurrent(dict(alif_p), 12, 20, weight_scale=3)
    xr = (rand(2, 12, 30) < 0.3).float()
    xin = xr.clone().requires_grad_(True)
    y1 = rec(xin)
    g_r = randn(*y1.shape)
    (y1 * g_r).sum().backward()
    with torch.no_grad():
        y2 = rec(xr)
    save('block_alif_recurrent', x=xr, weight_in=rec.input_synapse.weight.data,
         weight_rec=rec.recurrent_synapse.weight.data, out1=y1, grad_out=g_r, grad_x=xin.grad,
         grad_weight_in=rec.input_synapse.weight.grad, grad_weight_rec=rec.recurrent_synapse.weight.grad, out2=y2)

    cuba_p = dict(threshold=1.25, current_decay=0.25, voltage_decay=0.03, requires_grad=True)
    for fam, params, name in ((slayer.block.cuba, cuba_p, 'block_cuba_kwta'), (slayer.block.alif, alif_p, 'block_alif_kwta')):
        torch.manual_seed(9)
        kw = fam.KWTA(dict(params), 10, 16, 3, self_excitation=0.4, weight_scale=4, delay_shift=False)  # with the
        # step delay the reference cannot be differentiated (in-place write into a custom function's output)
        xk = (rand(3, 10, 28) < 0.4).float()
        xin = xk.clone().requires_grad_(True)
        y1 = kw(xin)
        g_k = randn(*y1.shape)
        (y1 * g_k).sum().backward()
        with torch.no_grad():
            y2 = kw(xk)
        save(name, x=xk, weight=kw.synapse.weight.data, out1=y1, grad_out=g_k, grad_x=xin.grad,
             grad_weight=kw.synapse.weight.grad, grad_self_excitation=kw.self_excitation.grad, out2=y2)
        print(name, 'spike counts:', int(y1.sum()), int(y2.sum()))

    # shared parameters: per-channel ones on NCHWT input fail to broadcast on the reference's CPU path
    rf_p = dict(threshold=0.5, period=7, decay=0.1, requires_grad=True)
    adrf_p = dict(threshold=0.5, threshold_step=0.25, period=7, decay=0.1, threshold_decay=0.1,
                  refractory_decay=0.1, requires_grad=True)
    for fam, params, name in ((slayer.block.rf, rf_p, 'network_rf'), (slayer.block.adrf, adrf_p, 'network_adrf')):
        torch.manual_seed(10)
        net = [fam.Conv(dict(params), 2, 4, 3, padding=1, weight_scale=3), fam.Pool(dict(params), 2, weight_scale=2),
               fam.Flatten(), fam.Dense(dict(params), 4 * 3 * 3, 10, weight_scale=4, delay=True), fam.Average(5)]
        xn = (rand(2, 2, 6, 6, 40) < 0.3).float()
        xin = xn.clone().requires_grad_(True)
        acts, y = {}, xin
        for i, layer in enumerate(net):
            y = layer(y)
            acts[f'act{i}'] = y
        g_n = randn(*y.shape)
        (y * g_n).sum().backward()
        arrays = dict(x=xn, grad_out=g_n, grad_x=xin.grad, delay=net[3].delay.delay.data, **acts)
        for i in (0, 1, 3):
            for part in ('real', 'imag'):
                syn = getattr(net[i].synapse, part)
                arrays[f'weight{i}_{part}'] = syn.weight.data
                if syn.weight.grad is not None:
                    arrays[f'grad_weight{i}_{part}'] = syn.weight.grad
            for pname in ('sin_decay', 'cos_decay'):
                arrays[f'{pname}{i}'] = getattr(net[i].neuron, pname).data
        save(name, **arrays)
        print(name, 'spike counts per layer:', [int((acts[f'act{i}'] != 0).sum()) for i in range(4)])

    torch.manual_seed(11)
    inp = slayer.block.cuba.Input(dict(cuba_p), weight=1.5, bias=0.2)
    xi = randn(2, 7, 25, mean=0.5)
    xin = xi.clone().requires_grad_(True)
    yi = inp(xin)
    g_i = randn(*yi.shape)
    (yi * g_i).sum().backward()
    save('block_cuba_input', x=xi, out=yi, grad_out=g_i, grad_x=xin.grad, grad_weight=inp.weight.grad,
         grad_bias=inp.bias.grad)
    torch.manual_seed(12)
    sd_p = dict(threshold=0.1, activation=relu, tau_grad=0.5, scale_grad=1.0, requires_grad=False)
    outb = slayer.block.sigma_delta.Output(dict(sd_p), 9, 4, weight_scale=3)
    xo = (rand(2, 9, 20) < 0.3).float() * torch.round(rand(2, 9, 20) * 8) / 16
    with torch.no_grad():
        yo = outb(xo)
    save('block_sdnn_output', x=xo, weight=outb.synapse.weight.data, out=yo)

    total = 0
    for name, arrays in cases.items():
        path = os.path.join(out_dir, name + '.npz')
        np.savez_compressed(path, **arrays)
        total += os.path.getsize(path)
    print(f'wrote {len(cases)} cases, {total / 1024:.0f} KiB, to {out_dir}')


if __name__ == '__main__':
    main()
